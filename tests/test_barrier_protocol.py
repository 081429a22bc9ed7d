"""A model of the accumulator ring of the many-rows indexer (`glm_tpu_b200/csrc/indexer_rows_tcgen05.cu`) under every interleaving a
random scheduler finds: issuing threads fill TMEM accumulators, two epilogue groups drain them, and the only synchronisation is mbarrier
parity waits.  A parity wait tells the current phase from the previous one and nothing else, so two agents that share a barrier and may
drift a lap apart can pass a wait early.  The model shows that the layout in use (accumulator b owned by issuing thread b and by epilogue
group b & 1) is safe, and that a shared ring of five accumulators, the first design, is not.

No GPU is involved: this is the host-side stand-in for a race detector on the kernel's protocol.
"""

import random

import pytest


class Barrier:
    """mbarrier: `count` arrivals complete a phase; `passed(parity)` is what try_wait.parity reports."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase + 1

    def passed(self, parity):
        return (self.phase & 1) != parity  # true when the phase of that parity is not the one in progress


class Violation(Exception):
    pass


def run(tiles, issuers, buffers, rng, bias=None):
    """One random schedule.  Returns when every tile went through; raises Violation on an overwritten or misread accumulator."""
    full = [Barrier(1) for _ in range(buffers)]
    empty = [Barrier(1) for _ in range(buffers)]
    content = [None] * buffers  # which tile's accumulator a buffer holds

    def issuer(me):
        for n in range(tiles):
            if n % issuers != me:
                continue
            b, lap = n % buffers, n // buffers
            if lap > 0:
                yield lambda b=b, lap=lap: empty[b].passed((lap - 1) & 1)
            if content[b] is not None:
                raise Violation(f"tile {n} overwrites the live accumulator of tile {content[b]} in buffer {b}")
            content[b] = n
            yield  # the MMAs run
            full[b].arrive()
            yield

    def epilogue(group):
        for n in range(tiles):
            if n & 1 != group:
                continue
            b, lap = n % buffers, n // buffers
            yield lambda b=b, lap=lap: full[b].passed(lap & 1)
            if content[b] != n:
                raise Violation(f"the epilogue of tile {n} reads buffer {b} holding {content[b]}")
            content[b] = None
            yield  # the accumulator is in registers
            empty[b].arrive()
            yield

    agents = [issuer(i) for i in range(issuers)] + [epilogue(g) for g in range(2)]
    weights = bias or [1.0] * len(agents)
    waiting = {i: None for i in range(len(agents))}  # the wait an agent sits in (a predicate), None when it can simply run
    steps = 0
    while waiting:
        runnable = [i for i, wait in waiting.items() if wait is None or wait()]
        if not runnable:
            raise Violation("no agent can proceed: the barriers are out of step")
        k = rng.choices(runnable, weights=[weights[i] for i in runnable])[0]
        try:
            waiting[k] = next(agents[k])
        except StopIteration:
            del waiting[k]
        steps += 1
    return steps


@pytest.mark.parametrize("issuers,buffers", [(4, 4), (2, 2), (1, 5), (1, 4)])
def test_owned_accumulators_are_safe_under_random_schedules(issuers, buffers):
    """One issuing thread per accumulator (or a single issuing thread with any ring): no schedule breaks it, slow agents included."""
    rng = random.Random(7)
    for trial in range(300):
        bias = [rng.choice([0.02, 1.0, 5.0]) for _ in range(issuers + 2)]  # some agents almost never get a turn
        run(60, issuers, buffers, rng, bias)


def test_a_shared_ring_of_five_breaks_when_an_issuing_thread_lags():
    """Four issuing threads over five accumulators: thread n % 4 and buffer n % 5 drift apart, and a lagging thread lets another one
    pass its parity wait a lap early."""
    rng = random.Random(11)
    failures = 0
    for trial in range(300):
        bias = [1.0] * 6
        bias[rng.randrange(4)] = 0.02  # one issuing thread is slow
        try:
            run(60, 4, 5, rng, bias)
        except Violation:
            failures += 1
    assert failures > 0


# ------------------------------------------------------------------------------------------------------------------------------------
# The in-kernel all-reduce (`glm_tpu_b200/csrc/peer.cuh`, cta_allreduce_f32): every rank stores its partial into every peer's inbox of
# the channel, raises a sequence-numbered flag there, waits for all flags of this round and sums the inbox.  There is no second
# handshake: what keeps a fast rank from overwriting an inbox that a slow rank has not read yet is the rule that two consecutive
# all-reduces never use the same channel (`runner/admission.py:check_collective_plan`).  The model shows both halves of that statement.
def run_allreduces(world, channels, rng, bias):
    inbox = [[[None] * world for _ in range(2)] for _ in range(world)]   # [receiver][channel][source] = (round, value)
    flag = [[[0] * world for _ in range(2)] for _ in range(world)]       # [receiver][channel][source] = round number
    results = [[] for _ in range(world)]

    def rank(me):
        rounds = [0, 0]
        for step, ch in enumerate(channels):
            rounds[ch] += 1
            e = rounds[ch]
            for p in range(world):
                if p != me:
                    inbox[p][ch][me] = (step, 100 * step + me)
                    yield
                    flag[p][ch][me] = e
                    yield
            for p in range(world):
                if p != me:
                    yield lambda p=p, ch=ch, e=e: flag[me][ch][p] >= e
            total = 100 * step + me
            for p in range(world):
                if p != me:
                    got_step, value = inbox[me][ch][p]
                    if got_step != step:
                        raise Violation(f"rank {me} sums the partial of step {got_step} from rank {p} in step {step}")
                    total += value
                    yield
            results[me].append(total)

    agents = [rank(r) for r in range(world)]
    waiting = {i: None for i in range(world)}
    while waiting:
        runnable = [i for i, wait in waiting.items() if wait is None or wait()]
        if not runnable:
            raise Violation("no rank can proceed")
        k = rng.choices(runnable, weights=[bias[i] for i in runnable])[0]
        try:
            waiting[k] = next(agents[k])
        except StopIteration:
            del waiting[k]
    return results


@pytest.mark.parametrize("world", [2, 4, 8])
def test_alternating_channels_keep_the_one_handshake_all_reduce_safe(world):
    rng = random.Random(world)
    channels = [0, 1] * 6  # attention, MLP, attention, MLP, ...
    for trial in range(100):
        bias = [rng.choice([0.02, 1.0, 5.0]) for _ in range(world)]
        results = run_allreduces(world, channels, rng, bias)
        want = [sum(100 * step + r for r in range(world)) for step in range(len(channels))]
        assert all(r == want for r in results)


def test_reusing_a_channel_back_to_back_lets_a_fast_rank_overwrite_an_unread_inbox():
    rng = random.Random(3)
    failures = 0
    for trial in range(200):
        bias = [1.0] * 4
        bias[rng.randrange(4)] = 0.02
        try:
            run_allreduces(4, [0, 0, 0, 0], rng, bias)
        except Violation:
            failures += 1
    assert failures > 0


# ------------------------------------------------------------------------------------------------------------------------------------
# The same all-reduce with (value, sequence number) PAIRS (`GLMB_AR_PAIRS`, the protocol in use): there is no flag and no fence; every
# value is one aligned 8-byte store that lands whole, in any order relative to the other values, and the reader polls each word until
# its sequence number is this round's.  The model lets every word of a slice arrive on its own (a scheduler step per store) and lets a
# reader start summing words while others are still on their way.  Safe with alternating channels, for the same reason as above; a
# reused channel lets a fast rank overwrite a word a slow rank has not read yet, which the reader then takes for... nothing: it keeps
# polling for a round number that has already been overwritten by a later one, so the fault shows as a wait that never ends (on the
# device: the bounded wait gives up and raises the status word), never as a wrong sum.
def run_pair_allreduces(world, channels, rng, bias, width=3):
    word = [[[[(0, None)] * width for _ in range(world)] for _ in range(2)] for _ in range(world)]  # [receiver][channel][source][i] = (round, value)
    results = [[] for _ in range(world)]

    def rank(me):
        rounds = [0, 0]
        for step, ch in enumerate(channels):
            rounds[ch] += 1
            e = rounds[ch]
            mine = [1000 * step + 10 * me + i for i in range(width)]
            order = [(p, i) for p in range(world) if p != me for i in range(width)]
            rng.shuffle(order)  # the stores of a slice reach the peers in no particular order
            for p, i in order:
                word[p][ch][me][i] = (e, mine[i])
                yield
            sums = list(mine)
            for i in range(width):
                for p in range(world):
                    if p == me:
                        continue
                    yield lambda p=p, ch=ch, i=i, e=e: word[me][ch][p][i][0] == e  # exactly this round: a later one means the word was lost
                    got_round, value = word[me][ch][p][i]
                    if got_round != e or value != 1000 * step + 10 * p + i:
                        raise Violation(f"rank {me} adds {value} (round {got_round}) from rank {p} in step {step}")
                    sums[i] += value
            results[me].append(sums)

    agents = [rank(r) for r in range(world)]
    waiting = {i: None for i in range(world)}
    while waiting:
        runnable = [i for i, wait in waiting.items() if wait is None or wait()]
        if not runnable:
            raise Violation("no rank can proceed")
        k = rng.choices(runnable, weights=[bias[i] for i in runnable])[0]
        try:
            waiting[k] = next(agents[k])
        except StopIteration:
            del waiting[k]
    return results


@pytest.mark.parametrize("world", [2, 4, 8])
def test_pair_all_reduce_is_safe_with_alternating_channels(world):
    rng = random.Random(10 + world)
    channels = [0, 1] * 5
    for trial in range(60):
        bias = [rng.choice([0.02, 1.0, 5.0]) for _ in range(world)]
        results = run_pair_allreduces(world, channels, rng, bias)
        want = [[sum(1000 * step + 10 * r + i for r in range(world)) for i in range(3)] for step in range(len(channels))]
        assert all(r == want for r in results)


def test_pair_all_reduce_on_a_reused_channel_loses_words_and_stalls_instead_of_summing_wrong():
    rng = random.Random(5)
    stalled = wrong = 0
    for trial in range(200):
        bias = [1.0] * 4
        bias[rng.randrange(4)] = 0.02
        try:
            run_pair_allreduces(4, [0, 0, 0, 0], rng, bias)
        except Violation as exc:
            if "no rank can proceed" in str(exc):
                stalled += 1
            else:
                wrong += 1
    assert stalled > 0 and wrong == 0


# ------------------------------------------------------------------------------------------------------------------------------------
# Signals (`grid_signal_peers` / `cta_wait_signal`): a producer kernel stores its data into ONE buffer on every peer and raises the
# round's number; the consumer kernel of each rank waits for every rank's number and reads.  Nothing tells the producer that the peers
# have read: what protects the buffer is that an all-reduce, which no rank leaves before every rank has entered it, separates two rounds
# of the same signal.  The model shows the protected sequence to be safe and the unprotected one to break.
def run_signal_rounds(world, rounds, separated, rng, bias):
    data = [[None] * world for _ in range(world)]   # [receiver][source]: the round whose data sits in the buffer
    flag = [[0] * world for _ in range(world)]      # [receiver][source]
    entered = [0] * world                            # all-reduces a rank has entered

    def rank(me):
        for e in range(1, rounds + 1):
            for p in range(world):                   # producer kernel
                data[p][me] = e
                yield
                flag[p][me] = e
                yield
            for p in range(world):                   # consumer kernel
                yield lambda p=p, e=e: flag[me][p] >= e
            for p in range(world):
                if data[me][p] != e:
                    raise Violation(f"rank {me} reads round {data[me][p]} from rank {p} in round {e}")
                yield
            if separated:                            # the all-reduce that ends the layer: nobody leaves before everybody entered
                entered[me] = e
                for p in range(world):
                    yield lambda p=p, e=e: entered[p] >= e

    agents = [rank(r) for r in range(world)]
    waiting = {i: None for i in range(world)}
    while waiting:
        runnable = [i for i, wait in waiting.items() if wait is None or wait()]
        if not runnable:
            raise Violation("no rank can proceed")
        k = rng.choices(runnable, weights=[bias[i] for i in runnable])[0]
        try:
            waiting[k] = next(agents[k])
        except StopIteration:
            del waiting[k]


def test_signal_rounds_are_safe_when_an_all_reduce_separates_them_and_break_when_none_does():
    rng = random.Random(5)
    broken = 0
    for trial in range(150):
        bias = [1.0] * 4
        bias[rng.randrange(4)] = 0.02
        run_signal_rounds(4, 8, True, rng, bias)
        try:
            run_signal_rounds(4, 8, False, rng, bias)
        except Violation:
            broken += 1
    assert broken > 0
