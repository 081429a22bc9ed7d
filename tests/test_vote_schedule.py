"""The vote schedule as literal logs: for every way a request can fail, the exact sequence of (vote point, outcome) up to the
failing vote, on one rank and on two ranks where only one of them sees the failure.  A vote that moves, doubles or disappears
changes one of these lists.  (CPU, fake device: `tests/fakes.py`.)"""

import pytest

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.engine.llm_engine import LLMEngine
from glm_tpu_b200.engine.request_session import LocalVote
from glm_tpu_b200.exceptions import EngineFailure, PlanValidationError
from tests.fakes import FakeRunner, Script, ThreadFleet

PROFILE = rq.RequestProfile(vocab_size=1000, eos_ids=(997, 998, 999), capacities=(64, 128), prompt_limits={64: 64, 128: 128},
                            concurrent_capacity=64, max_new=100)
OK, BAD = True, False
HEAD = [("admission", OK), ("prefill_validity", OK), ("prefill_delivery", OK)]


def make(ids=(1, 2, 3), rid="r1", n=5):
    return rq.from_token_ids(list(ids), request_id=rid, max_new_tokens=n, context_capacity=64, profile=PROFILE)


def step(n):
    return [("validity", OK), ("delivery", OK)] * n


def run_one(script=None, sink=None, n=5, runner=None, **engine_kw):
    vote = LocalVote()
    engine = LLMEngine(runner or FakeRunner(script=script), vote=vote, profile=PROFILE, **engine_kw)
    try:
        engine.generate(make(n=n), sink)
        failed = None
    except Exception as exc:  # noqa: BLE001
        failed = exc
    return vote.log, failed, engine


# ------------------------------------------------------------------------------------------------ one rank
def test_clean_request():
    log, failed, engine = run_one(n=4)
    assert failed is None and log == HEAD + step(3) and not engine.poisoned


def test_eos_ends_the_schedule_after_a_complete_step():
    log, failed, _ = run_one(Script(eos_at={0: 2}), n=10)
    assert failed is None and log == HEAD + step(2)  # the EOS token is validated and delivered like any other


@pytest.mark.parametrize("at", [0, 1, 3])
def test_dirty_status_fails_the_validity_vote_of_that_step(at):
    log, failed, engine = run_one(Script(bad_status_at=at), n=6)
    assert isinstance(failed, EngineFailure) and engine.poisoned
    assert log == HEAD + step(at) + [("validity", BAD)]  # nothing is delivered, nothing is voted after a failed validity


@pytest.mark.parametrize("at", [0, 2])
def test_token_outside_the_vocabulary_fails_validity(at):
    log, failed, _ = run_one(Script(bad_token_at=at), n=6)
    assert isinstance(failed, EngineFailure) and log == HEAD + step(at) + [("validity", BAD)]


def test_dirty_status_after_prefill_fails_the_first_vote_after_admission():
    log, failed, engine = run_one(Script(fail_prefill=True), n=6)
    assert isinstance(failed, EngineFailure) and engine.poisoned
    assert log == [("admission", OK), ("prefill_validity", BAD)]


@pytest.mark.parametrize("index", [0, 1, 3])
def test_failed_delivery_fails_the_delivery_vote_of_that_token(index):
    def sink(event):
        if event.index == index:
            raise OSError("disk full")

    log, failed, _ = run_one(sink=sink, n=6)
    assert isinstance(failed, EngineFailure)
    if index == 0:  # the first token comes out of the prefill
        assert log == [("admission", OK), ("prefill_validity", OK), ("prefill_delivery", BAD)]
    else:
        assert log == HEAD + step(index - 1) + [("validity", OK), ("delivery", BAD)]


def test_refused_admission_is_the_only_vote():
    class Full(FakeRunner):
        def admit_request(self):
            raise PlanValidationError("memory admission refused: needs 190.00 GiB, limit 170.00 GiB")

    log, failed, engine = run_one(runner=Full(), n=3)
    assert isinstance(failed, PlanValidationError) and log == [("admission", BAD)] and engine.poisoned


def test_deadline_turns_a_clean_step_into_a_failed_validity_vote():
    ticks = iter(range(1000))
    vote = LocalVote()
    engine = LLMEngine(FakeRunner(), vote=vote, profile=PROFILE, clock=lambda: float(next(ticks)))
    with pytest.raises(EngineFailure):
        engine.generate(make(n=50), deadline=12.0)
    points = [p for p, _ in vote.log]
    assert vote.log[-1][1] is BAD and all(ok for _, ok in vote.log[:-1])
    assert points[:3] == ["admission", "prefill_validity", "prefill_delivery"] and set(points[3:]) <= {"validity", "delivery"}


def test_a_poisoned_engine_votes_nothing():
    vote = LocalVote()
    engine = LLMEngine(FakeRunner(script=Script(bad_status_at=0)), vote=vote, profile=PROFILE)
    with pytest.raises(EngineFailure):
        engine.generate(make(n=3))
    before = list(vote.log)
    with pytest.raises(EngineFailure):
        engine.generate(make(n=3, rid="r2"))
    assert vote.log == before


# ------------------------------------------------------------------------------------------------ four chats on one rank
def test_concurrent_batch_votes_once_per_round_for_all_lanes():
    vote = LocalVote()
    engine = LLMEngine(FakeRunner(lanes=4, script=Script(eos_at={1: 2})), vote=vote, profile=PROFILE)
    requests = [make(rid=f"c{i}", ids=(i + 1, 2, 3), n=4) for i in range(3)]
    engine.generate_concurrent(rq.batch(requests, concurrent=True, profile=PROFILE))
    # one admission; a (validity, delivery) pair per prefilled chat; then one pair per decode ROUND (not per lane):
    # three rounds, the second chat leaving after its second token
    assert vote.log == [("admission", OK)] + [("prefill_validity", OK), ("prefill_delivery", OK)] * 3 + step(3)


def test_concurrent_batch_one_bad_lane_fails_the_round_for_all():
    vote = LocalVote()
    engine = LLMEngine(FakeRunner(lanes=4, script=Script(bad_token_at=1)), vote=vote, profile=PROFILE)
    requests = [make(rid=f"c{i}", ids=(i + 1, 2, 3), n=5) for i in range(2)]
    with pytest.raises(EngineFailure):
        engine.generate_concurrent(rq.batch(requests, concurrent=True, profile=PROFILE))
    assert vote.log == [("admission", OK)] + [("prefill_validity", OK), ("prefill_delivery", OK)] * 2 + step(1) + [("validity", BAD)]
    assert engine.poisoned


# ------------------------------------------------------------------------------------------------ two ranks
def two_ranks(scripts, n=5, sinks=(None, None)):
    fleet = ThreadFleet(2)

    def body(rank):
        engine = LLMEngine(FakeRunner(rank=rank, script=scripts[rank]), vote=fleet.vote(rank), profile=PROFILE)
        return engine.generate(make(n=n), sinks[rank])

    return fleet, fleet.run(body)


@pytest.mark.parametrize("bad_rank", [0, 1])
def test_two_ranks_one_dirty_status_both_stop_at_the_same_vote(bad_rank):
    scripts = [Script(), Script()]
    scripts[bad_rank] = Script(bad_status_at=2)
    fleet, out = two_ranks(scripts, n=8)
    assert all(isinstance(o, EngineFailure) for o in out)
    assert fleet.log == HEAD + step(2) + [("validity", BAD)]  # the healthy rank voted yes and still stops here


def test_two_ranks_only_rank_zero_delivers_and_its_failure_stops_both():
    def broken(event):
        if event.index == 2:
            raise OSError("pipe closed")

    fleet, out = two_ranks([Script(), Script()], n=8, sinks=(broken, None))
    assert all(isinstance(o, EngineFailure) for o in out)
    assert fleet.log == HEAD + step(1) + [("validity", OK), ("delivery", BAD)]


def test_two_ranks_clean_run_has_the_single_rank_schedule():
    fleet, out = two_ranks([Script(), Script()], n=4)
    assert all(isinstance(o, dict) for o in out) and out[0]["token_sha256"] == out[1]["token_sha256"]
    assert fleet.log == HEAD + step(3)


# ------------------------------------------------------------------------------------------------ the shared-memory vote itself
def _shm_rank(path, rank, world, rounds, bad, divergent, out, timeout):
    from glm_tpu_b200.engine.request_session import SharedMemoryVote

    def point_of(i):
        return "delivery" if (rank, i) == divergent else ("validity", "delivery")[i & 1] if divergent is None else "validity"

    try:
        vote = SharedMemoryVote(path, rank, world, timeout=timeout)
        out.put((rank, [vote.all((rank, i) not in bad, point_of(i)) for i in range(rounds)]))
    except Exception as exc:  # noqa: BLE001
        out.put((rank, f"{type(exc).__name__}: {exc}"))


def _run_shm(tmp_path, world, rounds, bad=(), divergent=None, absent=(), timeout=10.0):
    import multiprocessing as mp

    from glm_tpu_b200.engine.request_session import SharedMemoryVote

    path = tmp_path / "vote.shm"
    SharedMemoryVote(path, 0, world, create=True).close()
    ctx = mp.get_context("spawn")  # no fork from a threaded test process
    out = ctx.Queue()
    procs = [ctx.Process(target=_shm_rank, args=(path, r, world, rounds, set(bad), divergent, out, timeout)) for r in range(world) if r not in absent]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(10)
    return results


def test_shared_memory_vote_is_an_all_rank_and(tmp_path):
    results = _run_shm(tmp_path, 4, 300, bad={(2, 17), (0, 150), (3, 150)})
    want = [i not in (17, 150) for i in range(300)]
    assert all(results[r] == want for r in range(4))  # every rank sees the same verdict in every round, one round apart at most


def test_shared_memory_vote_refuses_a_diverged_schedule(tmp_path):
    results = _run_shm(tmp_path, 2, 5, divergent=(1, 3))
    assert all(isinstance(results[r], str) and "different points" in results[r] for r in range(2))


def test_shared_memory_vote_times_out_on_a_missing_rank_instead_of_hanging(tmp_path):
    results = _run_shm(tmp_path, 3, 2, absent={2}, timeout=0.5)
    # (a slow starter may be listed beside the absent rank: the absent one is always last)
    assert all(isinstance(results[r], str) and "waited" in results[r] and results[r].rstrip().endswith("2]") for r in (0, 1))
