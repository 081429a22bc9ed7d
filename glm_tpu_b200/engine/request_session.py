"""Request sessions: the per-token loop of one chat (``RequestSession``) or of several concurrent chats that share
the batched decode program (``BatchedSession``), with the all-rank vote schedule.

Every rank (one process per GPU) runs the same session.  A step is

    feed (the host hands the device the token(s) it committed last: a few bytes from pinned memory)
    ->  decode on the device  ->  read the produced token(s) and the device status word
    ->  vote 1 "validity" (all ranks: status clean, token inside the vocabulary, deadline not passed)
    ->  commit (the token becomes part of the session state; finish reasons are decided here)
    ->  deliver (rank 0 appends the TokenEvent line to the sink and flushes)
    ->  vote 2 "delivery" (all ranks learn whether the sink accepted it)

A false or failed vote raises ``EngineFailure`` on every rank at the same schedule point, so no rank is left inside a
collective its peers never enter.  State is committed before delivery, so an ambiguous sink failure can never emit a
token twice.  There is no retry and no recovery: the engine that owns a failed session refuses all later requests.

Parity: reference ``glm_tpu/engine/request_session.py:64-379`` (session/commit/delivery/vote order, lanes frozen at
EOS or length), ``glm_tpu/distributed/parallel_state.py:81-93`` (the host vote).
"""

from __future__ import annotations

import hashlib
import struct
import time
from dataclasses import dataclass, field
from typing import Callable, Protocol

from glm_tpu_b200.engine.outputs import TokenEvent
from glm_tpu_b200.exceptions import EngineFailure


class Vote(Protocol):
    def all(self, ok: bool, point: str) -> bool: ...


class LocalVote:
    """Single process: the vote is the local value (``log`` keeps the schedule for tests and records)."""

    def __init__(self):
        self.log: list[tuple[str, bool]] = []

    def all(self, ok: bool, point: str) -> bool:
        self.log.append((point, bool(ok)))
        return bool(ok)


class ProcessGroupVote:
    """All-rank AND over a CPU (gloo) process group: one int32 per rank and vote."""

    def __init__(self, group):
        self.group = group

    def all(self, ok: bool, point: str) -> bool:
        import torch
        import torch.distributed as dist

        flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        return bool(flag.item())


class SharedMemoryVote:
    """All-rank AND for ranks that share one machine: every rank publishes (round number, verdict, vote point) in its own
    cache line of a small memory-mapped file and spins until every rank has reached the round.  A vote costs a few
    microseconds instead of the ~100 us of a TCP all-reduce, which matters because the engine votes twice per token.

    Rounds alternate between two verdict slots per rank, so a rank that is one vote ahead never overwrites what a slower
    rank is still reading; no rank can be two ahead, because leaving round r needs every rank to have entered it.  Ranks that
    vote at different points (a diverged schedule) and a rank that never arrives within ``timeout`` seconds raise
    ``EngineFailure`` on everybody who waits -- the vote never hangs.

    Parity: reference ``glm_tpu/distributed/health.py`` (all-host agreement before anything irreversible), here without a
    network between the ranks.
    """

    LINE = 64  # bytes per rank: int64 round | int64 verdict[2] | int64 point[2]

    def __init__(self, path, rank: int, world: int, *, timeout: float = 600.0, create: bool = False):
        import mmap
        import os

        import numpy as np

        self.rank, self.world, self.timeout = rank, world, timeout
        size = self.LINE * world
        if create:
            fd = os.open(path, os.O_RDWR | os.O_CREAT | os.O_TRUNC, 0o600)
            os.ftruncate(fd, size)
        else:
            fd = os.open(path, os.O_RDWR)
            if os.fstat(fd).st_size != size:
                os.close(fd)
                raise EngineFailure("the vote file was made for another number of ranks")
        try:
            self._map = mmap.mmap(fd, size)
        finally:
            os.close(fd)
        self._words = np.frombuffer(self._map, dtype=np.int64).reshape(world, self.LINE // 8)
        self.round = 0
        self.log: list[tuple[str, bool]] = []

    @staticmethod
    def _point_code(point: str) -> int:
        import zlib

        return zlib.crc32(point.encode()) + 1

    def all(self, ok: bool, point: str) -> bool:
        import time

        self.round += 1
        r, slot, words = self.round, self.round & 1, self._words
        code = self._point_code(point)
        words[self.rank, 1 + slot] = 1 if ok else 0
        words[self.rank, 3 + slot] = code
        words[self.rank, 0] = r  # published last: the verdict and the point are in place when the round number shows
        started = time.monotonic()
        spins = 0
        while True:
            rounds = words[:, 0]
            if int(rounds.min()) >= r:
                break
            spins += 1
            if spins & 0x3FF == 0:
                # per-token votes meet within microseconds and never get here twice; a vote that waits for a peer's long phase
                # (a checkpoint load) backs off to a sleep instead of burning a core
                waited = time.monotonic() - started
                if waited > self.timeout:
                    behind = [i for i in range(self.world) if int(rounds[i]) < r]
                    raise EngineFailure(f"rank {self.rank} waited {self.timeout:.0f} s at vote {point!r} (round {r}) for ranks {behind}")
                time.sleep(0 if waited < 0.002 else 0.0005 if waited < 1.0 else 0.01)
        if any(int(words[i, 3 + slot]) != code for i in range(self.world)):
            raise EngineFailure(f"the ranks vote at different points in round {r} (this rank: {point!r})")
        result = all(int(words[i, 1 + slot]) == 1 for i in range(self.world))
        self.log.append((point, result))
        return result

    def close(self) -> None:
        self._words = None
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass


def fleet_vote(group, rank: int, world: int, directory, *, name: str = "vote.shm", timeout: float = 3600.0):
    """The vote for ``world`` ranks of one machine that already share a CPU process group: rank 0 creates the vote file in
    ``directory``, a barrier publishes it, everybody maps it.  ``GLM_B200_VOTE=gloo`` keeps the votes on the process group."""
    import os
    from pathlib import Path

    import torch.distributed as dist

    if os.environ.get("GLM_B200_VOTE", "shm") == "gloo":
        return ProcessGroupVote(group)
    path = Path(directory) / name
    vote = SharedMemoryVote(path, rank, world, timeout=timeout, create=True) if rank == 0 else None
    dist.barrier(group=group)
    if vote is None:
        vote = SharedMemoryVote(path, rank, world, timeout=timeout)
    dist.barrier(group=group)  # nobody votes before everybody has mapped the file
    return vote


@dataclass
class LaneState:
    request: dict
    lane: int
    tokens: list = field(default_factory=list)
    finish_reason: str | None = None
    step_seconds: list = field(default_factory=list)

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def token_digest(self) -> str:
        return hashlib.sha256(struct.pack(f"<{len(self.tokens)}i", *self.tokens)).hexdigest()


def _finish_reason(request: dict, tokens: list) -> str | None:
    if tokens[-1] in request["eos_ids"]:
        return "eos"
    if len(tokens) >= request["max_new_tokens"]:
        return "length"
    return None


class _SessionBase:
    def __init__(self, runner, vote: Vote, sink: Callable[[TokenEvent], None] | None, *, deadline: float | None = None,
                 clock: Callable[[], float] = time.perf_counter):
        self.runner, self.vote, self.sink = runner, vote, sink
        self.deadline, self.clock = deadline, clock
        self.failed = False

    def _vote(self, ok: bool, point: str) -> None:
        agreed = self.vote.all(ok, point)
        if not agreed:
            self.failed = True
            raise EngineFailure(f"fleet vote failed at {point}")

    def _deliver(self, events: list[TokenEvent]) -> bool:
        if self.sink is None:
            return True
        try:
            for ev in events:
                self.sink(ev)
            return True
        except Exception:  # noqa: BLE001 - any sink failure is reported through the vote, never retried
            return False

    def _valid_token(self, token: int, request: dict) -> bool:
        return isinstance(token, int) and 0 <= token < request["vocab_size"]

    def _in_time(self) -> bool:
        return self.deadline is None or self.clock() < self.deadline

    def _feed(self, tokens: dict) -> None:
        """Hand the device the tokens the fleet committed (``lane -> token``): what the next step consumes is what the votes
        agreed on, not whatever a rank's device happened to keep.  Runners without device-side token registers ignore it."""
        feed = getattr(self.runner, "feed_tokens", None)
        if feed is not None:
            feed(tokens)


class RequestSession(_SessionBase):
    """One chat on one lane."""

    def __init__(self, runner, request: dict, vote: Vote, sink=None, *, lane: int = 0, **kw):
        super().__init__(runner, vote, sink, **kw)
        self.state = LaneState(request, lane)

    @property
    def finished(self) -> bool:
        return self.state.finished

    def accept_prefill(self, token: int, status: int = 0) -> None:
        """The prefill produced the first token: validate, commit, deliver (index 0)."""
        st = self.state
        self._vote(status == 0 and self._valid_token(token, st.request) and self._in_time(), "prefill_validity")
        st.tokens.append(token)
        st.finish_reason = _finish_reason(st.request, st.tokens)
        delivered = self._deliver([TokenEvent(st.request["request_id"], 0, token, st.finish_reason)])
        self._vote(delivered, "prefill_delivery")
        if st.finished:
            self.runner.deactivate(st.lane)

    def step(self) -> None:
        st = self.state
        if st.finished:
            raise EngineFailure("step on a finished session")
        t0 = self.clock()
        self._feed({st.lane: st.tokens[-1]})
        self.runner.decode_step()
        token = self.runner.read_last_tokens()[st.lane]
        status = self.runner.read_status()
        st.step_seconds.append(self.clock() - t0)
        self._vote(status == 0 and self._valid_token(token, st.request) and self._in_time(), "validity")
        st.tokens.append(token)
        st.finish_reason = _finish_reason(st.request, st.tokens)
        delivered = self._deliver([TokenEvent(st.request["request_id"], len(st.tokens) - 1, token, st.finish_reason)])
        self._vote(delivered, "delivery")
        if st.finished:
            self.runner.deactivate(st.lane)


class BatchedSession(_SessionBase):
    """Several chats, one lane each, advanced together by the batched decode program."""

    def __init__(self, runner, requests: list[dict], vote: Vote, sink=None, **kw):
        super().__init__(runner, vote, sink, **kw)
        self.lanes = [LaneState(req, lane) for lane, req in enumerate(requests)]
        self.round = 0

    @property
    def finished(self) -> bool:
        return all(lane.finished for lane in self.lanes)

    def accept_prefill(self, lane: int, token: int, status: int = 0) -> None:
        st = self.lanes[lane]
        self._vote(status == 0 and self._valid_token(token, st.request) and self._in_time(), "prefill_validity")
        st.tokens.append(token)
        st.finish_reason = _finish_reason(st.request, st.tokens)
        delivered = self._deliver([TokenEvent(st.request["request_id"], 0, token, st.finish_reason, batch_round=0)])
        self._vote(delivered, "prefill_delivery")
        if st.finished:
            self.runner.deactivate(lane)

    def step(self) -> None:
        active = [lane for lane in self.lanes if not lane.finished]
        if not active:
            raise EngineFailure("step on a finished batch")
        t0 = self.clock()
        self._feed({st.lane: st.tokens[-1] for st in active})
        self.runner.decode_step()
        tokens = self.runner.read_last_tokens()
        status = self.runner.read_status()
        elapsed = self.clock() - t0
        self.round += 1
        ok = status == 0 and self._in_time() and all(self._valid_token(tokens[st.lane], st.request) for st in active)
        self._vote(ok, "validity")
        events = []
        for st in active:
            st.tokens.append(tokens[st.lane])
            st.step_seconds.append(elapsed)
            st.finish_reason = _finish_reason(st.request, st.tokens)
            events.append(TokenEvent(st.request["request_id"], len(st.tokens) - 1, tokens[st.lane], st.finish_reason, batch_round=self.round))
        delivered = self._deliver(events)
        self._vote(delivered, "delivery")
        for st in active:
            if st.finished:
                self.runner.deactivate(st.lane)  # a finished lane is frozen: no cache write, no position advance
