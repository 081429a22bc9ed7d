"""CPU stand-ins for the device side, so the engine, the workers and the servers can be tested without a GPU.

``FakeRunner`` has the interface of ``GpuModelRunner`` that the engine uses.  Its "model" is a deterministic function
of the prompt and the tokens so far; a ``Script`` injects failures (a dirty status word, an out-of-vocabulary token,
rank-dependent tokens) at chosen steps.  ``ThreadFleet`` runs several ranks as threads in lock-step and turns a rank
stuck in a vote its peers never enter into ``StrandedVote`` instead of a hang.
"""

from __future__ import annotations

import hashlib
import threading
from dataclasses import dataclass, field
from types import SimpleNamespace


@dataclass
class Script:
    bad_status_at: int | None = None  # decode step index whose status word is dirty
    bad_token_at: int | None = None  # decode step index that yields a token outside the vocabulary
    eos_at: dict = field(default_factory=dict)  # lane -> number of generated tokens after which EOS comes out
    rank_token_skew_at: int | None = None  # decode step at which rank != 0 produces another token
    fail_prefill: bool = False


class FakeRunner:
    def __init__(self, *, vocab=1000, eos=(997, 998, 999), capacity=64, lanes=1, rank=0, script: Script | None = None):
        self.vocab, self.eos, self.rank = vocab, tuple(eos), rank
        self.lanes = lanes
        self.cache = SimpleNamespace(context_capacity=capacity)
        self.g = SimpleNamespace(vocab_size=vocab, eos_ids=self.eos)
        self.script = script or Script()
        self.log: list = []
        self.history = [[] for _ in range(lanes)]
        self.prompts = [[] for _ in range(lanes)]
        self.active = [False] * lanes
        self.steps_issued = 0
        self._last = [-1] * lanes
        self._status = 0

    def _next(self, lane: int) -> int:
        n = len(self.history[lane])
        if lane in self.script.eos_at and n >= self.script.eos_at[lane]:
            return self.eos[0]
        h = hashlib.sha256(repr((self.prompts[lane], self.history[lane])).encode()).digest()
        return int.from_bytes(h[:4], "little") % (self.vocab - len(self.eos))

    def prefill(self, lane: int, ids) -> int:
        self.log.append(("prefill", lane, len(ids)))
        if self.script.fail_prefill:
            self._status = 4
        self.prompts[lane] = list(ids)
        self.history[lane] = []
        tok = self._next(lane)
        self.history[lane].append(tok)
        self.active[lane] = True
        return tok

    def build_decode_program(self):
        self.log.append(("build",))

    def decode_step(self) -> None:
        step = self.steps_issued
        self.log.append(("decode", step, tuple(self.active)))
        for lane in range(self.lanes):
            if not self.active[lane]:
                self._last[lane] = -1
                continue
            tok = self._next(lane)
            if self.script.bad_token_at == step:
                tok = self.vocab + 5
            if self.script.rank_token_skew_at == step and self.rank != 0:
                tok = (tok + 1) % (self.vocab - len(self.eos))
            self.history[lane].append(tok)
            self._last[lane] = tok
        if self.script.bad_status_at == step:
            self._status = 1
        self.steps_issued += 1

    def read_last_tokens(self):
        return list(self._last)

    def read_status(self) -> int:
        s, self._status = self._status, 0
        return s

    def deactivate(self, lane: int) -> None:
        self.log.append(("deactivate", lane))
        self.active[lane] = False

    def memory_stats(self):
        return {"allocated": 0}


class StrandedVote(RuntimeError):
    pass


class ThreadFleet:
    """``world`` ranks as threads; ``vote(rank)`` gives each rank an all-rank AND with a rendezvous."""

    def __init__(self, world: int, timeout: float = 5.0):
        self.world, self.timeout = world, timeout
        self._cond = threading.Condition()
        self._round: dict = {}
        self._done: dict = {}
        self.log: list = []

    def vote(self, rank: int):
        fleet = self
        counter = {"n": 0}

        class _Vote:
            def all(self, ok: bool, point: str) -> bool:
                key = (counter["n"], point)
                counter["n"] += 1
                with fleet._cond:
                    votes = fleet._round.setdefault(key, {})
                    votes[rank] = bool(ok)
                    fleet._cond.notify_all()
                    if not fleet._cond.wait_for(lambda: len(fleet._round[key]) == fleet.world, timeout=fleet.timeout):
                        raise StrandedVote(f"rank {rank} is alone at vote {key}")
                    result = all(fleet._round[key].values())
                    if rank == 0:
                        fleet.log.append((point, result))
                    return result

        return _Vote()

    def run(self, fn):
        """Run ``fn(rank)`` on every rank; returns the list of results or exceptions."""
        out = [None] * self.world

        def body(r):
            try:
                out[r] = fn(r)
            except BaseException as exc:  # noqa: BLE001
                out[r] = exc

        threads = [threading.Thread(target=body, args=(r,)) for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(self.timeout * 4)
        return out
