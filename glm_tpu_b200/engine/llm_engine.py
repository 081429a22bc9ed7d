"""``LLMEngine``: runs prepared requests on a model runner, one at a time or as a group of concurrent chats.

``generate(request)`` validates the request, starts from a fresh cache, prefills the prompt (the first token comes out
of the prefill), then drives a ``RequestSession`` token by token until EOS or the output budget, and returns the
per-request report.  ``generate_concurrent(batch)`` prefills each chat on its own lane and advances all of them with
the batched decode program; a lane that finishes is frozen while the others continue.

Failure model (no retries, no recovery): any failed vote, device status or exception marks the engine ``poisoned``;
a poisoned engine refuses every later request.  Each request ends with an output consensus: all ranks must hold the
same token digest.

Parity: reference ``glm_tpu/engine/llm_engine.py:22-244`` (generate / generate_concurrent, poison flag, deadline folded
into the votes, output consensus, report fields).
"""

from __future__ import annotations

import time
from typing import Callable

from glm_tpu_b200.engine import request as request_schema
from glm_tpu_b200.engine.outputs import TokenEvent
from glm_tpu_b200.engine.request_session import BatchedSession, LaneState, LocalVote, RequestSession, Vote
from glm_tpu_b200.exceptions import EngineFailure, RequestValidationError


class LLMEngine:
    def __init__(self, runner, *, vote: Vote | None = None, profile: request_schema.RequestProfile | None = None,
                 digest_consensus: Callable[[str], bool] | None = None, clock: Callable[[], float] = time.perf_counter):
        self.runner = runner
        self.vote = vote or LocalVote()
        self.profile = profile or request_schema.GLM53_PROFILE
        self.digest_consensus = digest_consensus  # str -> bool: do all ranks hold this digest?
        self.clock = clock
        self.poisoned = False
        self.requests_done = 0

    # ------------------------------------------------------------------ helpers
    def _guard(self) -> None:
        if self.poisoned:
            raise EngineFailure("this engine failed earlier and refuses further requests")

    def _admit(self) -> None:
        """Memory admission before every request (the runner's projection against the live device): refused on every rank
        together, so that no rank starts a prefill its peers will not join."""
        admit = getattr(self.runner, "admit_request", None)
        error = None
        if admit is not None:
            try:
                admit()
            except Exception as exc:  # noqa: BLE001
                error = exc
        if not self.vote.all(error is None, "admission"):
            raise error if error is not None else EngineFailure("a peer refused the request at memory admission")

    def _check_capacity(self, capacity: int, lanes: int) -> None:
        if capacity != self.runner.cache.context_capacity:
            raise RequestValidationError(f"the loaded model serves capacity {self.runner.cache.context_capacity}, not {capacity}")
        if lanes > self.runner.lanes:
            raise RequestValidationError(f"the loaded model has {self.runner.lanes} lanes, the batch needs {lanes}")

    def _report(self, st: LaneState, prefill_seconds: float, ttft: float, decode_wall: float) -> dict:
        prompt = len(st.request["prompt_ids"])
        timed = max(len(st.tokens) - 1, 0)
        return {
            "request_id": st.request["request_id"],
            "request_sha256": st.request["request_sha256"],
            "prompt_tokens": prompt,
            "emitted": len(st.tokens),
            "timed_decode_tokens": timed,
            "finish_reason": st.finish_reason,
            "stop_cause": request_schema.stop_cause(st.request, st.finish_reason),
            "prefill_seconds": prefill_seconds,
            "prefill_tokens_per_second": prompt / prefill_seconds if prefill_seconds > 0 else None,
            "decode_wall_seconds": decode_wall,
            "decode_tokens_per_second": timed / decode_wall if decode_wall > 0 and timed else None,
            "ttft_seconds": ttft,
            "token_sha256": st.token_digest(),
            "output_budget_tokens": st.request["max_new_tokens"],
            "sampling": "greedy",
            "speculative": False,
            "peak_memory": self.runner.memory_stats() if hasattr(self.runner, "memory_stats") else None,
        }

    def _consensus(self, st: LaneState) -> None:
        if self.digest_consensus is not None and not self.digest_consensus(st.token_digest()):
            raise EngineFailure("ranks disagree on the generated tokens")

    # ------------------------------------------------------------------ one request
    def generate(self, request: dict, sink: Callable[[TokenEvent], None] | None = None, *, deadline: float | None = None) -> dict:
        self._guard()
        request_schema.validate(request, self.profile)
        self._check_capacity(request["context_capacity"], 1)
        try:
            self._admit()
            t0 = self.clock()
            session = RequestSession(self.runner, request, self.vote, sink, lane=0, deadline=deadline, clock=self.clock)
            for lane in range(1, self.runner.lanes):  # a single chat on a multi-lane model: the other lanes stay frozen
                self.runner.deactivate(lane)
            first = self.runner.prefill(0, request["prompt_ids"])
            prefill_seconds = self.clock() - t0
            session.accept_prefill(first, self.runner.read_status())
            ttft = self.clock() - t0
            t1 = self.clock()
            while not session.finished:
                session.step()
            decode_wall = self.clock() - t1
            self._consensus(session.state)
            self.requests_done += 1
            return self._report(session.state, prefill_seconds, ttft, decode_wall)
        except Exception:
            self.poisoned = True
            raise

    # ------------------------------------------------------------------ concurrent chats
    def generate_concurrent(self, batch: dict, sink: Callable[[TokenEvent], None] | None = None, *, deadline: float | None = None) -> list[dict]:
        self._guard()
        request_schema.validate_payload(batch, self.profile)
        if not request_schema.is_concurrent(batch):
            raise RequestValidationError("generate_concurrent takes a concurrent batch")
        requests = batch["requests"]
        self._check_capacity(batch["context_capacity"], len(requests))
        try:
            self._admit()
            session = BatchedSession(self.runner, requests, self.vote, sink, deadline=deadline, clock=self.clock)
            prefill_seconds, ttft = [], []
            for lane, req in enumerate(requests):  # sequential prefills, each into its own lane
                t0 = self.clock()
                first = self.runner.prefill(lane, req["prompt_ids"])
                prefill_seconds.append(self.clock() - t0)
                session.accept_prefill(lane, first, self.runner.read_status())
                ttft.append(self.clock() - t0)
            for lane in range(len(requests), self.runner.lanes):
                self.runner.deactivate(lane)
            t1 = self.clock()
            walls = [0.0] * len(requests)
            while not session.finished:
                live = [st.lane for st in session.lanes if not st.finished]
                session.step()
                now = self.clock() - t1
                for lane in live:
                    walls[lane] = now
            reports = []
            for st in session.lanes:
                self._consensus(st)
                reports.append(self._report(st, prefill_seconds[st.lane], ttft[st.lane], walls[st.lane]))
            self.requests_done += len(requests)
            return reports
        except Exception:
            self.poisoned = True
            raise

    # ------------------------------------------------------------------ queue
    def run_payload(self, payload: dict, sink=None, *, deadline: float | None = None) -> list[dict]:
        """A single request, a sequential batch (each with a fresh cache) or a concurrent batch."""
        if request_schema.is_concurrent(payload):
            return self.generate_concurrent(payload, sink, deadline=deadline)
        return [self.generate(req, sink, deadline=deadline) for req in request_schema.requests_of(payload, self.profile)]
