"""A CPU runner built on the contract oracle: the engine's reference backend.

It has the interface of ``GpuModelRunner`` (``prefill`` / ``decode_step`` / ``read_last_tokens`` / ``read_status`` /
``deactivate``) but recomputes the whole sequence through ``oracle.contract.forward`` at every step.  It is the timed
CPU baseline for small models, the backend of the CPU end-to-end tests of the worker, the controller and the servers,
and an independent check of the incremental GPU runner (same tokens on the same checkpoint, up to near-ties).
"""

from __future__ import annotations

from types import SimpleNamespace

from glm_tpu_b200.oracle import contract


class OracleRunner:
    def __init__(self, geometry, checkpoint, *, context_capacity: int, lanes: int = 1):
        self.g = geometry
        self.weights = contract.OracleWeights.from_checkpoint(geometry, checkpoint)
        self.cache = SimpleNamespace(context_capacity=context_capacity)
        self.lanes = lanes
        self.world, self.rank = 1, 0
        self.kv_layout = "host"
        self.sequences: list[list[int]] = [[] for _ in range(lanes)]
        self.active = [False] * lanes
        self._last = [-1] * lanes
        self.steps_issued = 0

    def _next(self, lane: int) -> int:
        trace = contract.forward(self.weights, self.sequences[lane], capacity=self.cache.context_capacity)
        return int(trace.tokens[-1])

    def prefill(self, lane: int, token_ids) -> int:
        if not 0 < len(token_ids) < self.cache.context_capacity:
            raise ValueError("prompt does not fit the context capacity")
        self.sequences[lane] = list(token_ids)
        token = self._next(lane)
        self.sequences[lane].append(token)
        self.active[lane] = True
        return token

    def build_decode_program(self):
        return SimpleNamespace(name="decode", kind="host", rows=self.lanes, launches=0)

    def decode_step(self) -> None:
        for lane in range(self.lanes):
            if self.active[lane] and len(self.sequences[lane]) < self.cache.context_capacity:
                token = self._next(lane)
                self.sequences[lane].append(token)
                self._last[lane] = token
            else:
                self._last[lane] = -1
        self.steps_issued += 1

    def read_last_tokens(self) -> list[int]:
        return list(self._last)

    def read_status(self) -> int:
        return 0

    def deactivate(self, lane: int) -> None:
        self.active[lane] = False

    def memory_stats(self) -> dict:
        return {"device": "cpu"}

    def close(self) -> None:
        pass
