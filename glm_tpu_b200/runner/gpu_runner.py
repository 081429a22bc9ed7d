"""Per-GPU model runner: resident weights, caches, the prefill program and the CUDA-graph decode program.

The runner is what the engine drives.  It owns

* the resident weights (``DeviceWeights``) and the peer-buffer registry,
* the device state for ``lanes`` concurrent chats (striped KV/index caches, token/position registers),
* the *decode program*: one token for every lane, captured once in a CUDA graph and replayed per step
  (positions and tokens live in device memory, so the graph is static),
* the *prefill program*: chunks of one lane's prompt, launched eagerly.

Parity: reference ``glm_tpu/runner/tpu_runner.py:29-289`` (load phases, program set, batch programs),
``runner/programs.py:80-118``, ``runner/kv_cache_manager.py:15-57``, ``runner/compilation_manager.py:28-69``
(here a program is a captured CUDA graph instead of a compiled XLA executable).
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass, field

import torch

from glm_tpu_b200.config.cache import CacheConfig
from glm_tpu_b200.config.parallel import ParallelLayout, default_expert_split
from glm_tpu_b200.models.glm_moe_dsa.model import RING, DecoderState, GlmMoeDsaModel, Workspace
from glm_tpu_b200.models.glm_moe_dsa.weights import DeviceWeights
from glm_tpu_b200.ops import native
from glm_tpu_b200.parallel.peer import PeerGroup
from glm_tpu_b200.runner.admission import check_collective_plan, project_live, project_memory, require_admitted


@dataclass
class ProgramRecord:
    name: str
    kind: str  # 'cuda_graph' or 'eager'
    rows: int
    launches: int
    capture_seconds: float = 0.0


@dataclass
class RunnerReport:
    phases: dict = field(default_factory=dict)
    programs: list = field(default_factory=list)
    memory: dict = field(default_factory=dict)


class _LaunchCounter:
    """Counts kernel launches issued through the native library while a program is being recorded."""

    def __init__(self):
        self.count = 0

    def __enter__(self):
        from glm_tpu_b200.ops import native

        self._native = native
        self._orig = native._check

        def counting(code, what):
            self.count += 1
            self._orig(code, what)

        native._check = counting
        return self

    def __exit__(self, *exc):
        self._native._check = self._orig


class GpuModelRunner:
    def __init__(self, weights: DeviceWeights, *, context_capacity: int, lanes: int = 1, stripe: int = 64, comm: str | None = None,
                 group=None, prefill_chunk: int = 512, use_graphs: bool | None = None, wait_limit: int | None = None,
                 staging_bytes: int | None = None, kv_layout: str = "auto", replica_budget_bytes: int = 32 << 30,
                 decode_path: str = "auto", mega_compat_ksplit: bool | None = None, emulate_shard: bool = False):
        from glm_tpu_b200 import envs

        # what the caller leaves open comes from the environment registry (GLM_B200_COMM, GLM_B200_CUDA_GRAPHS, GLM_B200_WAIT_LIMIT)
        comm = envs.GLM_B200_COMM if comm is None else comm
        use_graphs = envs.GLM_B200_CUDA_GRAPHS if use_graphs is None else use_graphs
        wait_limit = envs.GLM_B200_WAIT_LIMIT if wait_limit is None else wait_limit
        if comm not in ("fused", "nccl"):
            raise ValueError("comm is 'fused' or 'nccl'")
        self.weights = weights
        self.g, self.layout = weights.geometry, weights.layout
        self.device = weights.embed.device
        self.world, self.rank = self.layout.world, self.layout.rank
        # KV layout: a full replica of the latent cache on every GPU removes all attention exchanges; stripe the caches
        # by position over the GPUs once a replica would not fit the budget (long contexts, many lanes).
        if kv_layout not in ("auto", "striped", "replicated"):
            raise ValueError("kv_layout is 'auto', 'striped' or 'replicated'")
        replica = CacheConfig(self.g, context_capacity, world=1, stripe=stripe, lanes=lanes)
        if kv_layout == "auto":
            kv_layout = "replicated" if replica.cache_bytes_per_gpu() <= replica_budget_bytes else "striped"
        self.kv_layout = kv_layout if self.world > 1 else "local"
        self.cache = replica if kv_layout == "replicated" else CacheConfig(self.g, context_capacity, world=self.world, stripe=stripe,
                                                                          lanes=lanes)
        self.lanes = lanes
        self.report = RunnerReport()
        self.use_graphs = use_graphs
        self.prefill_chunk = prefill_chunk
        t0 = time.perf_counter()
        if staging_bytes is None:
            g = self.g
            staging_bytes = lanes * (g.attention_heads * g.kv_row_width * 2 + context_capacity * 4
                                     + self.world * self.layout.heads_local * (g.kv_lora_rank + 2) * 4 + self.world * 8) + (1 << 20)
            if self.world > 1 and prefill_chunk > 8:  # output + partial-tile slots of the prefill GEMM with the fused all-reduce
                staging_bytes += prefill_chunk * g.hidden_size * 2 + native.gemm_allreduce_part_bytes(prefill_chunk, g.hidden_size, self.world) + 8192
        # memory admission BEFORE anything large is allocated: the projection (weights already resident + caches of every lane
        # + staging + workspaces) against the device's size and against what the driver reports as free right now
        self.report.memory = self._project(weights.bytes_resident, staging_bytes, already_resident=weights.bytes_resident)
        require_admitted(self.report.memory)
        self._staging_bytes = staging_bytes
        with torch.cuda.device(self.device):
            # emulate_shard (measurements only): this process holds rank `rank`'s shard of a `world`-GPU layout but runs alone:
            # every exchange is skipped, so the outputs mean nothing and the decode step costs what one GPU of the box spends
            # outside the exchanges (persistent decode kernel only)
            self.emulate_shard = bool(emulate_shard) and self.world > 1
            if self.emulate_shard:
                self.peer = PeerGroup(1, 0, staging_bytes=0, wait_limit=wait_limit, group=None, device=self.device)
            else:
                self.peer = PeerGroup(self.world, self.rank, staging_bytes=staging_bytes if self.world > 1 else 0,
                                      wait_limit=wait_limit, group=group, device=self.device)
            self.model = GlmMoeDsaModel(weights, self.cache, self.peer, comm=comm, group=group)
            self.model.emulated_shard = self.emulate_shard
            self.state = DecoderState.allocate(self.cache, self.device)
            self.decode_ws = Workspace(self.model, lanes, "decode")
            # decode program: 'kernels' (default) is the per-kernel sequence; 'phases' runs the fused phases of
            # csrc/decode_mega.cu as 11 kernels per layer, 'mega' as stretches of one persistent cooperative kernel.  Both fused
            # forms agree with 'kernels' bit for bit and are slower on B200 as measured (they give up occupancy, the L1 and a
            # small instruction footprint for fewer launches), so 'auto' means 'kernels'.  GLM_B200_DECODE overrides 'auto'.
            import os

            if decode_path == "auto":
                decode_path = os.environ.get("GLM_B200_DECODE", "kernels")
            if decode_path not in ("auto", "phases", "mega", "kernels"):
                raise ValueError("decode_path is 'auto', 'phases', 'mega' or 'kernels'")
            if mega_compat_ksplit is None and "GLM_B200_MEGA_KSPLIT" in os.environ:
                mega_compat_ksplit = os.environ["GLM_B200_MEGA_KSPLIT"] == "compat"
            self.mega = None
            if decode_path != "kernels":
                from glm_tpu_b200.models.glm_moe_dsa.mega import MegaDecoder

                mega = MegaDecoder(self.model, self.decode_ws, self.state, compat_ksplit=mega_compat_ksplit,
                                   mode="persistent" if decode_path == "mega" else "phases")
                if mega.supported:
                    self.mega = mega
                elif decode_path != "auto":
                    raise ValueError(f"the fused decode phases do not take this configuration (code {mega.supported_code})")
            self.decode_path = ("mega" if self.mega.mode == "persistent" else "phases") if self.mega is not None else "kernels"
            self.prefill_ws = None
            self._prefill_out = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._graph = None
            self._graph_stream = torch.cuda.Stream(device=self.device)
        self.report.phases["allocate"] = time.perf_counter() - t0
        self.decode_launches = 0
        self.steps_issued = 0
        self._feed_host = None
        self.fed_bytes_per_step = 0

    # ------------------------------------------------------------------ admission
    def _project(self, weight_bytes: int, staging_bytes: int, *, already_resident: int, mem_info=None) -> dict:
        projection = project_memory(self.g, self.layout, self.cache, weight_bytes, staging_bytes)
        free, total = mem_info if mem_info is not None else torch.cuda.mem_get_info(self.device)
        return project_live(projection, free, total, already_resident=already_resident)

    def admit_request(self, mem_info=None) -> dict:
        """Before every request: everything this runner projected is resident by now, so the device must still have the reserve
        free (another process on the GPU, a leak) and the status word must be clean.  Raises ``PlanValidationError``."""
        admitted = self._project(self.weights.bytes_resident, self._staging_bytes, already_resident=1 << 62, mem_info=mem_info)
        require_admitted(admitted)
        self.report.memory["last_request"] = {"device_free": admitted["device_free"], "reserve": admitted["reserve"]}
        return admitted

    # ------------------------------------------------------------------ decode program
    def _decode_body(self) -> None:
        st, ws, m = self.state, self.decode_ws, self.model
        if self.mega is not None:
            self.mega.step()
            return
        logits = m.run_rows(ws, st, st.tokens, st.positions, st.lane_ids, st.active, self.lanes, decode=True,
                            max_ctx=self.cache.context_capacity, head="argmax")
        m.sample(ws, st, logits, self.lanes, st.active, advance=3)

    def build_decode_program(self) -> ProgramRecord:
        """Warm up eagerly (lanes inactive: no cache write, no advance), then capture the step in a CUDA graph."""
        t0 = time.perf_counter()
        with torch.cuda.device(self.device):
            saved = self.state.active.clone()
            self.state.active.zero_()
            with _LaunchCounter() as counter, native.record_exchanges() as plan:
                self._decode_body()
            self.decode_launches = counter.count
            # the cross-GPU exchanges of the step, in launch order, against the rules the in-kernel protocol rests on (alternating
            # all-reduce channels, a signal at most once between two all-reduces, payloads within the slots): refused before capture
            check_collective_plan(plan, world=self.peer.world)
            self.report.phases["collective_plan"] = {"exchanges": len(plan), "allreduces": sum(1 for op in plan if op["kind"] == "allreduce")}
            torch.cuda.synchronize(self.device)
            kind = "eager"
            if self.use_graphs and self.model.comm_mode == "fused" or (self.use_graphs and self.world == 1):  # noqa: E129
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=self._graph_stream):
                        self._decode_body()
                except RuntimeError:
                    if self.mega is None:
                        raise
                    # a driver that will not record a cooperative launch: the same grid as an ordinary launch (it fits the GPU
                    # and nothing else runs beside it, so every CTA is resident all the same)
                    torch.cuda.synchronize(self.device)
                    native.set_mega_cooperative(0)
                    self.report.phases["mega_cooperative_capture"] = "refused: ordinary launch"
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=self._graph_stream):
                        self._decode_body()
                self._graph = graph
                kind = "cuda_graph"
            self.state.active.copy_(saved)
            self.state.step_counter.zero_()
            self.steps_issued = 0
            torch.cuda.synchronize(self.device)
            self.peer.check_status()
        rec = ProgramRecord("decode:" + self.decode_path, kind, self.lanes, self.decode_launches, time.perf_counter() - t0)
        self.report.programs.append(rec)
        return rec

    def decode_step(self) -> None:
        """Enqueue one decode step for every active lane (asynchronous)."""
        if self._graph is None and not self.report.programs:
            self.build_decode_program()
        if self._graph is not None:
            self._graph.replay()
        else:
            self._decode_body()
        self.steps_issued += 1

    def feed_tokens(self, tokens: dict) -> None:
        """Copy the committed tokens of the given lanes (``lane -> token``) from pinned host memory into the device's token
        registers (asynchronous, on the current stream: the next decode step reads them).  4 bytes per lane; a lane that is not
        named keeps being fed what it was fed last, which a frozen lane never uses."""
        if self._feed_host is None:
            self._feed_host = torch.zeros(self.lanes, dtype=torch.int32).pin_memory()
        for lane, token in tokens.items():
            self._feed_host[lane] = int(token)
        with torch.cuda.device(self.device):
            self.state.tokens.copy_(self._feed_host, non_blocking=True)
        self.fed_bytes_per_step = 4 * self.lanes

    def read_last_tokens(self) -> list[int]:
        """Tokens of the most recent decode step, one per lane (-1 for a frozen lane).  Synchronizes."""
        return self.read_step_tokens(self.steps_issued - 1)

    def read_status(self) -> int:
        """The device status word (0 = clean); reading clears it."""
        return self.peer.read_status()

    def read_step_tokens(self, step_index: int) -> list[int]:
        """Tokens produced by decode step ``step_index`` (synchronizes; one small D2H copy)."""
        row = self.state.out_tokens[step_index % RING].cpu()
        return [int(v) for v in row]

    # ------------------------------------------------------------------ prefill program
    def _ensure_prefill_ws(self) -> Workspace:
        if self.prefill_ws is None:
            with torch.cuda.device(self.device):
                self.prefill_ws = Workspace(self.model, self.prefill_chunk, "prefill", attn_rows=min(self.prefill_chunk, 64),
                                            score_stride=self.cache.context_capacity, peer_visible=False)
        return self.prefill_ws

    def prefill(self, lane: int, token_ids) -> int:
        """Run a prompt through ``lane`` with a fresh cache; returns the first generated token.

        After the call the lane is active, its position is ``len(token_ids)`` and its next input is that token.
        """
        n = len(token_ids)
        if not 0 < n < self.cache.context_capacity:
            raise ValueError("prompt does not fit the context capacity")
        ws = self._ensure_prefill_ws()
        st, m = self.state, self.model
        with torch.cuda.device(self.device):
            ids = torch.as_tensor(list(token_ids), dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            lane_t = torch.full((self.prefill_chunk,), lane, dtype=torch.int32, device=self.device)
            st.reset_lane(lane)
            logits = None
            for start in range(0, n, self.prefill_chunk):
                rows = min(self.prefill_chunk, n - start)
                pos = torch.arange(start, start + rows, dtype=torch.int32, device=self.device)
                last = start + rows == n
                logits = m.run_rows(ws, st, ids[start : start + rows], pos, lane_t, None, rows, decode=False, max_ctx=start + rows,
                                    head_rows=slice(rows - 1, rows) if last else slice(0, 1), lane_of_rows=lane)
            m.sample(ws, st, logits, 1, None, advance=1, tokens_out=st.tokens[lane : lane + 1], positions=st.positions[lane : lane + 1],
                     out=self._prefill_out)
            st.positions[lane] = n
            st.active[lane] = 1
            token = int(self._prefill_out.cpu()[0])
            self.peer.check_status()
        return token

    def memory_stats(self) -> dict:
        """Device memory as the allocator and the driver see it, plus what this runner knows it holds (per-request records)."""
        free, total = torch.cuda.mem_get_info(self.device)
        st = self.state
        return {
            "device_total_bytes": int(total), "device_free_bytes": int(free),
            "torch_allocated_bytes": int(torch.cuda.memory_allocated(self.device)),
            "torch_peak_allocated_bytes": int(torch.cuda.max_memory_allocated(self.device)),
            "weights_bytes": int(self.model.w.bytes_resident),
            "kv_cache_bytes": int(st.kv_cache.numel() * st.kv_cache.element_size()),
            "index_cache_bytes": int(st.index_cache.numel() * st.index_cache.element_size()),
            "staging_bytes": int(self.peer._total) if self.peer.world > 1 else 0,
            "kv_layout": self.kv_layout,
            "fallbacks": dict(self.model.fallbacks),  # library routines taken in place of the hand-written kernels, with counts
        }

    def synthetic_context(self, lane: int, depth: int, seed: int = 0) -> None:
        """Benchmarks only: make ``lane`` look ``depth`` tokens deep without running a prefill.

        The lane's cache rows are filled with random bf16 values (a normalized latent and a rotated key have this
        scale), its position is set to ``depth`` and it is activated; decode steps then cost what they cost at that
        depth (indexer scoring over ``depth`` keys, top-k, 2,048 selected rows), which a short prompt does not show.
        """
        if not 0 < depth < self.cache.context_capacity:
            raise ValueError("depth does not fit the context capacity")
        st = self.state
        with torch.cuda.device(self.device):
            native.fill_random_bf16(st.kv_cache[lane], seed * 2 + 1, 0.0, 0.5)
            native.fill_random_bf16(st.index_cache[lane], seed * 2 + 2, 0.0, 0.5)
            st.tokens[lane] = 1 + (seed % 1000)
            st.positions[lane] = depth
            st.active[lane] = 1
            torch.cuda.synchronize(self.device)

    def deactivate(self, lane: int) -> None:
        self.state.active[lane] = 0

    def close(self) -> None:
        self._graph = None
        if self.peer.world > 1:
            torch.cuda.synchronize(self.device)
            self.peer.check_canaries()  # a kernel (of any rank) that overran a staging region wrote into its guard band
        self.peer.close()


def build_runner(geometry, *, world: int = 1, rank: int = 0, device=None, checkpoint=None, seed: int = 0, expert_split: str | None = None,
                 **kwargs) -> GpuModelRunner:
    """Convenience constructor: shard ``checkpoint`` (a runtime-layout mapping) or random-init on the device."""
    from glm_tpu_b200.models.glm_moe_dsa.weights import random_device_weights, shard_checkpoint

    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    if expert_split is None and checkpoint is not None and "__expert_split__" in checkpoint:
        expert_split = checkpoint["__expert_split__"]  # a packed checkpoint was cut one way: the layout follows it
    layout = ParallelLayout(geometry, world, rank, expert_split or default_expert_split(geometry, world))
    with torch.cuda.device(device):
        weights = shard_checkpoint(checkpoint, layout, device) if checkpoint is not None else random_device_weights(layout, device, seed)
    return GpuModelRunner(weights, **kwargs)
