"""The GLM-MoE-DSA decoder as a sequence of CUDA kernel launches on one GPU of the box.

One ``GlmMoeDsaModel`` lives in each per-GPU process.  ``run_rows`` pushes ``R`` token rows through all layers:

* decode (``R`` = live lanes, 1..8): every projection is a weight-streaming skinny kernel; cross-GPU sums and
  gathers happen *inside* kernels over peer memory (``comm='fused'``) or through NCCL (``comm='nccl'``, the
  baseline).  The launch sequence is static, reads positions/tokens from device memory and is captured in a CUDA
  graph by the runner.
* prefill (``R`` up to a few thousand rows of one lane): projections run on the tcgen05 GEMM (with the all-reduce of
  K-split partial tiles fused into its epilogue on several GPUs), routed experts on the grouped tcgen05 kernel that decodes
  FP8 on the way to the tensor core, everything else through the same hand-written kernels as decode; the score and
  attention-partial merges of prefill use NCCL.

Per layer (decode): add+RMSNorm -> q_a|kv_a|indexer projections -> LoRA norms, RoPE, cache-row write -> q_b ->
query RoPE -> q-absorb (+ all-gather of queries) -> [full layers: indexer scores (+ all-gather) -> exact top-k]
-> owner-local sparse MLA partials -> merge (+ exchange to head owners) -> value projection -> o_proj (+ all-reduce)
-> add+RMSNorm -> dense MLP, or router -> routed FP8 experts + shared expert -> combine (+ all-reduce).

Parity: reference ``glm_tpu/models/glm_moe_dsa/model.py:46-159`` (decode_step), ``decoder_layer.py:538-740`` (layer
bodies), ``prefill.py:49-235``; the reference's ``lax.psum`` / ``all_gather`` call sites are replaced as described above.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from glm_tpu_b200.config.cache import CacheConfig
from glm_tpu_b200.models.glm_moe_dsa.weights import DeviceWeights, LayerWeights
from glm_tpu_b200.ops import native
from glm_tpu_b200.oracle.contract import rope_table
from glm_tpu_b200.parallel.peer import PeerGroup

RING = 64


def _f32(x: float) -> float:
    return float(np.float32(x))


@dataclass
class DecoderState:
    """Device-resident caches and lane registers (reference ``models/glm_moe_dsa/state.py:23-69``)."""

    kv_cache: torch.Tensor  # [lanes, layers, local_cap, W] bf16
    index_cache: torch.Tensor  # [lanes, full_layers, local_cap, D] bf16
    tokens: torch.Tensor  # [lanes] int32: the token each lane feeds next
    positions: torch.Tensor  # [lanes] int32: its position (= tokens already cached)
    active: torch.Tensor  # [lanes] int32
    lane_ids: torch.Tensor  # [lanes] int32 arange
    out_tokens: torch.Tensor  # [RING, lanes] int32
    step_counter: torch.Tensor  # [1] int32

    @classmethod
    def allocate(cls, cache: CacheConfig, device) -> "DecoderState":
        dev = torch.device(device)
        z = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)  # noqa: E731
        return cls(
            kv_cache=torch.zeros(cache.kv_cache_shape, dtype=torch.bfloat16, device=dev),
            index_cache=torch.zeros(cache.index_cache_shape, dtype=torch.bfloat16, device=dev),
            tokens=z(cache.lanes),
            positions=z(cache.lanes),
            active=z(cache.lanes),
            lane_ids=torch.arange(cache.lanes, dtype=torch.int32, device=dev),
            out_tokens=torch.full((RING, cache.lanes), -1, dtype=torch.int32, device=dev),
            step_counter=z(1),
        )

    def reset_lane(self, lane: int) -> None:
        """Fresh cache for a new request on ``lane`` (stale rows are never read: reads are bounded by the position)."""
        self.positions[lane] = 0
        self.tokens[lane] = 0
        self.active[lane] = 0


class Workspace:
    """Scratch tensors for ``rows`` token rows.  Peer-visible ones live in the staging buffer when world > 1."""

    def __init__(self, model: "GlmMoeDsaModel", rows: int, tag: str, attn_rows: int | None = None, score_stride: int | None = None,
                 peer_visible: bool = True):
        g, lay, dev = model.g, model.layout, model.device
        self.peer_visible = peer_visible and model.peer.world > 1 and model.comm_mode == "fused"
        self.rows = rows
        self.attn_rows = min(rows, attn_rows or rows)
        H, Q, L, rd, W = g.hidden_size, g.q_lora_rank, g.kv_lora_rank, g.qk_rope_head_dim, g.kv_row_width
        IH, D, k = g.index_heads, g.index_head_dim, g.index_top_k
        hl, ht = lay.heads_local, model.attn_heads
        bf = lambda *s: torch.empty(s, dtype=torch.bfloat16, device=dev)  # noqa: E731
        f32 = lambda *s: torch.empty(s, dtype=torch.float32, device=dev)  # noqa: E731
        i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)  # noqa: E731
        self.residual, self.x, self.update = bf(rows, H), bf(rows, H), bf(rows, H)
        self.proj_a = f32(rows, (Q + W + D + IH + 3) // 4 * 4)  # rows stay 16-byte aligned for float4 loads
        self.q_resid = bf(rows, Q)
        self.head_w = f32(rows, IH)
        self.q_proj = f32(rows, hl * g.qk_head_dim + IH * D)
        self.q_nope = bf(rows, hl, g.qk_nope_head_dim)
        self.q_idx = f32(rows, IH, D)
        self.score_stride = score_stride or model.cache.context_capacity
        peer = model.peer
        self.r_q = self.r_scores = self.r_xpart = self.r_cand = None
        if self.peer_visible:
            self.r_cand = peer.region(f"{tag}.cand", peer.world * rows * 8)
            self.cand = peer.tensor(self.r_cand, (peer.world, rows), torch.int64)
        else:
            self.cand = torch.zeros((max(1, peer.world), rows), dtype=torch.int64, device=dev)
        if self.peer_visible and model.striped:  # the attention exchanges exist only with position-striped caches
            self.r_q = peer.region(f"{tag}.q_full", rows * ht * W * 2)
            self.r_scores = peer.region(f"{tag}.scores", rows * self.score_stride * 4)
            self.r_xpart = peer.region(f"{tag}.xpart", peer.world * self.attn_rows * hl * (L + 2) * 4)
            self.q_full = peer.tensor(self.r_q, (rows, ht, W), torch.bfloat16)
            self.scores = peer.tensor(self.r_scores, (rows, self.score_stride), torch.float32)
        else:
            self.q_full = bf(rows, ht, W)
            self.scores = f32(rows, self.score_stride)
        # N operand of the many-rows indexer (three bf16 pieces of every fp32 query row): prefill workspaces only
        self.idx_pieces = (torch.empty(native.indexer_rows_scratch_bytes(rows), dtype=torch.uint8, device=dev)
                           if rows >= native.INDEXER_ROWS_MIN and native.indexer_takes_raw_query(g.index_heads, g.index_head_dim) else None)
        self.local_best = torch.zeros(rows, dtype=torch.int64, device=dev)  # packed argmax keys of this rank's vocabulary slice
        self.sel_global, self.sel_local, self.sel_counts = i32(rows, k), i32(rows, k), i32(rows, 2)
        self.max_chunks = -(-k // native.attn_chunk())
        self.part_o = f32(self.attn_rows, self.max_chunks, ht, L)
        self.part_ml = f32(self.attn_rows, self.max_chunks, ht, 2)
        self.o_lat = bf(rows, hl, L)
        self.attn_v = bf(rows, hl * g.v_head_dim)
        self.attn_out = bf(rows, H)
        self.partial = f32(rows, H)
        E, tk, I = g.num_routed_experts, g.routed_top_k, lay.moe_cols_local
        self.router_logits = f32(rows, E)
        self.topk_ids, self.topk_w = i32(rows, tk), f32(rows, tk)
        self.act = bf(rows * tk, I)
        self.dw = bf(rows * tk, H)
        self.act_shared = bf(rows, max(lay.shared_cols_local, 8))
        self.dense_act = bf(rows, max(lay.dense_cols_local, 8))
        self.routed_partial = f32(rows, H)
        self.logits = bf(rows, lay.vocab_local)
        self.kv_new = bf(rows, W)
        self.idx_key_new = bf(rows, D)
        self._sorted = None
        self._route = None
        self._route8 = None
        self._pairs: dict = {}
        # many-row workspaces on several GPUs: output and partial-tile slots of the GEMM with the fused all-reduce
        self.r_gemm_out = self.r_gemm_part = None
        if rows > 8 and peer.world > 1 and model.comm_mode == "fused":
            try:
                self.r_gemm_out = peer.region(f"{tag}.gemm_out", rows * H * 2)
                self.r_gemm_part = peer.region(f"{tag}.gemm_part", native.gemm_allreduce_part_bytes(rows, H, peer.world))
                self.gemm_out = peer.tensor(self.r_gemm_out, (rows, H), torch.bfloat16)
            except MemoryError:  # staging sized without it: the caller falls back to the library all-reduce, and says so
                self.r_gemm_out = self.r_gemm_part = None
                model.note_fallback("GEMM then library all-reduce", f"the staging buffer has no room for the fused GEMM all-reduce of {rows} rows")

    def partial_pair(self, rows: int, H: int) -> torch.Tensor:
        """``[2, rows, H]`` fp32 (routed and shared partial sums of a chunk, all-reduced together), kept per row count."""
        pair = self._pairs.get(rows)
        if pair is None:
            if len(self._pairs) >= 4:
                self._pairs.clear()
            pair = self._pairs[rows] = torch.empty((2, rows, H), dtype=torch.float32, device=self.residual.device)
        return pair

    def route_buffers(self, routes: int, el: int):
        """``tiles [routes / 128 + el, 4]``, ``n_tiles [1]``, ``perm [routes]`` of the expert sort, allocated on first use."""
        if self._route is None or self._route[2].shape[0] < routes or self._route[0].shape[0] < routes // 128 + el:
            dev = self.residual.device
            self._route = (torch.zeros((routes // 128 + el, 4), dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev),
                           torch.empty(routes, dtype=torch.int32, device=dev))
        return self._route[0][: routes // 128 + el], self._route[1], self._route[2][:routes]

    def route_buffers8(self, routes: int, el: int):
        """``tile_expert [routes / 8 + el]``, ``tile_routes [.., 8]``, ``n_tiles [1]``, ``perm [routes]`` of the 8-route expert sort."""
        tiles = routes // 8 + el
        if self._route8 is None or self._route8[3].shape[0] < routes or self._route8[0].shape[0] < tiles:
            dev = self.residual.device
            self._route8 = (torch.full((tiles,), -1, dtype=torch.int32, device=dev), torch.full((tiles, 8), -1, dtype=torch.int32, device=dev),
                            torch.zeros(1, dtype=torch.int32, device=dev), torch.empty(routes, dtype=torch.int32, device=dev))
        return self._route8[0][:tiles], self._route8[1][:tiles], self._route8[2], self._route8[3][:routes]

    def sorted_buffers(self, routes: int, H: int, I: int):
        """Expert-sorted activations and SwiGLU outputs of the grouped (prefill) expert GEMM, allocated on first use."""
        if self._sorted is None or self._sorted[0].shape[0] < routes:
            dev = self.residual.device
            self._sorted = (torch.empty((routes, H), dtype=torch.bfloat16, device=dev), torch.empty((routes, I), dtype=torch.bfloat16, device=dev))
        return self._sorted[0][:routes], self._sorted[1][:routes]


class GlmMoeDsaModel:
    def __init__(self, weights: DeviceWeights, cache: CacheConfig, peer: PeerGroup, *, comm: str = "fused", group=None):
        self.w, self.cache, self.peer = weights, cache, peer
        self.g, self.layout = weights.geometry, weights.layout
        self.device = weights.embed.device
        self.world, self.rank = self.layout.world, self.layout.rank
        # cache.world == world: caches striped by position over the GPUs (needed when a replica would not fit);
        # cache.world == 1 with several GPUs: every GPU keeps the whole latent cache (it is shared by all heads),
        # attends with its own heads only, and attention needs no cross-GPU exchange at all.
        if cache.world not in (1, self.world):
            raise ValueError("the caches are either replicated (cache world 1) or striped over all GPUs")
        self.striped = cache.world > 1
        self.cache_rank = self.rank if self.striped else 0
        self.attn_heads = self.g.attention_heads if (self.striped or self.world == 1) else self.layout.heads_local
        self.head_base = self.rank * self.layout.heads_local if self.striped else 0
        if comm not in ("fused", "nccl"):
            raise ValueError("comm is 'fused' or 'nccl'")
        self.comm_mode = comm
        self.group = group
        g = self.g
        self.rope = rope_table(cache.context_capacity, g.qk_rope_head_dim, g.rope_theta).to(self.device)
        j = torch.arange(0, g.qk_rope_head_dim, 2, dtype=torch.float32)
        self.inv_freq = torch.pow(torch.tensor(g.rope_theta, dtype=torch.float32), -j / g.qk_rope_head_dim).to(self.device)
        self.status = None  # kernels that take a status pointer get the registry's word
        self.softmax_scale = _f32(g.qk_head_dim**-0.5)
        self.index_scale = _f32(g.index_head_dim**-0.5)
        self.head_scale = _f32(g.index_heads**-0.5)
        self.trace = None  # set to a dict to record intermediates (tests)
        native.set_moe_experts_total(self.g.num_routed_experts)
        self.fallbacks: dict[str, int] = {}  # library routines taken in place of the hand-written kernels (see note_fallback)
        self.emulated_shard = False  # measurements: this process holds one rank's shard and skips every exchange (see GpuModelRunner)
        import os

        # independent branches of the decode step (shared expert | routed experts; absorbed query | indexer + top-k) run on two
        # streams; GLM_B200_OVERLAP=0 keeps everything on one stream
        self.side = torch.cuda.Stream(device=self.device) if os.environ.get("GLM_B200_OVERLAP", "1") != "0" else None
        self.fold_q_post = os.environ.get("GLM_B200_FOLD_Q_POST", "1") != "0"
        self.nvtx = os.environ.get("GLM_B200_NVTX", "0") == "1"
        # the one-launch expert sort takes up to 256 resident experts and contiguous ids; other shapes use the library-op sort
        # (`_route_tiles128`), and tests set this attribute to compare the two on shapes both take
        self.route_sort_kernel = True
        self.few_routes_gemv = True  # prefill chunks with few routes per expert on average: GEMV kernels on 8-route tiles (tests compare)
        self.few_routes_limit = int(os.environ.get("GLM_B200_FEW_ROUTES", "12"))  # mean routes per expert up to which that path is taken
        self.merge_vproj = os.environ.get("GLM_B200_MERGE_VPROJ", "1") != "0"  # decode: chunk merge + value projection in one launch
        self.prefill_rows_attention = os.environ.get("GLM_B200_PREFILL_ATTENTION", "rows") != "split"
        # Prefill projections whose K is split over the GPUs use the GEMM with the all-reduce in its epilogue (about 1.2x the
        # GEMM + library all-reduce on 2 and on 8 GPUs); GLM_B200_PREFILL_GEMM_AR=nccl selects the library path.
        self.prefill_gemm_allreduce = os.environ.get("GLM_B200_PREFILL_GEMM_AR", "fused") != "nccl"

    # ------------------------------------------------------------------------------ helpers
    @property
    def _kc(self):
        """PeerComm for kernels with fused communication (None: single GPU or NCCL baseline)."""
        return self.peer.kernel_comm if self.comm_mode == "fused" else None

    def note_fallback(self, what: str, why: str) -> None:
        """A hand-written kernel was passed over for a library routine: counted per (what, why) for the runner's report and
        logged the first time, so a slow path never hides."""
        key = f"{what}: {why}"
        seen = self.fallbacks.get(key, 0)
        self.fallbacks[key] = seen + 1
        if not seen:
            import logging

            logging.getLogger("glm_tpu_b200.fallback").warning("rank %d falls back to %s", self.rank, key)

    def _allreduce_rows(self, partial_f32: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        if self.world > 1 and not self.emulated_shard:
            dist.all_reduce(partial_f32, group=self.group)
        return partial_f32

    def _mm(self, x: torch.Tensor, w: torch.Tensor, f32: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
        """``x @ w.T`` (bf16 operands, fp32 accumulate) for many rows: the tcgen05 GEMM; shapes it does not take
        (a dimension that is not a multiple of 8) go to the library GEMM.  ``out``: a ``[rows, N]`` view (unit column stride,
        16-byte aligned rows) that the kernel writes in place of a fresh tensor."""
        rows, K = x.shape
        N = w.shape[0]
        dtype = torch.float32 if f32 else torch.bfloat16
        if K % 8 == 0 and N % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 \
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            direct = (out is not None and out.dtype == dtype and tuple(out.shape) == (rows, N) and out.stride(1) == 1
                      and out.stride(0) % (4 if f32 else 8) == 0 and out.data_ptr() % 16 == 0)
            target = out if direct else torch.empty((rows, N), dtype=dtype, device=x.device)
            native.gemm_bf16_tc(x, w, target, status=self.peer.status_ptr)
            if out is not None and not direct:
                out.copy_(target)
            return out if out is not None else target
        self.note_fallback("library GEMM", f"operands [{rows}x{K}] x [{N}x{K}] are not 16-byte aligned rows of a multiple of 8")
        result = torch.mm(x, w.t(), out_dtype=torch.float32) if f32 else torch.mm(x, w.t())
        if out is not None:
            out.copy_(result)
            return out
        return result

    def _fork(self):
        """Make the side stream wait for everything issued so far on the current stream; returns the current stream."""
        main = torch.cuda.current_stream()
        event = torch.cuda.Event()
        event.record(main)
        self.side.wait_event(event)
        return main

    def _join(self, main) -> None:
        event = torch.cuda.Event()
        event.record(self.side)
        main.wait_event(event)

    def _mm_allreduce(self, ws: "Workspace", x: torch.Tensor, w: torch.Tensor) -> torch.Tensor | None:
        """``bf16(sum over GPUs of x_r @ w_r.T)`` ([rows, hidden]) in one kernel: tcgen05 tiles whose epilogue exchanges the
        partial tiles over NVLink.  None when this workspace has no staging for it or the shape does not fit."""
        rows, K = x.shape
        if not self.prefill_gemm_allreduce:
            return None
        if ws.r_gemm_out is None or w.shape[0] != self.g.hidden_size or K % 8 or x.stride(1) != 1 or x.stride(0) % 8 \
                or x.data_ptr() % 16 or w.data_ptr() % 16 or w.stride(0) % 8:
            if self.comm_mode == "fused":
                self.note_fallback("GEMM then library all-reduce", "no staging for the fused GEMM all-reduce in this workspace" if ws.r_gemm_out is None
                                   else f"shape [{rows}x{K}] x [{w.shape[0]}x{K}] does not fit the fused GEMM all-reduce")
            return None
        native.gemm_bf16_tc_allreduce(x, w, self.peer.comm, ws.r_gemm_part.offset, ws.r_gemm_out.offset, status=self.peer.status_ptr)
        native.wait_signal(self.peer.comm, native.SIG_GEMM)
        return ws.gemm_out[:rows]

    @staticmethod
    def _swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """``bf16(g * sigmoid(g) * u)`` of the bf16 gate / up projections of a prefill chunk (written over ``gate``)."""
        if gate.is_contiguous() and up.is_contiguous() and gate.numel() % 8 == 0 and gate.dtype == torch.bfloat16:
            return native.swiglu_rows(gate, up, gate)
        g32, u32 = gate.float(), up.float()  # odd shapes of fixtures only
        return (g32 * torch.sigmoid(g32) * u32).to(torch.bfloat16)

    def _linear_f32(self, x, w, out, decode: bool):
        """``out[:, :N] = x @ w.T`` in fp32."""
        n = w.shape[0]
        if decode:
            native.skinny_bf16(x, w, out, native.SK_OUT_F32, N=n, K=w.shape[1])
        else:
            self._mm(x, w, f32=True, out=out[: x.shape[0], :n])

    # ------------------------------------------------------------------------------ attention
    def _attention(self, ws: Workspace, lw: LayerWeights, layer: int, rows: int, row_pos, row_lane, row_active, state: DecoderState,
                   decode: bool, max_ctx: int, lane_of_rows: int | None = None):
        g, lay, cache = self.g, self.layout, self.cache
        full = g.indexer_types[layer] == "full"
        Q, L, rd, W = g.q_lora_rank, g.kv_lora_rank, g.qk_rope_head_dim, g.kv_row_width
        IH, D = g.index_heads, g.index_head_dim
        hl, ht, hb = lay.heads_local, self.attn_heads, self.head_base
        fused = ws.peer_visible
        kc = self.peer.comm if fused else None
        cw, cr = cache.world, self.cache_rank
        gather = self.striped and self.world > 1  # attention spans the GPUs: queries, scores and partials are exchanged
        xf = fused and gather                      # ... inside the kernels
        kx = kc if xf else None
        x = ws.x[:rows]
        a = native.QkvPostArgs()
        a.proj, a.proj_stride = ws.proj_a.data_ptr(), ws.proj_a.stride(0)
        a.q_norm_w, a.kv_norm_w = lw.q_a_norm.data_ptr(), lw.kv_a_norm.data_ptr()
        a.rope_table, a.inv_freq = self.rope.data_ptr(), self.inv_freq.data_ptr()
        a.k_norm_w = lw.k_norm_w.data_ptr() if full else None
        a.k_norm_b = lw.k_norm_b.data_ptr() if full else None
        a.row_pos, a.row_lane = row_pos.data_ptr(), row_lane.data_ptr()
        a.row_active = row_active.data_ptr() if row_active is not None else None
        a.q_resid, a.kv_new = ws.q_resid.data_ptr(), ws.kv_new.data_ptr()
        a.kv_cache, a.index_cache = state.kv_cache.data_ptr(), state.index_cache.data_ptr()
        a.head_w, a.idx_key_new = ws.head_w.data_ptr(), ws.idx_key_new.data_ptr()
        a.Q, a.L, a.rd, a.D, a.IH = Q, L, rd, D, IH
        a.has_indexer = int(full)
        a.layer, a.layers = layer, g.num_layers
        a.index_slot, a.full_layers = g.index_slot(layer), len(g.full_layers)
        a.local_cap, a.stripe, a.world, a.rank, a.capacity = cache.local_capacity, cache.stripe, cw, cr, cache.context_capacity
        a.eps, a.key_eps, a.head_scale = g.rms_norm_eps, cache.dsa.key_norm_eps, self.head_scale
        a.status = self.peer.status_ptr
        self._linear_f32(x, lw.w_qkv_a, ws.proj_a, decode)
        native.qkv_a_post(a, rows)

        self._linear_f32(ws.q_resid[:rows], lw.w_q_b, ws.q_proj, decode)
        b = native.QPostArgs()
        b.q, b.q_stride = ws.q_proj.data_ptr(), ws.q_proj.stride(0)
        b.rope_table, b.inv_freq, b.row_pos = self.rope.data_ptr(), self.inv_freq.data_ptr(), row_pos.data_ptr()
        b.q_nope, b.q_full, b.q_idx = ws.q_nope.data_ptr(), ws.q_full.data_ptr(), ws.q_idx.data_ptr()
        b.heads_local, b.head_base, b.heads_total = hl, hb, ht
        b.nope, b.rd, b.L, b.IH, b.D = g.qk_nope_head_dim, rd, L, IH, D
        b.has_indexer, b.capacity = int(full), cache.context_capacity
        # decode: the q_post work is folded into its consumers (q_absorb rounds and rotates its heads, the tcgen05 indexer
        # rotates the index query), one launch less per layer; prefill and other head shapes keep the separate kernel
        fold = decode and self.fold_q_post and self.trace is None and (not full or native.indexer_takes_raw_query(IH, D))
        if not fold:
            native.q_post(b, rows)
        fold_args = dict(q_proj=ws.q_proj, rope_table=self.rope, row_pos=row_pos, capacity=cache.context_capacity) if fold else {}

        forked = None
        if decode:
            if full and not gather and self.side is not None:
                # the absorbed query (needed by the attention) and the indexer scores + top-k (needed by the attention too)
                # depend on the same inputs and not on each other: run the former on the side stream
                forked = self._fork()
                with torch.cuda.stream(self.side):
                    native.q_absorb(ws.q_nope, rows, lw.kv_b, hl, hb, ht, g.qk_nope_head_dim, g.v_head_dim, L, rd, ws.q_full, 0, None,
                                    native.SIG_Q, **fold_args)
            else:
                native.q_absorb(ws.q_nope, rows, lw.kv_b, hl, hb, ht, g.qk_nope_head_dim, g.v_head_dim, L, rd, ws.q_full,
                                ws.r_q.offset if xf else 0, kx, native.SIG_Q, **fold_args)
            if gather and not xf:
                self._allgather_heads(ws.q_full[:rows])
        else:
            w_k = lw.kv_b[:, : g.qk_nope_head_dim, :]  # [hl, nope, L]
            q_c = torch.einsum("rhd,hdc->rhc", ws.q_nope[:rows], w_k)
            ws.q_full[:rows, hb : hb + hl, :L] = q_c
            if gather:
                self._allgather_heads(ws.q_full[:rows])

        if full:
            native.indexer_score(ws.q_idx, ws.head_w, state.index_cache, row_pos, row_lane, rows, IH, D, g.index_slot(layer),
                                 len(g.full_layers), cache.local_capacity, cache.stripe, cw, cr,
                                 cache.context_capacity, max_ctx, ws.score_stride, self.index_scale, ws.scores,
                                 ws.r_scores.offset if xf else 0, kx, native.SIG_SCORES, self.peer.status_ptr,
                                 **(dict(q_raw=ws.q_proj, q_offset=hl * g.qk_head_dim, inv_freq=self.inv_freq, rd=rd) if fold else {}),
                                 **(dict(pieces=ws.idx_pieces, lane=lane_of_rows) if lane_of_rows is not None and ws.idx_pieces is not None else {}))
            if gather and not xf:
                self._merge_scores(ws.scores[:rows], max_ctx)
            native.topk_select(ws.scores, row_pos, rows, cache.context_capacity, ws.score_stride, g.index_top_k, cache.stripe,
                               cw, cr, ws.sel_global, ws.sel_local, ws.sel_counts, kx, native.SIG_SCORES)
            if self.trace is not None:
                self.trace.setdefault("sel_global", {})[layer] = ws.sel_global[:rows].clone()
                self.trace.setdefault("scores", {})[layer] = ws.scores[:rows].clone()

        if forked is not None:
            self._join(forked)
        if not decode and not gather and self.prefill_rows_attention:
            # many rows, every key local: one kernel, running softmax per (row, 16 heads), bf16 output, no partials
            native.sparse_mla_rows(ws.q_full, state.kv_cache, ws.sel_local, ws.sel_counts, row_lane, rows, ht, L, rd, layer, g.num_layers,
                                   cache.local_capacity, g.index_top_k, self.softmax_scale, ws.o_lat, self.peer.status_ptr)
        # decode with every key local and all rows in one pass: the merge and the value projection share a launch
        merged_vproj = decode and not gather and rows <= ws.attn_rows and self.merge_vproj and L % 8 == 0 and L <= 512 and g.v_head_dim % 2 == 0
        # owner-local partial attention for ALL heads, in passes of attn_rows query rows
        for r0 in range(0, rows, ws.attn_rows) if (decode or gather or not self.prefill_rows_attention) else ():
            n = min(ws.attn_rows, rows - r0)
            native.sparse_mla_partial(ws.q_full[r0:], state.kv_cache, ws.sel_local[r0:], ws.sel_counts[r0:], row_lane[r0:], n, ht, L, rd,
                                      layer, g.num_layers, cache.local_capacity, g.index_top_k, ws.max_chunks, self.softmax_scale,
                                      ws.part_o, ws.part_ml, kx, native.SIG_Q if xf else -1, self.peer.status_ptr)
            if merged_vproj:
                native.attn_merge_vproj(ws.part_o, ws.part_ml, ws.sel_counts, rows, ht, L, g.index_top_k, ws.max_chunks, lw.kv_b,
                                        g.qk_nope_head_dim, ws.o_lat, ws.attn_v)
            elif not gather:
                native.attn_local_merge(ws.part_o, ws.part_ml, ws.sel_counts[r0:], n, ht, L, g.index_top_k, ws.max_chunks, ws.o_lat[r0:], hl)
            elif xf:
                native.attn_local_merge(ws.part_o, ws.part_ml, ws.sel_counts[r0:], n, ht, L, g.index_top_k, ws.max_chunks, None, hl,
                                        ws.r_xpart.offset, kx, native.SIG_ATTN)
                native.attn_final_merge(n, L, hl, ws.r_xpart.offset, ws.o_lat[r0:], kx, native.SIG_ATTN)
            else:
                self._merge_partials_nccl(ws, r0, n)
        # value projection per head, then the K-split output projection with its reduction
        if decode:
            if not merged_vproj:
                native.skinny_bf16(ws.o_lat, lw.kv_b[:, g.qk_nope_head_dim :, :], ws.attn_v, native.SK_OUT_BF16, rows=rows, N=g.v_head_dim,
                                   K=L, xs=hl * L, ws=L, os_=hl * g.v_head_dim, batch=hl, xb=L, wb=g.kv_b_rows_per_head * L, ob=g.v_head_dim)
            if fused or self.world == 1 or self.emulated_shard:
                native.skinny_bf16(ws.attn_v[:rows], lw.w_o, ws.attn_out, native.SK_OUT_ALLREDUCE_BF16, comm=kc, channel=native.CH_ATTN)
            else:
                native.skinny_bf16(ws.attn_v[:rows], lw.w_o, ws.partial, native.SK_OUT_F32)
                ws.attn_out[:rows] = self._allreduce_rows(ws.partial[:rows]).to(torch.bfloat16)
        else:
            w_v = lw.kv_b[:, g.qk_nope_head_dim :, :]  # [hl, v, L]
            v = torch.einsum("rhc,hvc->rhv", ws.o_lat[:rows], w_v).reshape(rows, hl * g.v_head_dim)
            if self.world == 1:
                self._mm(v, lw.w_o, out=ws.attn_out[:rows])
            else:
                fused_out = self._mm_allreduce(ws, v, lw.w_o)
                if fused_out is not None:
                    ws.attn_out[:rows] = fused_out
                else:
                    part = self._mm(v, lw.w_o, f32=True)
                    ws.attn_out[:rows] = self._allreduce_rows(part).to(torch.bfloat16)
        if self.trace is not None:
            self.trace.setdefault("attn_out", {})[layer] = ws.attn_out[:rows].clone()
            self.trace.setdefault("kv_new", {})[layer] = ws.kv_new[:rows].clone()

    def select_keys_decode(self, ws: Workspace, state: DecoderState, layer: int, rows: int) -> None:
        """Indexer scores and the exact top-k of a layer with its own indexer, for the rows of a decode step whose q_b projection
        (``ws.q_proj``), head weights and index-cache row are already in place: the two launches between two stretches of the
        persistent decode kernel.  Keys of this GPU's cache only (one GPU, or a replicated cache)."""
        g, lay, cache = self.g, self.layout, self.cache
        IH, D, rd, L = g.index_heads, g.index_head_dim, g.qk_rope_head_dim, g.kv_lora_rank
        hl = lay.heads_local
        row_pos, row_lane = state.positions, state.lane_ids
        raw = native.indexer_takes_raw_query(IH, D)
        if not raw:  # head shapes the tcgen05 indexer does not take: rotate the index query with the stand-alone kernel first
            b = native.QPostArgs()
            b.q, b.q_stride = ws.q_proj.data_ptr(), ws.q_proj.stride(0)
            b.rope_table, b.inv_freq, b.row_pos = self.rope.data_ptr(), self.inv_freq.data_ptr(), row_pos.data_ptr()
            b.q_nope, b.q_full, b.q_idx = ws.q_nope.data_ptr(), ws.q_full.data_ptr(), ws.q_idx.data_ptr()
            b.heads_local, b.head_base, b.heads_total = hl, self.head_base, self.attn_heads
            b.nope, b.rd, b.L, b.IH, b.D = g.qk_nope_head_dim, rd, L, IH, D
            b.has_indexer, b.capacity = 1, cache.context_capacity
            native.q_post(b, rows)
        native.indexer_score(ws.q_idx, ws.head_w, state.index_cache, row_pos, row_lane, rows, IH, D, g.index_slot(layer),
                             len(g.full_layers), cache.local_capacity, cache.stripe, cache.world, self.cache_rank,
                             cache.context_capacity, cache.context_capacity, ws.score_stride, self.index_scale, ws.scores, 0, None,
                             native.SIG_SCORES, self.peer.status_ptr,
                             **(dict(q_raw=ws.q_proj, q_offset=hl * g.qk_head_dim, inv_freq=self.inv_freq, rd=rd) if raw else {}))
        native.topk_select(ws.scores, row_pos, rows, cache.context_capacity, ws.score_stride, g.index_top_k, cache.stripe, cache.world,
                           self.cache_rank, ws.sel_global, ws.sel_local, ws.sel_counts, None, native.SIG_SCORES)

    # NCCL baseline pieces ---------------------------------------------------------------------
    def _allgather_heads(self, q_full: torch.Tensor) -> None:
        import torch.distributed as dist

        hl = self.layout.heads_local
        mine = q_full[:, self.rank * hl : (self.rank + 1) * hl].contiguous()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        for p, part in enumerate(parts):
            q_full[:, p * hl : (p + 1) * hl] = part

    def _merge_scores(self, scores: torch.Tensor, max_ctx: int) -> None:
        """Every rank wrote only the positions it owns; combine with a masked sum (other entries zeroed first)."""
        import torch.distributed as dist

        pos = torch.arange(max_ctx, device=scores.device)
        mine = ((pos // self.cache.stripe) % self.world) == self.rank
        view = scores[:, :max_ctx]
        merged = torch.where(mine[None, :], view, torch.zeros((), device=scores.device)).contiguous()
        merged.nan_to_num_(0.0, 0.0, 0.0)
        dist.all_reduce(merged, group=self.group)
        view.copy_(merged)

    def _merge_partials_nccl(self, ws: Workspace, r0: int, n: int) -> None:
        import torch.distributed as dist

        g, hl = self.g, self.layout.heads_local
        L, ht = g.kv_lora_rank, g.attention_heads
        counts = ws.sel_counts[r0 : r0 + n, 1].clamp(0, g.index_top_k)
        chunks = (counts + native.attn_chunk() - 1) // native.attn_chunk()
        valid = torch.arange(ws.max_chunks, device=self.device)[None, :] < chunks[:, None]  # [n, chunks]
        m = torch.where(valid[:, :, None], ws.part_ml[:n, :, :, 0], torch.tensor(float("-inf"), device=self.device))
        M = m.max(dim=1).values  # [n, ht]
        wgt = torch.where(valid[:, :, None], torch.exp(m - M[:, None, :]), torch.zeros((), device=self.device))
        wgt = torch.nan_to_num(wgt, nan=0.0)
        o = (ws.part_o[:n] * wgt[..., None]).sum(dim=1)  # [n, ht, L]
        l = (torch.where(valid[:, :, None], ws.part_ml[:n, :, :, 1], torch.zeros((), device=self.device)) * wgt).sum(dim=1)
        packed = torch.cat([o, M[..., None], l[..., None]], dim=-1)  # [n, ht, L+2]
        gathered = [torch.empty_like(packed) for _ in range(self.world)]
        dist.all_gather(gathered, packed.contiguous(), group=self.group)
        allp = torch.stack(gathered)[:, :, self.rank * hl : (self.rank + 1) * hl]  # [world, n, hl, L+2]
        Mg = allp[..., L].max(dim=0).values
        wg = torch.nan_to_num(torch.exp(allp[..., L] - Mg[None]), nan=0.0)
        num = (allp[..., :L] * wg[..., None]).sum(dim=0)
        den = (allp[..., L + 1] * wg).sum(dim=0)
        out = torch.where(den[..., None] > 0, num / den[..., None], torch.zeros((), device=self.device))
        ws.o_lat[r0 : r0 + n] = out.to(torch.bfloat16)

    # ------------------------------------------------------------------------------ MLP
    def _mlp(self, ws: Workspace, lw: LayerWeights, layer: int, rows: int, decode: bool):
        g, lay = self.g, self.layout
        H = g.hidden_size
        fused = ws.peer_visible
        kc = self.peer.comm if fused else None
        x = ws.x[:rows]
        if g.mlp_layer_types[layer] == "dense":
            if decode:
                native.skinny_bf16_swiglu(x, lw.dense_gate, lw.dense_up, ws.dense_act)
                if fused or self.world == 1 or self.emulated_shard:
                    native.skinny_bf16(ws.dense_act[:rows], lw.dense_down, ws.update, native.SK_OUT_ALLREDUCE_BF16, comm=kc,
                                       channel=native.CH_MLP)
                else:
                    native.skinny_bf16(ws.dense_act[:rows], lw.dense_down, ws.partial, native.SK_OUT_F32)
                    ws.update[:rows] = self._allreduce_rows(ws.partial[:rows]).to(torch.bfloat16)
            else:
                act = self._swiglu(self._mm(x, lw.dense_gate), self._mm(x, lw.dense_up))
                if self.world == 1:
                    self._mm(act, lw.dense_down, out=ws.update[:rows])
                else:
                    fused_out = self._mm_allreduce(ws, act, lw.dense_down)
                    if fused_out is not None:
                        ws.update[:rows] = fused_out
                    else:
                        ws.update[:rows] = self._allreduce_rows(self._mm(act, lw.dense_down, f32=True)).to(torch.bfloat16)
            return
        # whole experts: this GPU's `el` experts from `ebase`, full width; sliced: I columns of every expert
        tk, I, E = g.routed_top_k, lay.moe_cols_local, g.num_routed_experts
        el, ebase = lay.experts_resident, lay.expert_base
        one_launch = decode and lay.sliced and (fused or self.world == 1 or self.emulated_shard) and tk <= 8 and I % 64 == 0 and H % 16 == 0
        forked = None
        if decode and self.side is not None:
            # the shared expert needs only the normalized hidden state: it runs on the side stream while the main stream
            # goes through router -> top-8 -> routed gate/up -> routed down; the combine joins the two
            forked = self._fork()
            with torch.cuda.stream(self.side):
                native.skinny_bf16_swiglu(x, lw.shared_gate, lw.shared_up, ws.act_shared)
                native.skinny_bf16(ws.act_shared[:rows], lw.shared_down, ws.partial, native.SK_OUT_F32)
        self._linear_f32(x, lw.router_w, ws.router_logits, decode)
        native.router_topk(ws.router_logits[:rows], lw.router_bias, tk, ws.topk_ids, ws.topk_w)
        if self.trace is not None:
            self.trace.setdefault("topk_ids", {})[layer] = ws.topk_ids[:rows].clone()
            self.trace.setdefault("topk_w", {})[layer] = ws.topk_w[:rows].clone()
        sort_kernel = self.route_sort_kernel and el <= 256 and ws.topk_ids[:rows].is_contiguous()
        # A chunk with few routes per expert (a short prompt: 200 rows x 8 routes over 256 experts are ~6 each) is bound by streaming
        # and decoding the weights of nearly every expert once: the tensor-core GEMV kernels on 8-route tiles do that at a third of
        # the instructions per weight of the grouped GEMM, whose 128-row tiles would be 95 % padding.  Measured on one rank's shard
        # of eight: 0.93 ms less per 3 MoE layers at 200 rows, 0.46 ms less at 320, level at 512; taken below a mean of 12 routes.
        few_per_expert = self.few_routes_gemv and sort_kernel and rows * tk < self.few_routes_limit * E
        if not decode and not few_per_expert and rows * tk >= 128 and H % 16 == 0 and I % 16 == 0:
            # many rows: expert-sorted routes through the tcgen05 grouped GEMM (FP8 decoded inside the kernel)
            if sort_kernel:
                tiles_t, n_tiles, perm = ws.route_buffers(rows * tk, el)
                native.route_sort128(ws.topk_ids[:rows], ebase, el, tiles_t, n_tiles, perm)
            else:
                tiles_t, n_tiles, perm = self._route_tiles128(ws.topk_ids[:rows], ebase, el)
            xs, acts = ws.sorted_buffers(rows * tk, H, I)
            native.gather_rows(x, perm, tk, xs)
            native.moe_grouped_fp8w(xs, lw.exp_gate_bits, lw.exp_up_bits, lw.exp_gate_scale, lw.exp_up_scale, tiles_t, n_tiles, 0, acts,
                                    status=self.peer.status_ptr)
            native.moe_grouped_fp8w(acts, lw.exp_down_bits, None, lw.exp_down_scale, None, tiles_t, n_tiles, 1, ws.dw, perm=perm,
                                    route_weight=ws.topk_w, status=self.peer.status_ptr)
        else:
            if decode:
                tile_expert, tile_routes, n_tiles, tiles, rt = ws.topk_ids, None, None, rows * tk, 1
            elif sort_kernel:
                tile_expert, tile_routes, n_tiles, scratch = ws.route_buffers8(rows * tk, el)
                native.route_sort8(ws.topk_ids[:rows], ebase, el, tile_expert, tile_routes, n_tiles, scratch)
                tiles, rt = tile_expert.shape[0], 8
            else:
                tile_expert, tile_routes, n_tiles, tiles, rt = self._route_tiles(ws.topk_ids[:rows], E)
            native.moe_gateup_fp8(x, tk, tile_expert, tile_routes, n_tiles, tiles, rt, lw.exp_gate_bits, lw.exp_up_bits,
                                  lw.exp_gate_scale, lw.exp_up_scale, ebase, ws.act)
            if not one_launch:
                native.moe_down_fp8(ws.act, ws.topk_w, tile_expert, tile_routes, n_tiles, tiles, rt, lw.exp_down_bits, lw.exp_down_scale,
                                    ebase, ws.dw)
        if decode:
            if forked is not None:
                self._join(forked)
            else:
                native.skinny_bf16_swiglu(x, lw.shared_gate, lw.shared_up, ws.act_shared)
                native.skinny_bf16(ws.act_shared[:rows], lw.shared_down, ws.partial, native.SK_OUT_F32)
            shared_partial = ws.partial
        else:
            act = self._swiglu(self._mm(x, lw.shared_gate), self._mm(x, lw.shared_up))
            library_reduce = not (fused or self.world == 1 or self.emulated_shard)
            # with a library all-reduce ahead the shared partial sums are produced where they will travel from
            both = ws.partial_pair(rows, H) if library_reduce else None
            shared_partial = self._mm(act, lw.shared_down, f32=True, out=both[1] if both is not None else None)
        if one_launch:
            native.moe_down_combine(ws.act, ws.topk_w, ws.topk_ids, lw.exp_down_bits, lw.exp_down_scale, shared_partial, rows, tk,
                                    g.routed_scaling_factor, ws.update, kc, native.CH_MLP)
        elif fused or self.world == 1 or self.emulated_shard:
            native.moe_combine(ws.dw, ws.topk_ids, shared_partial, rows, tk, H, ebase, el, g.routed_scaling_factor, False, ws.update,
                               None, kc, native.CH_MLP)
        else:
            # library all-reduce (the NCCL baseline, and prefill chunks): both partial sums travel as one buffer, one kernel finishes
            if decode:  # (the NCCL baseline of the decode step keeps its shared partial sums in the workspace)
                both = ws.partial_pair(rows, H)
                both[1].copy_(shared_partial[:rows])
            native.moe_combine(ws.dw, ws.topk_ids, None, rows, tk, H, ebase, el, g.routed_scaling_factor, False, None, both[0])
            self._allreduce_rows(both)
            native.moe_finish(both[0], both[1], g.routed_scaling_factor, ws.update[:rows])

    def _route_tiles128(self, topk_ids: torch.Tensor, ebase: int, el: int):
        """Sort this GPU's routes by expert and cut them into 128-route tiles (device-side, no host sync).

        Returns ``tiles [max_tiles, 4]`` (first sorted row, end row, local expert, 0), ``n_tiles [1]`` and
        ``perm [routes]`` (sorted position -> route id ``row * top_k + slot``; -1 past this GPU's routes).
        """
        dev = topk_ids.device
        ids = topk_ids.reshape(-1).long() - ebase
        P = ids.numel()
        key = torch.where((ids >= 0) & (ids < el), ids, torch.full_like(ids, el))  # other GPUs' routes sort last
        order = torch.argsort(key, stable=True)
        counts = torch.bincount(key, minlength=el + 1)[:el]
        n_local = counts.sum()
        perm = torch.where(torch.arange(P, device=dev) < n_local, order, torch.full_like(order, -1)).to(torch.int32).contiguous()
        tiles_per = (counts + 127) // 128
        tile_end = torch.cumsum(tiles_per, 0)
        route_start = torch.cumsum(counts, 0) - counts
        max_tiles = P // 128 + el
        t = torch.arange(max_tiles, device=dev)
        expert = torch.searchsorted(tile_end, t, right=True).clamp(max=el - 1)
        within = t - (tile_end[expert] - tiles_per[expert])
        valid = t < tile_end[-1]
        row0 = route_start[expert] + within * 128
        row_end = route_start[expert] + counts[expert]
        zero = torch.zeros_like(t)
        tiles = torch.stack([torch.where(valid, row0, zero), torch.where(valid, row_end, zero), torch.where(valid, expert, zero), zero], dim=1)
        return tiles.to(torch.int32).contiguous(), tile_end[-1:].to(torch.int32).contiguous(), perm

    def _route_tiles(self, topk_ids: torch.Tensor, E: int):
        """Group routes by expert into tiles of 8 (device-side, no host sync)."""
        ids = topk_ids.reshape(-1).long()
        P = ids.numel()
        order = torch.argsort(ids, stable=True)
        counts = torch.bincount(ids, minlength=E)
        tiles_per = (counts + 7) // 8
        tile_end = torch.cumsum(tiles_per, 0)
        route_start = torch.cumsum(counts, 0) - counts
        max_tiles = P // 8 + E
        t = torch.arange(max_tiles, device=ids.device)
        expert = torch.searchsorted(tile_end, t, right=True).clamp(max=E - 1)
        within = t - (tile_end[expert] - tiles_per[expert])
        valid_tile = t < tile_end[-1]
        slot = within[:, None] * 8 + torch.arange(8, device=ids.device)[None, :]
        ok = valid_tile[:, None] & (slot < counts[expert][:, None])
        src = (route_start[expert][:, None] + slot).clamp(max=P - 1)
        routes = torch.where(ok, order[src], torch.full_like(src, -1)).to(torch.int32).contiguous()
        tile_expert = torch.where(valid_tile, expert, torch.full_like(expert, -1)).to(torch.int32).contiguous()
        n_tiles = tile_end[-1:].to(torch.int32).contiguous()
        return tile_expert, routes, n_tiles, max_tiles, 8

    # ------------------------------------------------------------------------------ whole model
    def run_rows(self, ws: Workspace, state: DecoderState, tokens: torch.Tensor, row_pos: torch.Tensor, row_lane: torch.Tensor,
                 row_active, rows: int, *, decode: bool, max_ctx: int, head_rows: slice | None = None, head: str = "logits",
                 lane_of_rows: int | None = None):
        """Push ``rows`` token rows through the decoder.

        ``lane_of_rows``: the cache lane that EVERY row belongs to (a prefill chunk of one chat), when the caller knows it; it
        lets the indexer keep the key tiles resident while the rows stream past them.

        ``head='logits'`` returns the bf16 logits of ``head_rows`` (this rank's vocabulary slice).  ``head='argmax'``
        (decode) fuses the greedy reduction into the lm_head kernel: the packed best candidate of every row lands in
        ``ws.local_best`` and ``None`` is returned; ``sample`` then finishes the step.
        """
        g = self.g
        native.embed_rows(tokens, self.w.embed, ws.residual, self.peer.status_ptr)
        update = None
        mark = torch.cuda.nvtx.range_push if self.nvtx else (lambda name: None)
        done = torch.cuda.nvtx.range_pop if self.nvtx else (lambda: None)
        for i, lw in enumerate(self.w.layers):
            mark(f"layer{i}.attention.{g.indexer_types[i]}")  # region names for profilers (GLM_B200_NVTX=1)
            native.add_rmsnorm(update, ws.residual[:rows], lw.input_norm, ws.x, g.rms_norm_eps)
            self._attention(ws, lw, i, rows, row_pos, row_lane, row_active, state, decode, max_ctx, lane_of_rows)
            done()
            mark(f"layer{i}.mlp.{g.mlp_layer_types[i]}")
            native.add_rmsnorm(ws.attn_out, ws.residual[:rows], lw.post_norm, ws.x, g.rms_norm_eps)
            self._mlp(ws, lw, i, rows, decode)
            done()
            update = ws.update
            if self.trace is not None:
                self.trace.setdefault("update", {})[i] = ws.update[:rows].clone()
        native.add_rmsnorm(update, ws.residual[:rows], self.w.final_norm, ws.x, g.rms_norm_eps)
        hs = head_rows or slice(0, rows)
        xh = ws.x[hs]
        n = xh.shape[0]
        if head == "argmax":
            native.skinny_bf16(xh, self.w.lm_head, ws.local_best, native.SK_OUT_ARGMAX, comm=self.peer.comm,
                               channel=self.rank * self.layout.vocab_local, os_=0)
            return None
        if n <= native.MAX_ROWS:
            native.skinny_bf16(xh, self.w.lm_head, ws.logits, native.SK_OUT_BF16)
        else:
            self._mm(xh, self.w.lm_head, out=ws.logits[:n])
        return ws.logits[:n]

    def sample(self, ws: Workspace, state: DecoderState, logits: torch.Tensor, rows: int, row_active, *, advance: int,
               tokens_out=None, positions=None, out=None) -> None:
        """Greedy sampling with the cross-GPU candidate exchange.

        ``advance`` bit 0 stores the token into ``tokens_out`` (default: the lane registers), bit 1 increments the
        positions.  The token also goes to ``out`` (``[rows]`` int32) or, by default, to the ``out_tokens`` ring.
        """
        lay = self.layout
        fused = ws.peer_visible
        kc = self.peer.comm if fused else None
        local_best = None
        if logits is None:
            local_best = ws.local_best  # filled by the lm_head kernel in argmax mode
            if self.world > 1 and not fused and not self.emulated_shard:
                ws.cand[0, :rows] = ws.local_best[:rows]
                ws.local_best.zero_()
                local_best = None
        else:
            native.argmax_rows(logits, rows, lay.vocab_local, self.rank * lay.vocab_local, ws.cand, ws.r_cand.offset if fused else 0,
                               kc, native.SIG_SAMPLE, self.peer.status_ptr)
        cand = ws.cand
        if self.world > 1 and not fused and not self.emulated_shard:
            import torch.distributed as dist

            mine = ws.cand[0, :rows].contiguous()  # without a PeerComm the kernel writes set 0
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            cand = torch.stack(parts).contiguous()
        tokens = tokens_out if tokens_out is not None else state.tokens
        pos = positions if positions is not None else state.positions
        if out is None:
            out, counter, ring = state.out_tokens, state.step_counter, RING
        else:
            counter, ring = None, 1
        native.step_finalize(cand, self.world, rows, row_active, tokens, pos, out, counter, ring, advance, kc, native.SIG_SAMPLE,
                             local_best=local_best, cand_offset=ws.r_cand.offset if fused else 0)
