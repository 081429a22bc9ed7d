"""The decode step through the persistent kernel (``csrc/decode_mega.cu``).

``MegaDecoder`` owns what the persistent kernel needs beyond the decode workspace: the per-layer pointer table in
device memory, the two residual buffers the add + RMSNorm prologues alternate between, the grid-barrier words and the
argument block.  ``step`` issues one decode step as a handful of launches: a *stretch* of the persistent kernel runs
from the first phase of a layer to the phase before the next layer with its own indexer needs its selection; that
layer's tcgen05 indexer and cluster top-k run as the kernels they are; the next stretch picks up at the attention
phase.  GLM-5.3 has 21 such layers, so a step is 22 stretches + 42 indexer launches instead of ~1,360 launches.

Parity: the stretch list replaces the launch sequence of reference ``glm_tpu/models/glm_moe_dsa/model.py:86-135``
(one XLA program per step there).
"""

from __future__ import annotations

import ctypes as C

import torch

from glm_tpu_b200.ops import native

# phases of a layer, and of the head (layer index == number of layers); see csrc/decode_mega.cu
QKV_A, Q_B, ABSORB, ATTN, MERGE, VPROJ, OPROJ, MLP_A, MLP_B, MOE_DOWN, COMBINE = range(1, 12)
HEAD_LOGITS, HEAD_FINALIZE = 1, 2

_LAYER_POINTERS = (
    "input_norm", "post_norm", "w_qkv_a", "q_a_norm", "kv_a_norm", "w_q_b", "kv_b", "w_o", "k_norm_w", "k_norm_b",
    "dense_gate", "dense_up", "dense_down", "router_w", "router_bias", "exp_gate", "exp_up", "exp_down",
    "exp_gate_scale", "exp_up_scale", "exp_down_scale", "shared_gate", "shared_up", "shared_down",
)
_ARG_POINTERS = (
    "layers", "embed", "final_norm", "lm_head", "rope_table", "inv_freq", "tokens", "positions", "active", "lane_ids",
    "out_tokens", "step_counter", "kv_cache", "index_cache", "residual_a", "residual_b", "x", "update", "attn_out", "proj_a",
    "q_resid", "head_w", "kv_new", "idx_key_new", "q_proj", "q_full", "sel_local", "sel_counts", "part_o", "part_ml", "o_lat",
    "attn_v", "router_logits", "topk_ids", "topk_w", "act_shared", "dense_act", "partial", "act", "dw", "local_best", "cand",
    "bar", "status", "timeline",
)
_ARG_INT64 = ("proj_stride", "q_stride", "act_shared_stride", "dense_act_stride", "cand_offset", "timeline_cap", "prefetch_cap")
_ARG_INTS = (
    "rows", "H", "Q", "L", "rd", "nope", "vdim", "D", "IH",
    "heads_local", "head_base", "heads_total", "E", "top_k", "I", "experts_local", "expert_base", "shared_cols", "dense_cols",
    "vocab", "vocab_local", "vocab_base", "num_layers", "n_full_layers", "index_top_k", "max_chunks",
    "local_cap", "stripe", "cache_world", "cache_rank", "capacity", "ring", "compat_ksplit",
)
_ARG_FLOATS = ("eps", "key_eps", "head_scale", "softmax_scale", "routed_scale")


class MegaLayer(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in _LAYER_POINTERS] + [
        ("full", C.c_int), ("dense", C.c_int), ("index_slot", C.c_int), ("n_qkv_a", C.c_int), ("n_q_b", C.c_int), ("pad_", C.c_int),
    ]


class MegaArgs(C.Structure):
    _fields_ = (
        [(name, C.c_void_p) for name in _ARG_POINTERS]
        + [(name, C.c_int64) for name in _ARG_INT64]
        + [(name, C.c_int) for name in _ARG_INTS]
        + [("bar_limit", C.c_uint32)]
        + [(name, C.c_float) for name in _ARG_FLOATS]
        + [("layer0", C.c_int), ("phase0", C.c_int), ("layer1", C.c_int), ("phase1", C.c_int)]
        + [("comm", native.PeerComm)]
    )


def _check_layout(lib) -> None:
    lib.glmb_mega_args_sizeof.restype = C.c_size_t
    lib.glmb_mega_layer_sizeof.restype = C.c_size_t
    offsets = (C.c_size_t * 6)()
    lib.glmb_mega_args_offsets(offsets)
    mine = (MegaArgs.proj_stride.offset, MegaArgs.rows.offset, MegaArgs.eps.offset, MegaArgs.comm.offset, MegaLayer.full.offset,
            MegaArgs.timeline_cap.offset)
    if lib.glmb_mega_args_sizeof() != C.sizeof(MegaArgs) or lib.glmb_mega_layer_sizeof() != C.sizeof(MegaLayer) or tuple(offsets) != mine:
        raise RuntimeError("MegaArgs / MegaLayer layout differs between Python and the CUDA library")


def _ptr(t) -> int | None:
    return None if t is None else int(t.data_ptr())


class MegaDecoder:
    """One decode step of ``model`` over the rows of ``ws`` (the decode workspace) as stretches of the persistent kernel."""

    def __init__(self, model, ws, state, *, compat_ksplit: bool | None = None, prefetch_bytes: int | None = None, mode: str = "phases"):
        if mode not in ("phases", "persistent"):
            raise ValueError("mode is 'phases' (a kernel per phase) or 'persistent' (stretches of one cooperative kernel)")
        if compat_ksplit is None:
            # a kernel per phase keeps the K split and the grids of the stand-alone projection kernels (many small CTAs, every
            # byte of a table requested at once); the persistent grid has a fixed 296 CTAs and balances the rows over them
            compat_ksplit = mode == "phases"
        self.mode = mode
        self.model, self.ws, self.state = model, ws, state
        lib = native.lib()
        _check_layout(lib)
        self._lib = lib
        g, lay, cache, dev = model.g, model.layout, model.cache, model.device
        rows = ws.rows
        self.rows = rows
        # per-layer pointer table
        table = (MegaLayer * g.num_layers)()
        alias = {"exp_gate": "exp_gate_bits", "exp_up": "exp_up_bits", "exp_down": "exp_down_bits"}
        for i, lw in enumerate(model.w.layers):
            entry = table[i]
            for name in _LAYER_POINTERS:
                setattr(entry, name, _ptr(getattr(lw, alias.get(name, name))))
            entry.full = int(g.indexer_types[i] == "full")
            entry.dense = int(g.mlp_layer_types[i] == "dense")
            entry.index_slot = g.index_slot(i) if entry.full else 0
            entry.n_qkv_a = lw.w_qkv_a.shape[0]
            entry.n_q_b = lw.w_q_b.shape[0]
        self._table = table
        raw = bytes(table) if g.num_layers else b"\0" * C.sizeof(MegaLayer)
        self.layer_table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        H = g.hidden_size
        self.residual_a = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        self.residual_b = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
        lib.glmb_mega_barrier_sizeof.restype = C.c_size_t
        self.barrier = torch.zeros(int(lib.glmb_mega_barrier_sizeof()) // 4, dtype=torch.int32, device=dev)
        a = MegaArgs()
        fused = ws.peer_visible
        pointers = dict(
            layers=self.layer_table, embed=model.w.embed, final_norm=model.w.final_norm, lm_head=model.w.lm_head, rope_table=model.rope,
            inv_freq=model.inv_freq, tokens=state.tokens, positions=state.positions, active=state.active, lane_ids=state.lane_ids,
            out_tokens=state.out_tokens, step_counter=state.step_counter, kv_cache=state.kv_cache, index_cache=state.index_cache,
            residual_a=self.residual_a, residual_b=self.residual_b, x=ws.x, update=ws.update, attn_out=ws.attn_out, proj_a=ws.proj_a,
            q_resid=ws.q_resid, head_w=ws.head_w, kv_new=ws.kv_new, idx_key_new=ws.idx_key_new, q_proj=ws.q_proj, q_full=ws.q_full,
            sel_local=ws.sel_local, sel_counts=ws.sel_counts, part_o=ws.part_o, part_ml=ws.part_ml, o_lat=ws.o_lat, attn_v=ws.attn_v,
            router_logits=ws.router_logits, topk_ids=ws.topk_ids, topk_w=ws.topk_w, act_shared=ws.act_shared, dense_act=ws.dense_act,
            partial=ws.partial, act=ws.act, dw=ws.dw, local_best=ws.local_best, cand=ws.cand, bar=self.barrier,
        )
        for name, tensor in pointers.items():
            setattr(a, name, _ptr(tensor))
        a.status = model.peer.status_ptr
        a.proj_stride, a.q_stride = ws.proj_a.stride(0), ws.q_proj.stride(0)
        a.act_shared_stride, a.dense_act_stride = ws.act_shared.stride(0), ws.dense_act.stride(0)
        a.cand_offset = ws.r_cand.offset if fused else 0
        a.rows, a.H, a.Q, a.L, a.rd = rows, H, g.q_lora_rank, g.kv_lora_rank, g.qk_rope_head_dim
        a.nope, a.vdim, a.D, a.IH = g.qk_nope_head_dim, g.v_head_dim, g.index_head_dim, g.index_heads
        a.heads_local, a.head_base, a.heads_total = lay.heads_local, model.head_base, model.attn_heads
        a.E, a.top_k, a.I = g.num_routed_experts, g.routed_top_k, g.moe_intermediate_size
        a.experts_local, a.expert_base = lay.experts_local, model.rank * lay.experts_local
        a.shared_cols, a.dense_cols = lay.shared_cols_local, lay.dense_cols_local
        a.vocab, a.vocab_local, a.vocab_base = g.vocab_size, lay.vocab_local, model.rank * lay.vocab_local
        a.num_layers, a.n_full_layers, a.index_top_k, a.max_chunks = g.num_layers, len(g.full_layers), g.index_top_k, ws.max_chunks
        a.local_cap, a.stripe, a.cache_world, a.cache_rank = cache.local_capacity, cache.stripe, cache.world, model.cache_rank
        a.capacity, a.ring, a.compat_ksplit = cache.context_capacity, state.out_tokens.shape[0], int(compat_ksplit)
        a.bar_limit = min(4 * max(1, model.peer.wait_limit), 0xFFFFFFFF)
        if prefetch_bytes is None:
            import os

            prefetch_bytes = int(os.environ.get("GLM_B200_MEGA_PREFETCH", str(24 << 20)))
        a.prefetch_cap = max(0, int(prefetch_bytes))  # per weight table, requested into the L2 a few phases ahead; 0: off
        self.timeline = None
        a.eps, a.key_eps, a.head_scale = g.rms_norm_eps, cache.dsa.key_norm_eps, model.head_scale
        a.softmax_scale, a.routed_scale = model.softmax_scale, g.routed_scaling_factor
        comm = model.peer.comm if fused else None
        if comm is not None:
            C.memmove(C.byref(a, MegaArgs.comm.offset), C.byref(comm), C.sizeof(native.PeerComm))
        else:
            a.comm.world, a.comm.rank, a.comm.status = 1, 0, model.peer.status_ptr
        self.args = a
        self._device_args = torch.zeros(C.sizeof(MegaArgs), dtype=torch.uint8, device=dev)
        self._uploaded = None
        self.supported_code = int(lib.glmb_mega_supported(C.byref(a)))
        if model.world > 1 and not fused and not getattr(model, "emulated_shard", False):
            self.supported_code = self.supported_code or 100  # the library-collective baseline keeps the per-kernel path
        if lay.sliced and lay.world > 1:
            self.supported_code = self.supported_code or 101  # column-sliced experts exist in the per-kernel path only
        self.launches = 0

    # ------------------------------------------------------------------ per-phase timing
    def enable_timeline(self, entries: int = 8192) -> None:
        """Make CTA 0 stamp the global timer after every phase (with its barrier) into a device buffer; for measurements only."""
        self.timeline = torch.zeros(1 + 2 * entries, dtype=torch.int64, device=self.model.device)
        self.args.timeline, self.args.timeline_cap = int(self.timeline.data_ptr()), entries

    def read_timeline(self, reset: bool = True) -> list[tuple[int, int, float]]:
        """``[(layer, code, microseconds since the previous stamp), ...]``.  code 0: a stretch began; code = phase once the
        phase's grid barrier is passed; phase | 0x80 when CTA 0 finished its own work of the phase (so the next entry is the
        wait for the slowest CTA plus the barrier); phase | step << 16 for a step inside a phase.  Synchronizes."""
        torch.cuda.synchronize(self.model.device)
        host = self.timeline.cpu().tolist()
        n = min(host[0], (len(host) - 1) // 2)
        out, prev = [], None
        for i in range(n):
            code, t = host[1 + 2 * i], host[2 + 2 * i]
            out.append(((code >> 8) & 255, (code & 255) | (code >> 16 << 16), 0.0 if prev is None else (t - prev) / 1e3))
            prev = t
        if reset:
            self.timeline.zero_()
        return out

    def barrier_nanoseconds(self, iters: int = 2000, variant: int = 1) -> float:
        """Device time of one grid barrier of the persistent kernel's grid, measured over ``iters`` back-to-back barriers."""
        ns = torch.zeros(1, dtype=torch.int64, device=self.model.device)
        native._check(self._lib.glmb_mega_barrier_bench(C.c_void_p(self.barrier.data_ptr()), int(iters), int(variant), C.c_uint32(self.args.bar_limit),
                                                        C.c_void_p(self.model.peer.status_ptr), C.c_void_p(ns.data_ptr()), native._stream()),
                      "mega_barrier_bench")
        torch.cuda.synchronize(self.model.device)
        return float(ns.item()) / iters

    @property
    def supported(self) -> bool:
        return self.supported_code == 0

    def grid(self) -> int:
        return int(self._lib.glmb_mega_grid(self.rows))

    def _sync_args(self) -> None:
        """The kernel reads its argument block from device memory: upload it whenever the host copy has changed."""
        raw = bytes(self.args)
        if raw != self._uploaded:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the argument block of the persistent decode kernel changed during a graph capture")
            self._device_args.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
            torch.cuda.synchronize(self.model.device)
            self._uploaded = raw

    def stretch(self, first: tuple[int, int], last: tuple[int, int]) -> None:
        """Launch the persistent kernel over the phases ``first .. last`` (``(layer, phase)`` pairs, both inclusive)."""
        self._sync_args()
        if native._exchanges is not None and self.args.comm.world > 1:
            g, grid = self.model.g, self.grid()
            for layer in range(first[0], last[0] + 1):
                head = layer >= g.num_layers
                lo = first[1] if layer == first[0] else 1
                hi = last[1] if layer == last[0] else (HEAD_FINALIZE if head else COMBINE)
                for ph in range(lo, hi + 1):
                    self._note_exchange(layer, ph, grid)
        native._check(self._lib.glmb_mega_decode(C.byref(self.args), C.c_void_p(self._device_args.data_ptr()), first[0], first[1], last[0], last[1],
                                                 native._stream()), "mega_decode")

    def _note_exchange(self, layer: int, phase: int, persistent_grid: int = 0) -> None:
        """Tell the collective-plan recorder what this phase exchanges between the GPUs."""
        if native._exchanges is None or self.args.comm.world <= 1:
            return
        entry = C.byref(self._table[layer]) if layer < self.model.g.num_layers else None
        out = (C.c_int * 4)()
        native._check(self._lib.glmb_mega_phase_exchange(C.byref(self.args), entry, layer, phase, persistent_grid, out), "mega_phase_exchange")
        if out[0] == 1:
            native._exchanges.append({"kind": "allreduce", "channel": out[1], "ctas": out[2], "floats_per_cta": out[3], "op": f"phase{phase}"})
        elif out[0] == 2:
            native._exchanges.append({"kind": "signal", "signal": out[1], "op": f"phase{phase}"})

    def phase(self, layer: int, phase: int) -> None:
        """Launch one phase as a kernel of its own (``layer == num_layers``: the head)."""
        self._note_exchange(layer, phase)
        entry = C.byref(self._table[layer]) if layer < self.model.g.num_layers else None
        native._check(self._lib.glmb_mega_phase(C.byref(self.args), entry, layer, phase, native._stream()), "mega_phase")

    def plan(self) -> list[tuple]:
        """The launch list of one step, in order: ``("stretch", first, last)`` (persistent mode) or ``("phase", layer, phase)``
        entries, and ``("indexer", layer)`` where a layer computes its own selection."""
        g = self.model.g
        if self.mode == "phases":
            out = []
            for i in range(g.num_layers):
                dense = g.mlp_layer_types[i] == "dense"
                for ph in range(QKV_A, COMBINE + 1):
                    if dense and ph in (MOE_DOWN, COMBINE):
                        continue
                    out.append(("phase", i, ph))
                    if ph == ABSORB and g.indexer_types[i] == "full":
                        out.append(("indexer", i))
            out += [("phase", g.num_layers, HEAD_LOGITS), ("phase", g.num_layers, HEAD_FINALIZE)]
            return out
        out, start = [], (0, QKV_A)
        for i in range(g.num_layers):
            if g.indexer_types[i] == "full":
                out.append(("stretch", start, (i, ABSORB)))
                out.append(("indexer", i))
                start = (i, ATTN)
        out.append(("stretch", start, (g.num_layers, HEAD_FINALIZE)))
        return out

    def step(self) -> None:
        """Enqueue one decode step on the current stream (token, position and sequence registers live on the device)."""
        for entry in self.plan():
            if entry[0] == "stretch":
                self.stretch(entry[1], entry[2])
            elif entry[0] == "phase":
                self.phase(entry[1], entry[2])
            else:
                self.model.select_keys_decode(self.ws, self.state, entry[1], self.rows)
