"""ctypes binding of ``libglmb200.so`` (the hand-written sm_100a kernels).

The library is built in-tree by ``glm_tpu_b200.csrc.build`` and loaded with ``ctypes`` (it links only the
CUDA runtime).  Every wrapper takes torch CUDA tensors, passes raw device pointers plus the current torch
stream, and raises on a non-zero return code.  There is no fallback: if the library is missing or a launch
fails on a GPU machine the call raises.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libglmb200.so"
MAX_WORLD = 8
MAX_ROWS = 8

SK_OUT_F32, SK_OUT_BF16, SK_OUT_ALLREDUCE_BF16, SK_OUT_ARGMAX = 0, 1, 2, 3
STATUS_WAIT_TIMEOUT, STATUS_BAD_INDEX, STATUS_NONFINITE, STATUS_BAD_SHAPE = 1, 2, 4, 8

# signals (producer -> consumer exchanges) and all-reduce channels used by the model
SIG_Q, SIG_SCORES, SIG_ATTN, SIG_SAMPLE, SIG_GEMM, SIG_TEST = 0, 1, 2, 3, 4, 15
CH_ATTN, CH_MLP = 0, 1


class PeerComm(C.Structure):
    _fields_ = [
        ("world", C.c_int),
        ("rank", C.c_int),
        ("wait_limit", C.c_uint32),
        ("protocol", C.c_uint32),
        ("status", C.c_void_p),
        ("seq", C.c_void_p),
        ("data", C.c_void_p * MAX_WORLD),
        ("flags", C.c_void_p * MAX_WORLD),
    ]


class QkvPostArgs(C.Structure):
    _fields_ = [
        ("proj", C.c_void_p), ("proj_stride", C.c_int64),
        ("q_norm_w", C.c_void_p), ("kv_norm_w", C.c_void_p), ("rope_table", C.c_void_p), ("inv_freq", C.c_void_p),
        ("k_norm_w", C.c_void_p), ("k_norm_b", C.c_void_p),
        ("row_pos", C.c_void_p), ("row_lane", C.c_void_p), ("row_active", C.c_void_p),
        ("q_resid", C.c_void_p), ("kv_new", C.c_void_p), ("kv_cache", C.c_void_p), ("index_cache", C.c_void_p),
        ("head_w", C.c_void_p), ("idx_key_new", C.c_void_p),
        ("Q", C.c_int), ("L", C.c_int), ("rd", C.c_int), ("D", C.c_int), ("IH", C.c_int),
        ("has_indexer", C.c_int),
        ("layer", C.c_int), ("layers", C.c_int), ("index_slot", C.c_int), ("full_layers", C.c_int), ("local_cap", C.c_int),
        ("stripe", C.c_int), ("world", C.c_int), ("rank", C.c_int), ("capacity", C.c_int),
        ("eps", C.c_float), ("key_eps", C.c_float), ("head_scale", C.c_float),
        ("status", C.c_void_p),
    ]


class QPostArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_stride", C.c_int64),
        ("rope_table", C.c_void_p), ("inv_freq", C.c_void_p), ("row_pos", C.c_void_p),
        ("q_nope", C.c_void_p), ("q_full", C.c_void_p), ("q_idx", C.c_void_p),
        ("heads_local", C.c_int), ("head_base", C.c_int), ("heads_total", C.c_int), ("nope", C.c_int), ("rd", C.c_int),
        ("L", C.c_int), ("IH", C.c_int), ("D", C.c_int), ("has_indexer", C.c_int), ("capacity", C.c_int),
    ]


_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m glm_tpu_b200.csrc.build`")
        _lib = C.CDLL(str(LIB_PATH))
        _lib.glmb_peer_ar_bytes.restype = C.c_size_t
        _lib.glmb_peer_comm_sizeof.restype = C.c_size_t
        _lib.glmb_peer_data.restype = C.c_void_p
        _lib.glmb_peer_status_ptr.restype = C.c_void_p
        _lib.glmb_indexer_rows_scratch_bytes.restype = C.c_int64
        if _lib.glmb_peer_comm_sizeof() != C.sizeof(PeerComm):
            raise RuntimeError("PeerComm layout differs between Python and the CUDA library")
        import os

        if os.environ.get("GLM_B200_PDL", "1") == "0":  # programmatic dependent launch off: plain stream order
            _lib.glmb_set_pdl(0)
        if os.environ.get("GLM_B200_AR", "pairs") == "flags":  # all-reduce with fence + flag instead of (value, sequence) pairs
            _lib.glmb_set_ar_protocol(0)
    return _lib if _timeline is None else _TimedLib(_lib)


_timeline = None  # when a list: every launch appends (entry point, plain integer arguments, start event, end event)


class _TimedLib:
    """Brackets every entry point that launches on the current stream with a pair of CUDA events."""

    def __init__(self, inner):
        self._inner = inner

    def __getattr__(self, name):
        fn = getattr(self._inner, name)
        if not name.startswith("glmb_") or name.startswith(("glmb_peer_", "glmb_set_", "glmb_attn_chunk")):
            return fn

        def timed(*args):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            code = fn(*args)
            end.record()
            ints = tuple(a if isinstance(a, int) else a.value for a in args if isinstance(a, (int, C.c_int64, C.c_int)))
            _timeline.append((name[5:], ints, start, end))
            return code

        return timed


class kernel_timeline:
    """``with kernel_timeline() as tl:`` collects per-launch device times (eager launches only, not graph replays).

    ``tl.rows()`` synchronizes and returns ``[(entry point, integer arguments, milliseconds), ...]`` in launch order.
    """

    def __enter__(self):
        global _timeline
        self.events = _timeline = []
        return self

    def __exit__(self, *exc):
        global _timeline
        _timeline = None

    def rows(self):
        torch.cuda.synchronize()
        return [(name, ints, start.elapsed_time(end)) for name, ints, start, end in self.events]


_exchanges = None  # when a list: every launch that exchanges data between GPUs appends what it does (the collective plan)


class record_exchanges:
    """``with record_exchanges() as plan:`` collects the cross-GPU exchanges of the launches issued inside, in order:
    ``{"kind": "allreduce", "channel": c, "ctas": n, "floats_per_cta": f, "op": name}`` or ``{"kind": "signal", "signal": s,
    "op": name}``.  The runner checks the list against the rules the in-kernel protocol depends on before it captures a program."""

    def __enter__(self):
        global _exchanges
        self.plan = _exchanges = []
        return self.plan

    def __exit__(self, *exc):
        global _exchanges
        _exchanges = None


def _note_allreduce(op: str, comm, channel: int, ctas: int, floats_per_cta: int) -> None:
    if _exchanges is not None and comm is not None and comm.world > 1:
        _exchanges.append({"kind": "allreduce", "channel": int(channel), "ctas": int(ctas), "floats_per_cta": int(floats_per_cta), "op": op})


def _note_signal(op: str, comm, sig: int) -> None:
    if _exchanges is not None and comm is not None and comm.world > 1:
        _exchanges.append({"kind": "signal", "signal": int(sig), "op": op})


def _skinny_ksplit(units: int, K: int) -> int:
    """The K split the skinny kernels pick (``pick_ksplit`` in csrc/gemv.cu)."""
    ks = 1
    while ks < 8 and units * ks < 148 * 4 * 8 and K % (ks * 2 * 256) == 0 and K // (ks * 2) >= 512:
        ks *= 2
    return ks


def _p(t):
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current CUDA stream of the current device as a pointer.  Asked for on every launch, so it goes through the two raw
    accessors of the framework (well under a microsecond) instead of building a ``torch.cuda.Stream`` object (~15 us)."""
    if _raw_stream is not None and _raw_device is not None:
        return C.c_void_p(_raw_stream(_raw_device()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


def _comm(comm):
    return C.byref(comm) if comm is not None else None


def f32(x: float) -> C.c_float:
    return C.c_float(x)


# ----------------------------------------------------------------------------- projections
def skinny_bf16(x, w, out, mode=SK_OUT_F32, *, rows=None, comm=None, channel=0, batch=1, xb=0, wb=0, ob=0, N=None, K=None,
                xs=None, ws=None, os_=None):
    """``out[r, n] = sum_k x[r, k] w[n, k]`` for 1..8 rows; see ``glmb_skinny_bf16``."""
    rows = x.shape[0] if rows is None else rows
    N = w.shape[-2] if N is None else N
    K = w.shape[-1] if K is None else K
    xs = x.stride(0) if xs is None else xs
    ws = w.stride(-2) if ws is None else ws
    os_ = out.stride(0) if os_ is None else os_
    if mode == SK_OUT_ALLREDUCE_BF16 and _exchanges is not None:
        ks = _skinny_ksplit(-(-N // 2) * batch, K)
        while ks > 1 and -(-N // ((8 // ks) * 2)) * batch > 148 * 3:  # the all-reduce keeps its grid within one wave (csrc/gemv.cu)
            ks //= 2
        groups = 8 // ks
        _note_allreduce("skinny_bf16", comm, channel, -(-N // (groups * 2)) * batch, groups * 2 * (1 if rows <= 1 else 2 if rows <= 2 else 4 if rows <= 4 else 8))
    _check(
        lib().glmb_skinny_bf16(_p(x), C.c_int64(xs), rows, _p(w), C.c_int64(ws), N, K, _p(out), C.c_int64(os_), mode, batch,
                               C.c_int64(xb), C.c_int64(wb), C.c_int64(ob), _comm(comm), channel, _stream()),
        "skinny_bf16",
    )


def skinny_bf16_swiglu(x, wg, wu, act):
    _check(
        lib().glmb_skinny_bf16_swiglu(_p(x), C.c_int64(x.stride(0)), x.shape[0], _p(wg), _p(wu), C.c_int64(wg.stride(0)),
                                      wg.shape[0], wg.shape[1], _p(act), C.c_int64(act.stride(0)), _stream()),
        "skinny_bf16_swiglu",
    )


def set_moe_experts_total(experts: int) -> None:
    """Tell the expert GEMV launchers how many routed experts the model has in all (they see only this GPU's share): the
    expected number of local routes selects how deep the kernels pipeline their loads."""
    lib().glmb_set_moe_experts_total(int(experts))


def set_moe_mma(enabled: int) -> None:
    """1 (default): FP8 expert GEMVs feed mma.sync; 0: the fp32-FMA kernels."""
    lib().glmb_set_moe_mma(int(enabled))


def moe_gateup_fp8(x, top_k, tile_expert, tile_routes, n_tiles, tiles, rt, wg, wu, sg, su, expert_base, act):
    experts_local, I, H = wg.shape
    _check(
        lib().glmb_moe_gateup_fp8(_p(x), C.c_int64(x.stride(0)), top_k, _p(tile_expert), _p(tile_routes), _p(n_tiles), tiles, rt,
                                  _p(wg), _p(wu), _p(sg), _p(su), expert_base, experts_local, I, H, _p(act), _stream()),
        "moe_gateup_fp8",
    )


def moe_down_fp8(act, route_weight, tile_expert, tile_routes, n_tiles, tiles, rt, wd, sd, expert_base, dw):
    experts_local, H, I = wd.shape
    _check(
        lib().glmb_moe_down_fp8(_p(act), _p(route_weight), _p(tile_expert), _p(tile_routes), _p(n_tiles), tiles, rt, _p(wd),
                                _p(sd), expert_base, experts_local, I, H, _p(dw), _stream()),
        "moe_down_fp8",
    )


def moe_down_combine(act, route_weight, topk_ids, wd, sd, shared_partial, rows, top_k, scale, out, comm=None, channel=CH_MLP):
    """Column-sliced experts, decode: down projection of every route, route sum, shared partial and all-reduce in one launch
    (``moe_down_combine_kernel``); the roundings of ``moe_down_fp8`` followed by ``moe_combine``."""
    experts, H, I = wd.shape
    _note_allreduce("moe_down_combine", comm, channel, (H // 16) * -(-rows // MAX_ROWS), 2 * min(rows, MAX_ROWS) * 16)
    _check(
        lib().glmb_moe_down_combine(_p(act), _p(route_weight), _p(topk_ids), _p(wd), _p(sd), experts, I, H, rows, top_k, _p(shared_partial),
                                    f32(scale), _p(out), _comm(comm), channel, _stream()),
        "moe_down_combine",
    )


def moe_grouped_fp8w(a_sorted, w0, w1, s0, s1, tiles, n_tiles, mode, out, *, perm=None, route_weight=None, status=None):
    """Grouped expert GEMM over expert-sorted routes with in-kernel FP8 decode (tcgen05); see ``glmb_moe_grouped_fp8w``.

    mode 0: ``out[sorted, I] = bf16(silu(a @ w0[e].T) * (a @ w1[e].T))``; mode 1: ``out[perm[sorted], H] = bf16(bf16(a @ w0[e].T) *
    bf16(route_weight))``.  ``tiles`` is ``[max_tiles, 4]`` int32 (first sorted row, end row, local expert, 0).
    """
    experts, N, K = w0.shape
    _check(
        lib().glmb_moe_grouped_fp8w(_p(a_sorted), a_sorted.shape[0], _p(w0), _p(w1), _p(s0), _p(s1), experts, N, K, _p(tiles),
                                    _p(n_tiles), tiles.shape[0], mode, _p(perm), _p(route_weight), _p(out), _p(status), _stream()),
        "moe_grouped_fp8w",
    )


def swiglu_rows(gate, up, act=None):
    """``bf16(g * sigmoid(g) * u)`` of two contiguous bf16 tensors (fp32 arithmetic, one rounding) in one launch; returns ``act``."""
    if act is None:
        act = torch.empty_like(gate)
    if not (gate.is_contiguous() and up.is_contiguous() and act.is_contiguous()) or gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16:
        raise ValueError("swiglu_rows takes contiguous bf16 tensors")
    _check(lib().glmb_swiglu_rows(_p(gate), _p(up), _p(act), C.c_int64(gate.numel()), _stream()), "swiglu_rows")
    return act


def route_sort128(topk_ids, ebase: int, el: int, tiles, n_tiles, perm) -> None:
    """Stable sort of this GPU's routes by expert, cut into 128-route tiles, in one launch (see csrc/route_sort.cu).

    ``topk_ids``: int32 ``[rows, top_k]`` contiguous; ``tiles``: int32 ``[>= P / 128 + el, 4]``; ``n_tiles``: int32 ``[1]``; ``perm``: int32 ``[P]``."""
    P = topk_ids.numel()
    _check(lib().glmb_route_sort128(_p(topk_ids), P, int(ebase), int(el), tiles.shape[0], _p(tiles), _p(n_tiles), _p(perm), _stream()), "route_sort128")


def route_sort8(topk_ids, ebase: int, el: int, tile_expert, tile_routes, n_tiles, perm) -> None:
    """The same stable sort cut into tiles of 8 routes for the tensor-core GEMV expert kernels (few routes per expert).

    ``tile_expert``: int32 ``[>= P / 8 + el]`` (global expert ids, -1 past the last tile); ``tile_routes``: int32 ``[tiles, 8]`` (route ids,
    -1 in empty slots); ``n_tiles``: int32 ``[1]``; ``perm``: int32 ``[P]`` scratch."""
    P = topk_ids.numel()
    if tile_routes.shape[0] < tile_expert.shape[0] or tile_routes.shape[1] != 8 or not tile_routes.is_contiguous():
        raise ValueError("route_sort8: tile_routes must be a contiguous [tiles, 8] tensor with a row per tile_expert entry")
    _check(lib().glmb_route_sort8(_p(topk_ids), P, int(ebase), int(el), tile_expert.shape[0], _p(tile_expert), _p(tile_routes), _p(n_tiles),
                                  _p(perm), _stream()), "route_sort8")


def gather_rows(src, idx, divisor, dst):
    """``dst[i] = src[idx[i] // divisor]`` (a row of zeros where ``idx[i] < 0``); bf16 rows, width a multiple of 8."""
    _check(lib().glmb_gather_rows(_p(src), C.c_int64(src.stride(0)), _p(idx), divisor, _p(dst), dst.shape[0], dst.shape[1], _stream()),
           "gather_rows")


def moe_finish(routed_sum, shared_sum, scale, out):
    """``out = bf16(bf16(bf16(routed_sum) * scale) + bf16(shared_sum))`` over contiguous fp32 tensors of one shape: the step after a
    library all-reduce of the two partial sums of a prefill chunk."""
    if not (routed_sum.is_contiguous() and shared_sum.is_contiguous() and out.is_contiguous()) or routed_sum.shape != shared_sum.shape:
        raise ValueError("moe_finish takes contiguous tensors of one shape")
    _check(lib().glmb_moe_finish(_p(routed_sum), _p(shared_sum), C.c_int64(routed_sum.numel()), f32(scale), _p(out), _stream()), "moe_finish")


def moe_combine(dw, topk_ids, shared_partial, rows, top_k, H, expert_base, experts_local, scale, plain, out, routed_partial=None,
                comm=None, channel=CH_MLP):
    if routed_partial is None:
        _note_allreduce("moe_combine", comm, channel, -(-H // 16) * -(-rows // MAX_ROWS), (1 if plain else 2) * min(rows, MAX_ROWS) * 16)
    _check(
        lib().glmb_moe_combine(_p(dw), _p(topk_ids), _p(shared_partial), rows, top_k, H, expert_base, experts_local, f32(scale),
                               int(plain), _p(out), _p(routed_partial), _comm(comm), channel, _stream()),
        "moe_combine",
    )


# ----------------------------------------------------------------------------- norms / rope / queries
def embed_rows(tokens, table, residual, status):
    _check(lib().glmb_embed_rows(_p(tokens), _p(table), tokens.shape[0], table.shape[0], table.shape[1], _p(residual), _p(status),
                                 _stream()), "embed_rows")


def add_rmsnorm(update, residual, weight, out, eps):
    rows, H = residual.shape
    _check(lib().glmb_add_rmsnorm(_p(update), _p(residual), _p(weight), _p(out), rows, H, f32(eps), _stream()), "add_rmsnorm")


def set_qkv_fast(enabled: int) -> None:
    """1 (default): the single-round-trip qkv_a_post kernel; 0: the generic one."""
    lib().glmb_set_qkv_fast(int(enabled))


def qkv_a_post(args: QkvPostArgs, rows: int):
    _check(lib().glmb_qkv_a_post(C.byref(args), rows, _stream()), "qkv_a_post")


def q_post(args: QPostArgs, rows: int):
    _check(lib().glmb_q_post(C.byref(args), rows, _stream()), "q_post")


def q_absorb(q_nope, rows, kv_b, heads_local, head_base, heads_total, nope, vdim, L, rd, q_full, q_full_offset=0, comm=None,
             sig=SIG_Q, *, q_proj=None, rope_table=None, row_pos=None, capacity=0):
    """``q_proj`` (fp32 output of the q_b projection) replaces ``q_nope`` and makes the kernel do the q_post work of its heads too."""
    _note_signal("q_absorb", comm, sig)
    if q_proj is not None:
        _check(
            lib().glmb_q_absorb_from_proj(_p(q_proj), C.c_int64(q_proj.stride(0)), _p(rope_table), _p(row_pos), capacity, rows, _p(kv_b),
                                          heads_local, head_base, heads_total, nope, vdim, L, rd, _p(q_full), C.c_int64(q_full_offset),
                                          _comm(comm), sig, _stream()),
            "q_absorb_from_proj",
        )
        return
    _check(
        lib().glmb_q_absorb(_p(q_nope), rows, _p(kv_b), heads_local, head_base, heads_total, nope, vdim, L, rd, _p(q_full),
                            C.c_int64(q_full_offset), _comm(comm), sig, _stream()),
        "q_absorb",
    )


# ----------------------------------------------------------------------------- indexer
def indexer_takes_raw_query(IH: int, D: int) -> bool:
    return D == 128 and IH == 32 and _indexer_tensor_cores()


def _indexer_rows_kernel() -> bool:
    import os

    return os.environ.get("GLM_B200_INDEXER_ROWS", "1") != "0"  # '0': prefill chunks use the one-row kernel too (A/B runs)


def _indexer_tensor_cores() -> bool:
    import os

    return os.environ.get("GLM_B200_INDEXER", "tcgen05") != "cuda"  # 'cuda': force the CUDA-core kernel (A/B runs)


INDEXER_ROWS_MIN = 16  # from this many rows of one chat on, the many-rows indexer kernel is the faster one


def indexer_rows_scratch_bytes(rows: int) -> int:
    lib()
    return int(_lib.glmb_indexer_rows_scratch_bytes(int(rows)))


def indexer_score(q_idx, head_w, index_cache, row_pos, row_lane, rows, IH, D, index_slot, full_layers, local_cap, stripe, world,
                  rank, capacity, max_ctx, score_stride, scale, scores, scores_offset=0, comm=None, sig=SIG_SCORES, status=None, *,
                  q_raw=None, q_offset=0, inv_freq=None, rd=0, pieces=None, lane=None):
    """``q_raw`` (fp32 q_b projection, index heads at ``q_offset``) replaces ``q_idx``: the tcgen05 kernel applies the RoPE itself.

    ``pieces`` (scratch of :func:`indexer_rows_scratch_bytes`) with ``lane`` selects the many-rows kernel: every row belongs to
    the chat in cache lane ``lane`` (a prefill chunk), the key tiles stay resident while the rows stream past them."""
    _note_signal("indexer_score", comm, sig)
    if pieces is not None and rows >= INDEXER_ROWS_MIN and indexer_takes_raw_query(IH, D) and _indexer_rows_kernel():
        if lane is None:
            raise ValueError("the many-rows indexer needs the cache lane that all rows share")
        if pieces.numel() * pieces.element_size() < indexer_rows_scratch_bytes(rows):
            raise ValueError("indexer scratch too small")
        q = q_raw if q_raw is not None else q_idx
        _check(
            lib().glmb_indexer_score_tc_rows(_p(q), C.c_int64(q.stride(0) if q_raw is not None else IH * D), C.c_int64(q_offset if q_raw is not None else 0),
                                             _p(inv_freq) if q_raw is not None else None, rd if q_raw is not None else 0, _p(head_w),
                                             _p(index_cache), C.c_int64(index_cache.numel() // D), _p(row_pos), int(lane), rows, IH, D,
                                             index_slot, full_layers, local_cap, stripe, world, rank, capacity, max_ctx,
                                             C.c_int64(score_stride), f32(scale), _p(scores), C.c_int64(scores_offset), _p(pieces),
                                             _comm(comm), sig, _p(status), _stream()),
            "indexer_score_tc_rows",
        )
        return
    if q_raw is not None:
        if not indexer_takes_raw_query(IH, D):
            raise ValueError("the raw-query path needs the tcgen05 indexer (32 heads of 128)")
        _check(
            lib().glmb_indexer_score_tc_raw(_p(q_raw), C.c_int64(q_raw.stride(0)), C.c_int64(q_offset), _p(inv_freq), rd, _p(head_w),
                                            _p(index_cache), C.c_int64(index_cache.numel() // D), _p(row_pos), _p(row_lane), rows, IH, D,
                                            index_slot, full_layers, local_cap, stripe, world, rank, capacity, max_ctx,
                                            C.c_int64(score_stride), f32(scale), _p(scores), C.c_int64(scores_offset), _comm(comm), sig,
                                            _p(status), _stream()),
            "indexer_score_tc_raw",
        )
        return
    if D == 128 and IH == 32 and _indexer_tensor_cores():
        # the usual head shape: keys x query pieces on tcgen05 (see csrc/indexer_tcgen05.cu)
        _check(
            lib().glmb_indexer_score_tc(_p(q_idx), _p(head_w), _p(index_cache), C.c_int64(index_cache.numel() // D), _p(row_pos),
                                        _p(row_lane), rows, IH, D, index_slot, full_layers, local_cap, stripe, world, rank, capacity,
                                        max_ctx, C.c_int64(score_stride), f32(scale), _p(scores), C.c_int64(scores_offset),
                                        _comm(comm), sig, _p(status), _stream()),
            "indexer_score_tc",
        )
        return
    _check(
        lib().glmb_indexer_score(_p(q_idx), _p(head_w), _p(index_cache), _p(row_pos), _p(row_lane), rows, IH, D, index_slot,
                                 full_layers, local_cap, stripe, world, rank, capacity, max_ctx, C.c_int64(score_stride),
                                 f32(scale), _p(scores), C.c_int64(scores_offset), _comm(comm), sig, _p(status), _stream()),
        "indexer_score",
    )


def set_topk_cluster(enabled: int) -> None:
    """1 (default): exact top-k on an 8-CTA cluster per row; 0: the single-CTA kernel."""
    lib().glmb_set_topk_cluster(int(enabled))


def topk_select(scores, row_pos, rows, capacity, score_stride, top_k, stripe, world, rank, sel_global, sel_local, sel_counts,
                comm=None, sig=SIG_SCORES):
    _check(
        lib().glmb_topk_select(_p(scores), _p(row_pos), rows, capacity, C.c_int64(score_stride), top_k, stripe, world, rank,
                               _p(sel_global), _p(sel_local), _p(sel_counts), _comm(comm), sig, _stream()),
        "topk_select",
    )


# ----------------------------------------------------------------------------- attention
def attn_chunk() -> int:
    return lib().glmb_attn_chunk()


def sparse_mla_partial(q_full, kv_cache, sel_local, sel_counts, row_lane, rows, H, L, rd, layer, layers, local_cap, top_k,
                       max_chunks, scale, part_o, part_ml, comm=None, wait_sig=-1, status=None):
    _check(
        lib().glmb_sparse_mla_partial(_p(q_full), _p(kv_cache), _p(sel_local), _p(sel_counts), _p(row_lane), rows, H, L, rd, layer,
                                      layers, local_cap, top_k, max_chunks, f32(scale), _p(part_o), _p(part_ml), _comm(comm),
                                      wait_sig, _p(status), _stream()),
        "sparse_mla_partial",
    )


def sparse_mla_rows(q_full, kv_cache, sel_local, sel_counts, row_lane, rows, H, L, rd, layer, layers, local_cap, top_k, scale, o_lat,
                    status=None):
    """Attention of many query rows whose selected keys all live in this GPU's cache: one CTA per (row, 16 heads) walks every
    chunk with running softmax statistics and writes normalized bf16 ``o_lat [rows, H, L]`` (no partials, no merge)."""
    _check(
        lib().glmb_sparse_mla_rows(_p(q_full), _p(kv_cache), _p(sel_local), _p(sel_counts), _p(row_lane), rows, H, L, rd, layer, layers,
                                   local_cap, top_k, f32(scale), _p(o_lat), _p(status), _stream()),
        "sparse_mla_rows",
    )


def attn_merge_vproj(part_o, part_ml, sel_counts, rows, H, L, top_k, max_chunks, kv_b, nope, o_lat, attn_v):
    """Decode, every key local: merge of the chunk partials and the per-head value projection in one launch
    (``attn_merge_vproj_kernel``; the bits of ``attn_local_merge`` followed by the batched ``skinny_bf16``).
    ``kv_b``: ``[H, nope + v, L]`` bf16, the value rows start at row ``nope`` of every head."""
    per_head, v = kv_b.shape[1], kv_b.shape[1] - nope
    w_v = kv_b.data_ptr() + nope * L * 2
    _check(
        lib().glmb_attn_merge_vproj(_p(part_o), _p(part_ml), _p(sel_counts), rows, H, L, top_k, max_chunks, C.c_void_p(w_v),
                                    C.c_int64(per_head * L), v, _p(o_lat), _p(attn_v), _stream()),
        "attn_merge_vproj",
    )


def attn_local_merge(part_o, part_ml, sel_counts, rows, H, L, top_k, max_chunks, o_lat, heads_local, xpart_offset=0, comm=None,
                     sig=SIG_ATTN):
    _note_signal("attn_local_merge", comm, sig)
    _check(
        lib().glmb_attn_local_merge(_p(part_o), _p(part_ml), _p(sel_counts), rows, H, L, top_k, max_chunks, _p(o_lat), heads_local,
                                    C.c_int64(xpart_offset), _comm(comm), sig, _stream()),
        "attn_local_merge",
    )


def attn_final_merge(rows, L, heads_local, xpart_offset, o_lat, comm, sig=SIG_ATTN):
    _check(lib().glmb_attn_final_merge(rows, L, heads_local, C.c_int64(xpart_offset), _p(o_lat), _comm(comm), sig, _stream()),
           "attn_final_merge")


# ----------------------------------------------------------------------------- router / sampler / misc
def router_topk(logits, bias, top_k, ids, weights):
    rows, E = logits.shape
    _check(lib().glmb_router_topk(_p(logits), _p(bias), rows, E, top_k, _p(ids), _p(weights), _stream()), "router_topk")


def argmax_rows(logits, rows, V, vocab_base, cand, cand_offset=0, comm=None, sig=SIG_SAMPLE, status=None):
    _note_signal("argmax_rows", comm, sig)
    _check(
        lib().glmb_argmax_rows(_p(logits), C.c_int64(logits.stride(0)), rows, V, vocab_base, _p(cand), C.c_int64(cand_offset),
                               _comm(comm), sig, _p(status), _stream()),
        "argmax_rows",
    )


def step_finalize(cand, n_sets, rows, row_active, tokens, positions, out_tokens, step_counter, ring, advance, comm=None,
                  sig=SIG_SAMPLE, local_best=None, cand_offset=0):
    """Pick the best of ``n_sets`` packed candidates per row (``cand`` is ``[n_sets, rows]`` 64-bit keys).

    ``local_best`` (``[rows]`` int64 filled by the lm_head kernel in argmax mode) is first published as this rank's
    candidate.  advance: bit 0 writes the sampled token into ``tokens``, bit 1 increments ``positions``.
    """
    if local_best is not None:
        _note_signal("step_finalize", comm, sig)
    _check(
        lib().glmb_step_finalize(_p(cand), C.c_int64(cand_offset), _p(local_best), n_sets, rows, _p(row_active), _p(tokens),
                                 _p(positions), _p(out_tokens), _p(step_counter), ring, int(advance), _comm(comm), sig, _stream()),
        "step_finalize",
    )


def fp8_to_bf16(bits, scale, out, block=(128, 128), status=None):
    N, K = bits.shape[-2], bits.shape[-1]
    lead = bits.numel() // (N * K)
    if lead != 1:
        for i in range(lead):
            fp8_to_bf16(bits.reshape(lead, N, K)[i], scale.reshape(lead, *scale.shape[-2:])[i], out.reshape(lead, N, K)[i], block,
                        status)
        return
    _check(lib().glmb_fp8_to_bf16(_p(bits), _p(scale), C.c_int64(N), C.c_int64(K), block[0], block[1], _p(out), _p(status),
                                  _stream()), "fp8_to_bf16")


def fill_random_fp8(out, seed):
    _check(lib().glmb_fill_random_fp8(_p(out), C.c_int64(out.numel()), C.c_uint64(seed), _stream()), "fill_random_fp8")


def fill_random_bf16(out, seed, mean=0.0, std=0.02):
    _check(lib().glmb_fill_random_bf16(_p(out), C.c_int64(out.numel()), C.c_uint64(seed), f32(mean), f32(std), _stream()),
           "fill_random_bf16")


def fill_uniform_f32(out, seed, lo, hi):
    _check(lib().glmb_fill_uniform_f32(_p(out), C.c_int64(out.numel()), C.c_uint64(seed), f32(lo), f32(hi), _stream()),
           "fill_uniform_f32")


# ----------------------------------------------------------------------------- tcgen05 GEMM
def gemm_allreduce_part_bytes(rows: int, N: int, world: int) -> int:
    fn = lib().glmb_gemm_allreduce_part_bytes
    fn.restype = C.c_int64
    return int(fn(rows, N, world))


def gemm_bf16_tc_allreduce(a, b, comm, part_offset, out_offset, *, sig=SIG_GEMM, status=None):
    """One kernel: ``sum over ranks of a_r @ b_r.T`` (tcgen05 tiles + NVLink partial exchange), bf16 result ``[rows, N]`` at
    ``out_offset`` of every rank's staging buffer.  Follow with ``wait_signal(comm, sig)`` before reading it."""
    rows, K = a.shape
    N = b.shape[0]
    _check(
        lib().glmb_gemm_bf16_tcgen05_allreduce(_p(a), C.c_int64(a.stride(0)), _p(b), C.c_int64(b.stride(0)), rows, N, K, _comm(comm),
                                               C.c_int64(part_offset), C.c_int64(out_offset), sig, _p(status), _stream()),
        "gemm_bf16_tcgen05_allreduce",
    )


def wait_signal(comm, sig):
    _check(lib().glmb_wait_signal(_comm(comm), sig, _stream()), "wait_signal")


def set_mega_cooperative(enabled: int) -> None:
    """1 (default): the persistent decode kernel is launched cooperatively; 0: as an ordinary launch of the same grid."""
    lib().glmb_set_mega_cooperative(int(enabled))


def set_gemm_variant(variant: int) -> None:
    """0: pick by problem size (default); 1: one 128x128 tile per CTA; 2: the persistent 128x256 kernel."""
    lib().glmb_set_gemm_variant(int(variant))


def gemm_bf16_tc(a, b, out, *, experts=1, tiles=None, n_tiles=None, status=None):
    """``out[rows, N] = a[rows, K] @ b[N, K].T`` on the tcgen05 tensor cores (bf16 in, fp32 accumulate).

    ``b`` may be ``[experts, N, K]`` with ``tiles`` (``[max_tiles, 4]`` int32: first row, end row, expert, 0) and
    ``n_tiles`` (device int32) describing 128-row tiles of the expert-sorted ``a``: grouped mode.
    ``out`` is bf16 or fp32.
    """
    rows, K = a.shape
    N = b.shape[-2]
    out_f32 = int(out.dtype == torch.float32)
    max_tiles = tiles.shape[0] if tiles is not None else 0
    _check(
        lib().glmb_gemm_bf16_tcgen05(_p(a), C.c_int64(a.stride(0)), _p(b), C.c_int64(b.stride(-2)), _p(out), C.c_int64(out.stride(0)),
                                     rows, N, K, experts, _p(tiles), _p(n_tiles), max_tiles, out_f32, _p(status), _stream()),
        "gemm_bf16_tcgen05",
    )
