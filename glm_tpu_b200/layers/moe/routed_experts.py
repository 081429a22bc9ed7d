"""Routed FP8 experts of one GPU: for every route ``p = (row, slot)`` whose expert lives here,
``dw[p] = bf16( bf16( act_p @ W_down[e].T ) * bf16(weight_p) )`` with ``act_p = bf16(silu(bf16 gate) * bf16 up)`` and every
weight decoded as ``bf16(f32(e4m3) * scale)``; then ``out = bf16( bf16(sum_p dw[p]) * routed_scale ) + bf16(shared) )``.

GPU: 1-8 rows use the route-list GEMV kernels (decoded pairs feed ``mma.sync``); more rows are sorted by expert and run the
grouped tcgen05 kernel that decodes FP8 on the way to the tensor core.
Parity: reference ``glm_tpu/layers/moe/routed_experts.py:27-304``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.layers.contracts import RouterOutput
from glm_tpu_b200.oracle import contract


def routed_experts(x: torch.Tensor, routes: RouterOutput, gate, up, down, *, expert_base: int = 0, block=(128, 128)) -> torch.Tensor:
    """``gate/up/down`` are ``(bits [E_local, N, K] uint8, scale_inv)`` pairs.  Returns ``dw [rows * top_k, H]`` bf16 (rows of routes whose
    expert is not on this GPU are left untouched: zeros here)."""
    rows, H = x.shape
    tk = routes.expert_ids.shape[1]
    el, I = gate[0].shape[0], gate[0].shape[1]
    if x.is_cuda:
        from glm_tpu_b200.ops import native

        dev = x.device
        act = torch.zeros((rows * tk, I), dtype=torch.bfloat16, device=dev)
        dw = torch.zeros((rows * tk, H), dtype=torch.bfloat16, device=dev)
        xb = x.to(torch.bfloat16).contiguous()
        ids = routes.expert_ids.contiguous()
        for r0 in range(0, rows, native.MAX_ROWS):  # the route-list kernels take the routes of up to 8 rows per launch
            n = min(native.MAX_ROWS, rows - r0)
            sl = slice(r0 * tk, (r0 + n) * tk)
            native.moe_gateup_fp8(xb[r0 : r0 + n], tk, ids[r0 : r0 + n].contiguous(), None, None, n * tk, 1, gate[0], up[0], gate[1], up[1],
                                  expert_base, act[sl])
            native.moe_down_fp8(act[sl], routes.weights[r0 : r0 + n].contiguous(), ids[r0 : r0 + n].contiguous(), None, None, n * tk, 1,
                                down[0], down[1], expert_base, dw[sl])
        return dw
    wg, wu, wd = (contract.dequantize_fp8(b, s, block) for b, s in (gate, up, down))
    dw = torch.zeros(rows * tk, H)
    for r in range(rows):
        for k in range(tk):
            e = int(routes.expert_ids[r, k]) - expert_base
            if 0 <= e < el:
                act = contract.swiglu_act(contract.linear(x[r : r + 1], wg[e]), contract.linear(x[r : r + 1], wu[e]))
                dw[r * tk + k] = contract.bf16_round(contract.linear(act, wd[e])[0] * contract.bf16_round(routes.weights[r, k]))
    return dw.to(torch.bfloat16)


def combine(dw: torch.Tensor, shared: torch.Tensor, rows: int, top_k: int, routed_scale: float) -> torch.Tensor:
    """Single-GPU combine of the route outputs with the shared expert's output (both complete, not partial)."""
    routed = dw.float().reshape(rows, top_k, -1).sum(1)
    scaled = contract.bf16_round(contract.bf16_round(routed.cpu()) * routed_scale)
    return contract.bf16_round(scaled + contract.bf16_round(shared.float().cpu())).to(device=dw.device, dtype=torch.bfloat16)
