"""DSA lightning indexer: ``score[t] = sum_h w_h * relu(q_h . key_t * d^-1/2)`` in fp32, then the exact top-k under the total
order (descending score, ties to the lowest position, ``+0 > -0``), returned ascending in position.

GPU: tcgen05 scoring kernel (keys as the M operand) + 8-CTA cluster radix select.  Every GPU selects from the full score row, so
the reference's two-stage shortlist with its omitted-candidate proof is not needed.
Parity: reference ``glm_tpu/layers/attention/dsa_indexer.py:35-150,352-393``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.layers.contracts import SelectedPositions
from glm_tpu_b200.oracle import contract


def scores(query: torch.Tensor, head_weights: torch.Tensor, keys: torch.Tensor, context_lengths: torch.Tensor) -> torch.Tensor:
    """``query [rows, IH, D]`` fp32 (RoPE applied), ``head_weights [rows, IH]``, ``keys [ctx, D]`` bf16 -> ``[rows, ctx]`` fp32 (NaN beyond a row's context)."""
    rows, IH, D = query.shape
    ctx = keys.shape[0]
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    if query.is_cuda:
        from glm_tpu_b200.ops import native

        out = torch.full((rows, ctx), float("nan"), device=query.device)
        pos = (context_lengths.to(device=query.device, dtype=torch.int32) - 1).contiguous()
        lane = torch.zeros(rows, dtype=torch.int32, device=query.device)
        native.indexer_score(query.float().contiguous(), head_weights.float().contiguous(), keys.to(torch.bfloat16).contiguous().view(1, 1, ctx, D),
                             pos, lane, rows, IH, D, 0, 1, ctx, 64, 1, 0, ctx, ctx, ctx, scale, out)
        return out
    dots = torch.einsum("shd,td->sht", query.float(), keys.float()) * scale
    out = torch.einsum("sh,sht->st", head_weights.float(), torch.relu(dots))
    beyond = torch.arange(ctx)[None, :] >= context_lengths[:, None]
    return out.masked_fill(beyond, float("nan"))


def select(score_rows: torch.Tensor, context_lengths: torch.Tensor, top_k: int) -> SelectedPositions:
    rows, ctx = score_rows.shape
    if score_rows.is_cuda:
        from glm_tpu_b200.ops import native

        dev = score_rows.device
        sel_g = torch.empty((rows, top_k), dtype=torch.int32, device=dev)
        sel_l = torch.empty((rows, top_k), dtype=torch.int32, device=dev)
        counts = torch.zeros((rows, 2), dtype=torch.int32, device=dev)
        pos = (context_lengths.to(device=dev, dtype=torch.int32) - 1).contiguous()
        native.topk_select(score_rows.float().contiguous(), pos, rows, ctx, ctx, top_k, 64, 1, 0, sel_g, sel_l, counts)
        return SelectedPositions(sel_g, sel_l, counts)
    sel = torch.full((rows, top_k), -1, dtype=torch.int32)
    counts = torch.zeros((rows, 2), dtype=torch.int32)
    for r in range(rows):
        chosen = contract.top_k_positions(score_rows[r], int(context_lengths[r]), top_k)
        sel[r, : chosen.numel()] = chosen.to(torch.int32)
        counts[r] = chosen.numel()
    return SelectedPositions(sel, sel.clone(), counts)
