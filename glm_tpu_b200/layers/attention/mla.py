"""Absorbed multi-head latent attention over selected cache rows.

``scores = (q_c . latent + q_rope . k_rope) * scale`` in fp32, softmax with the probabilities rounded to bf16 before ``P . latent``,
one final normalization, an empty selection gives zeros.  GPU: gather with ``cp.async``, ``mma.sync`` tiles, running softmax.
Parity: reference ``glm_tpu/layers/attention/mla.py:58-502``, ``glm_tpu/kernels/sparse_mla/kernel.py:128-183``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.layers.contracts import SelectedPositions
from glm_tpu_b200.oracle import contract


def sparse_attention(q_absorbed: torch.Tensor, cache_rows: torch.Tensor, selected: SelectedPositions, latent: int, scale: float) -> torch.Tensor:
    """``q_absorbed [rows, H, latent + rope]`` bf16, ``cache_rows [ctx, latent + rope]`` bf16 -> ``[rows, H, latent]`` bf16."""
    rows, H, W = q_absorbed.shape
    rd = W - latent
    if q_absorbed.is_cuda:
        from glm_tpu_b200.ops import native

        dev = q_absorbed.device
        out = torch.empty((rows, H, latent), dtype=torch.bfloat16, device=dev)
        lane = torch.zeros(rows, dtype=torch.int32, device=dev)
        ctx = cache_rows.shape[0]
        native.sparse_mla_rows(q_absorbed.to(torch.bfloat16).contiguous(), cache_rows.to(torch.bfloat16).contiguous().view(1, 1, ctx, W),
                               selected.local_rows.contiguous(), selected.counts.contiguous(), lane, rows, H, latent, rd, 0, 1, ctx,
                               selected.positions.shape[1], scale, out)
        return out
    q = q_absorbed.float()
    return torch.stack([contract.absorbed_attention_row(q[r, :, :latent], q[r, :, latent:], cache_rows.float(), selected.row(r), scale)
                        for r in range(rows)]).to(torch.bfloat16)
