"""Router: fp32 sigmoid scores; the correction bias enters the *choice* only; the weights are the unbiased scores of the chosen
experts normalized in fp32; ties go to the lowest expert id; the routed scale (2.5) is applied by the combine, not here.

Parity: reference ``glm_tpu/layers/moe/router.py:20-167``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.layers.contracts import RouterOutput
from glm_tpu_b200.oracle import contract


def route(logits: torch.Tensor, bias: torch.Tensor, top_k: int) -> RouterOutput:
    """``logits [rows, E]`` fp32 (``x @ W_router.T``)."""
    rows, E = logits.shape
    if logits.is_cuda:
        from glm_tpu_b200.ops import native

        ids = torch.empty((rows, top_k), dtype=torch.int32, device=logits.device)
        weights = torch.empty((rows, top_k), dtype=torch.float32, device=logits.device)
        native.router_topk(logits.float().contiguous(), bias.float().contiguous(), top_k, ids, weights)
        return RouterOutput(ids, weights)
    scores = torch.sigmoid(logits.float())
    choice = scores + bias.float()[None, :]
    ids = torch.argsort(-contract.orderable_key(choice), dim=-1, stable=True)[:, :top_k]
    picked = torch.gather(scores, 1, ids)
    return RouterOutput(ids.to(torch.int32), picked / (picked.sum(-1, keepdim=True) + 1e-20))
