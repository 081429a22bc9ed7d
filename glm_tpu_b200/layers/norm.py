"""RMSNorm family.

Contract: statistics in fp32; ``bf16(x * rsqrt(mean(x^2) + eps))`` is rounded to bf16 *before* it is multiplied by the bf16 weight
(second rounding); the fused add + norm sums update and residual in fp32, normalizes the unrounded sum and carries ``bf16(sum)`` as
the new residual.  Parity: reference ``glm_tpu/layers/norm.py:29-122``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.oracle import contract


def add_rms_norm(update: torch.Tensor | None, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """Returns ``(normalized bf16 [rows, H], new residual bf16 [rows, H])``; ``update=None`` normalizes the residual alone."""
    if residual.is_cuda:
        from glm_tpu_b200.ops import native

        residual = residual.to(torch.bfloat16).contiguous().clone()
        out = torch.empty_like(residual)
        native.add_rmsnorm(None if update is None else update.to(torch.bfloat16).contiguous(), residual, weight.to(torch.bfloat16), out, eps)
        return out, residual
    x, new_residual = contract.add_rms_norm(update, residual, weight, eps)
    return x.to(torch.bfloat16), new_residual.to(torch.bfloat16)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return add_rms_norm(None, x, weight, eps)[0]


def layer_norm_affine(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Indexer key normalization (fp32 throughout); on the GPU it is part of ``qkv_a_post``, here the plain form."""
    return contract.layer_norm_affine(x.float().cpu(), weight.float().cpu(), bias.float().cpu(), eps).to(x.device)
