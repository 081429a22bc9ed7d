"""Rotary embeddings: interleaved pairs ``(2j, 2j+1)``.

Main attention: a bf16 ``cos | sin`` table built with fp32 NumPy arithmetic, fp32 products, one bf16 rounding of the result.
Indexer: fp32 ``cos/sin(position * theta^(-2j/d))`` on the first ``rope_dim`` features, result stays fp32.
On the GPU both are fused into ``qkv_a_post`` / ``q_post`` / ``q_absorb`` / the tcgen05 indexer; these are the standalone forms.
Parity: reference ``glm_tpu/layers/rope.py:20-199``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.oracle import contract

rope_table = contract.rope_table


def apply_rotary_table(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return contract.rope_interleaved_table(x.cpu(), positions.cpu(), table.cpu()).to(device=x.device, dtype=torch.bfloat16)


def apply_rotary_fp32(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: int) -> torch.Tensor:
    return contract.rope_interleaved_fp32(x.cpu(), positions.cpu(), theta, rope_dim).to(x.device)
