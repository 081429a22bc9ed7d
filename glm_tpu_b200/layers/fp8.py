"""FP8 weight decode: ``bf16(f32(e4m3fn) * scale_inv[n // 128, k // 128])``, bit-exact on both paths.

Parity: reference ``glm_tpu/layers/fp8.py:18-72,113-143`` (exact 256-entry table, per-table decode).
"""

from __future__ import annotations

import torch

from glm_tpu_b200.oracle import contract


def decode(bits: torch.Tensor, scale_inv: torch.Tensor, block: tuple[int, int] = (128, 128)) -> torch.Tensor:
    if bits.is_cuda:
        from glm_tpu_b200.ops import native

        out = torch.empty(bits.shape, dtype=torch.bfloat16, device=bits.device)
        native.fp8_to_bf16(bits.contiguous(), scale_inv.float().contiguous(), out, block)
        return out
    return contract.dequantize_fp8(bits, scale_inv, block)
