"""``y = x @ W.T`` with bf16 operands and fp32 accumulation, rounded once to bf16 (or kept fp32).

GPU: 1-8 rows stream the weight through the skinny GEMV kernel; more rows run the tcgen05 GEMM.  K-split partial sums over
several GPUs are reduced inside those kernels (see ``models/glm_moe_dsa/model.py``); this function is the single-GPU op.
Parity: reference ``glm_tpu/layers/linear.py:26-128``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.oracle import contract


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    if x.is_cuda:
        from glm_tpu_b200.ops import native

        x, weight = x.to(torch.bfloat16).contiguous(), weight.to(torch.bfloat16).contiguous()
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        if x.shape[0] <= native.MAX_ROWS and weight.shape[1] % 8 == 0:
            native.skinny_bf16(x, weight, out, native.SK_OUT_BF16 if out_dtype == torch.bfloat16 else native.SK_OUT_F32)
        elif weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0:
            native.gemm_bf16_tc(x, weight, out)
        else:
            out = torch.mm(x, weight.t()).to(out_dtype)
        return out
    return contract.linear(x, weight, out_bf16=out_dtype == torch.bfloat16).to(out_dtype)
