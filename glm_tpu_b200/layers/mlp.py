"""Dense SwiGLU MLP: ``down( bf16( silu(bf16 gate) * bf16 up ) )``.

Parity: reference ``glm_tpu/layers/mlp.py:21-68``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.layers.linear import linear
from glm_tpu_b200.oracle import contract


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.shape[0] <= 8:
        from glm_tpu_b200.ops import native

        act = torch.empty((x.shape[0], w_gate.shape[0]), dtype=torch.bfloat16, device=x.device)
        native.skinny_bf16_swiglu(x.to(torch.bfloat16).contiguous(), w_gate.contiguous(), w_up.contiguous(), act)
        return act
    gate, up = linear(x, w_gate).float(), linear(x, w_up).float()
    return contract.swiglu_act(gate.cpu(), up.cpu()).to(device=x.device, dtype=torch.bfloat16)


def dense_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    return linear(swiglu(x, w_gate, w_up), w_down)
