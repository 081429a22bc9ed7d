"""Token embedding lookup (bf16 rows of a replicated table); an out-of-range id is clamped and recorded in the status word.

Parity: reference ``glm_tpu/layers/embed.py:32-74`` (owner-masked lookup + reduction there; replicated table here).
"""

from __future__ import annotations

import torch


def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if table.is_cuda:
        from glm_tpu_b200.ops import native

        out = torch.empty((tokens.shape[0], table.shape[1]), dtype=torch.bfloat16, device=table.device)
        status = torch.zeros(1, dtype=torch.int32, device=table.device)
        native.embed_rows(tokens.to(device=table.device, dtype=torch.int32), table, out, status)
        return out
    return table[tokens.long()].to(torch.bfloat16)
