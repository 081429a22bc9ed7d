"""Greedy sampling over bf16 logits: the highest logit wins, ties go to the lowest token id, ``-0`` equals ``+0``.

With the vocabulary split over GPUs each rank reduces its slice to one packed 64-bit candidate
(``orderable(logit) << 32 | ~id``) and the candidates are exchanged; here the single-GPU op.
Parity: reference ``glm_tpu/layers/sampler.py:34-135``.
"""

from __future__ import annotations

import torch

from glm_tpu_b200.oracle import contract


def greedy(logits: torch.Tensor) -> torch.Tensor:
    """``[rows, vocab]`` -> ``[rows]`` int64."""
    if logits.is_cuda:
        from glm_tpu_b200.ops import native

        rows, vocab = logits.shape
        logits = logits.to(torch.bfloat16).contiguous()
        cand = torch.zeros((1, rows), dtype=torch.int64, device=logits.device)
        native.argmax_rows(logits, rows, vocab, 0, cand)
        return (0xFFFFFFFF - (cand[0] & 0xFFFFFFFF)).long()
    return contract.greedy(contract.bf16_round(logits.float()))
