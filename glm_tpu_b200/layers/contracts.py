"""Small state types shared by the layer functions.

Parity: reference ``glm_tpu/layers/contracts.py:26-71`` (``SelectedPositions`` and the per-block weight bundles).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class SelectedPositions:
    """DSA selection of a batch of query rows: ascending positions, ``-1`` padded, plus the counts."""

    positions: torch.Tensor  # [rows, top_k] int32, global positions
    local_rows: torch.Tensor  # [rows, top_k] int32, rows of this GPU's cache slice among them
    counts: torch.Tensor  # [rows, 2] int32: selected, selected and owned by this GPU

    def row(self, r: int) -> torch.Tensor:
        return self.positions[r, : int(self.counts[r, 0])].long()


@dataclass
class RouterOutput:
    expert_ids: torch.Tensor  # [rows, top_k] int32, descending choice score, ties to the lowest expert id
    weights: torch.Tensor  # [rows, top_k] fp32, normalized unbiased sigmoid scores (the routed scale is applied later)
