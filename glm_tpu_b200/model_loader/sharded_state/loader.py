"""Loading a packed checkpoint on one GPU rank.

``load_rank_checkpoint(dir, rank, world)`` verifies the seal/manifest and this rank's two files, then returns the
runtime-layout mapping ``name -> tensor``: every shared tensor whole (FP8 pairs as stored; the model code decodes them to
bf16 on the device and slices heads / MLP columns / vocabulary rows) and the routed experts of this rank already cut
(``[experts_local, N, K]``).  Finiteness of bf16/fp32 tensors and the absence of FP8 NaN codes are checked while
reading.  ``load_full_checkpoint`` reassembles the full stacked layout (CPU oracle, small models only).

Parity: reference ``glm_tpu/model_loader/sharded_state/loader.py:58-154``.
"""

from __future__ import annotations

from pathlib import Path

import torch

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.model_loader.sharded_state.verify import read_geometry, verify_runtime_checkpoint

__all__ = ["read_geometry", "load_rank_checkpoint", "load_full_checkpoint"]


def _read_all(path: Path) -> dict:
    header, start = fmt.read_header(path)
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        t = fmt.read_tensor(path, header, start, name)
        if entry["dtype"] == "F8_E4M3":
            fmt.refuse_fp8_nan(name, t)
        elif t.is_floating_point() and not bool(torch.isfinite(t.float()).all()):
            raise CheckpointValidationError(f"{name}: non-finite values")
        out[name] = t
    return out


def load_rank_checkpoint(target: Path, rank: int, world: int, *, pins: dict | None = None, rehash: bool = True) -> dict:
    target = Path(target)
    report = verify_runtime_checkpoint(target, files=[fmt.SHARED_FILE, fmt.expert_file(rank, world)], pins=pins, rehash=rehash)
    if report["world"] != world:
        raise CheckpointValidationError(f"the checkpoint was packed for {report['world']} GPUs, not {world}")
    arrays = _read_all(target / fmt.SHARED_FILE)
    arrays.update(_read_all(target / fmt.expert_file(rank, world)))
    arrays["__experts_presliced__"] = torch.tensor([rank, world])
    arrays["__expert_split__"] = report.get("expert_split", "whole")
    return arrays


def load_full_checkpoint(target: Path) -> dict:
    target = Path(target)
    report = verify_runtime_checkpoint(target)
    arrays = _read_all(target / fmt.SHARED_FILE)
    parts = [_read_all(target / fmt.expert_file(r, report["world"])) for r in range(report["world"])]
    for name in parts[0]:
        arrays[name] = torch.cat([p[name] for p in parts], dim=0)
    return arrays
