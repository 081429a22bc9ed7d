"""Packing: source checkpoint -> ``shared.safetensors`` + one expert file per GPU.

``pack_files(inventory, target, geometry, world, files)`` writes the named files (``"shared"`` and/or rank numbers):
each source tensor is validated against the placement contract (dtype, shape), read, FP8 payloads are checked for NaN
codes, routed experts are stacked into ``[experts_local, N, K]`` in expert order, and the file is written canonically
through ``.partial`` + fsync + rename, then re-read and re-hashed.  The return value is a *receipt* per file; the
manifest is assembled from the receipts only after every file exists.  An existing target file is refused.

Parity: reference ``glm_tpu/model_loader/sharded_state/writer.py:80-234`` (slice, write .partial, fsync, rename,
destination record).
"""

from __future__ import annotations

from pathlib import Path

import torch

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader import placement, source_inventory
from glm_tpu_b200.model_loader.sharded_state import format as fmt


def _metadata(geometry, world: int, kind: str, rank) -> dict:
    return {"format": fmt.FORMAT_VERSION, "geometry_sha256": geometry.geometry_hash, "world": world, "kind": kind,
            "rank": "" if rank is None else rank}


def pack_files(inv: source_inventory.SourceInventory, target: Path, geometry, world: int, files: list) -> dict:
    target = Path(target)
    target.mkdir(parents=True, exist_ok=True)
    expected = placement.expected_sources(geometry)
    for name, t in inv.tensors.items():
        placement.require_source_contract(name, t.dtype, t.shape, geometry, expected)
    missing = [n for n in expected if n not in inv.tensors]
    if missing:
        raise CheckpointValidationError(f"the source lacks {len(missing)} tensors, e.g. {missing[:3]}")
    plan = placement.placements(geometry, world)
    receipts = {}
    for which in files:
        rank = None if which == "shared" else int(which)
        name = fmt.SHARED_FILE if rank is None else fmt.expert_file(rank, world)
        path = target / name
        if path.exists():
            raise CheckpointValidationError(f"{name} already exists: packing never overwrites")
        tensors: dict = {}
        fp8 = set()
        if rank is None:
            for p in plan:
                if p.file == "shared":
                    tensors[p.target] = source_inventory.read_source_tensor(inv, p.source)
                    if p.dtype == "F8_E4M3":
                        fp8.add(p.target)
        else:
            shapes = placement.packed_tensor_shapes(geometry, world, rank)
            for tname, (dtype, shape) in shapes.items():
                tensors[tname] = torch.empty(shape, dtype=fmt.DTYPES[dtype][0])
                if dtype == "F8_E4M3":
                    fp8.add(tname)
            for p in plan:
                if p.file == "experts" and p.rank == rank:
                    tensors[p.target][p.expert_slot] = source_inventory.read_source_tensor(inv, p.source)
        record = fmt.write_file(path, tensors, _metadata(geometry, world, "shared" if rank is None else "experts", rank), fp8)
        if fmt.file_sha256(path) != record["sha256"]:  # read back what reached the disk
            raise CheckpointValidationError(f"{name}: the bytes on disk differ from the bytes written")
        receipts[name] = record
    return receipts
