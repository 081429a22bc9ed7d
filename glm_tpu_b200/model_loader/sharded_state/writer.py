"""Packing: source checkpoint -> ``shared.safetensors`` + one expert file per GPU.

``pack_files(inventory, target, geometry, world, files, split)`` writes the named files (``"shared"`` and/or rank numbers).
Each source tensor is validated against the placement contract (dtype, shape).  A file is laid out from the shapes alone
(``format.FileWriter``) and filled piece by piece at final offsets: a shared tensor streams from its source in pieces of at
most ``format.PIECE_BYTES``; a stacked expert tensor is filled one expert at a time (the expert's own table, or this GPU's
column slice of it), never stacked in memory first.  Every piece is checked (FP8 NaN codes, finiteness) and hashed on its
way, the file goes through ``.partial`` + fsync + re-read + rename.  The return value is a *receipt* per file; the manifest is
assembled from the receipts only after every file exists.  An existing target file is refused.

With column-sliced experts every expert file needs a slice of every expert's tables: the row slices of gate/up are read as
byte ranges, a down table (its columns are cut) is read whole, one expert at a time.

Parity: reference ``glm_tpu/model_loader/sharded_state/writer.py:80-234`` (slice, write .partial, fsync, rename,
destination record).
"""

from __future__ import annotations

from pathlib import Path

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader import placement, source_inventory
from glm_tpu_b200.model_loader.sharded_state import format as fmt


def file_metadata(geometry, world: int, kind: str, rank, split: str) -> dict:
    return {"format": fmt.FORMAT_VERSION, "geometry_sha256": geometry.geometry_hash, "world": world, "kind": kind,
            "rank": "" if rank is None else rank, "expert_split": split}


def pack_files(inv: source_inventory.SourceInventory, target: Path, geometry, world: int, files: list, split: str = "whole") -> dict:
    target = Path(target)
    target.mkdir(parents=True, exist_ok=True)
    expected = placement.expected_sources(geometry)
    for name, t in inv.tensors.items():
        placement.require_source_contract(name, t.dtype, t.shape, geometry, expected)
    missing = [n for n in expected if n not in inv.tensors]
    if missing:
        raise CheckpointValidationError(f"the source lacks {len(missing)} tensors, e.g. {missing[:3]}")
    plan = placement.placements(geometry, world, split)
    receipts = {}
    for which in files:
        rank = None if which == "shared" else int(which)
        name = fmt.SHARED_FILE if rank is None else fmt.expert_file(rank, world)
        path = target / name
        if path.exists():
            raise CheckpointValidationError(f"{name} already exists: packing never overwrites")
        specs = placement.packed_tensor_shapes(geometry, world, rank, split)
        out = fmt.FileWriter(path, specs, file_metadata(geometry, world, "shared" if rank is None else "experts", rank, split))
        try:
            if rank is None:
                for p in plan:
                    if p.file == "shared":
                        for piece in source_inventory.read_source_pieces(inv, p.source):
                            out.append(p.target, piece)
            else:
                # expert slots of one stacked tensor arrive in slot order: the plan lists the experts in ascending order
                mine = [p for p in plan if p.file == "experts" and p.rank in (None, rank)]
                for p in sorted(mine, key=lambda q: (q.target, q.expert_slot)):
                    if p.axis == 0:  # a run of rows is a byte range of the source: read just that
                        out.append(p.target, source_inventory.read_source_tensor(inv, p.source, rows=(rank * p.unit, (rank + 1) * p.unit)))
                    else:
                        out.append(p.target, p.cut(source_inventory.read_source_tensor(inv, p.source), rank))
            receipts[name] = out.close()
        except BaseException:
            out.abort()
            raise
    return receipts
