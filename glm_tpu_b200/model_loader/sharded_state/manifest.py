"""The manifest: one record per packed file, assembled from the writers' receipts and published last.

Parity: reference ``glm_tpu/model_loader/sharded_state/manifest.py:14-76``.
"""

from __future__ import annotations

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader.sharded_state import format as fmt


def expected_files(world: int) -> list[str]:
    return [fmt.SHARED_FILE] + [fmt.expert_file(r, world) for r in range(world)]


def assemble_manifest(receipts: list[dict], geometry, world: int, source_inventory_sha256: str, expert_split: str = "whole") -> dict:
    files: dict = {}
    for receipt in receipts:
        for name, record in receipt.items():
            if name in files:
                raise CheckpointValidationError(f"two receipts claim {name}")
            files[name] = record
    want = expected_files(world)
    if sorted(files) != sorted(want):
        raise CheckpointValidationError(f"receipts cover {sorted(files)}, the checkpoint needs {sorted(want)}")
    return {"schema": "glm_b200_manifest_v2", "format": fmt.FORMAT_VERSION, "geometry_sha256": geometry.geometry_hash,
            "world": world, "expert_split": expert_split, "source_inventory_sha256": source_inventory_sha256, "files": {n: files[n] for n in sorted(files)},
            "total_bytes": sum(r["size"] for r in files.values())}
