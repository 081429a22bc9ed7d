"""Verification of a packed checkpoint: seal -> manifest -> files (size, digest, header contents vs the placement plan).

``verify_runtime_checkpoint(dir, files=None, pins=None)`` checks the seal and the manifest, re-derives from the geometry
which tensors every file must hold (names, dtypes, shapes, for the expert split the manifest names), compares every header
with it and with the manifest's record (header digest, a content digest per tensor), re-hashes the listed files whole
(default: all; ``rehash=False`` leaves the payload to the per-tensor digests the loader checks while it streams) and
compares optional pins (manifest digest).  Any difference raises ``CheckpointValidationError``.

Parity: reference ``glm_tpu/model_loader/sharded_state/verify.py:156-323``.
"""

from __future__ import annotations

import json
from pathlib import Path

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader import placement
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.model_loader.sharded_state import manifest as manifest_mod
from glm_tpu_b200.model_loader.sharded_state import seal as seal_mod


def read_geometry(target: Path) -> ModelGeometry:
    raw = seal_mod.read_json_object(Path(target) / fmt.GEOMETRY_FILE, "the geometry file")
    try:
        for key in ("indexer_types", "mlp_layer_types", "fp8_block_shape", "eos_ids"):
            raw[key] = tuple(raw[key])
        return ModelGeometry(**raw)
    except (KeyError, TypeError, ValueError) as exc:
        raise CheckpointValidationError(f"the geometry file does not describe a model geometry: {exc}") from None


def verify_runtime_checkpoint(target: Path, files: list | None = None, pins: dict | None = None, rehash: bool = True) -> dict:
    target = Path(target)
    seal, manifest = seal_mod.read_seal(target)
    geometry = read_geometry(target)
    if geometry.geometry_hash != manifest["geometry_sha256"] or manifest["geometry_sha256"] != seal["geometry_sha256"]:
        raise CheckpointValidationError("geometry, manifest and seal disagree")
    if pins and pins.get("manifest_sha256") not in (None, "", seal["manifest_sha256"]):
        raise CheckpointValidationError("the checkpoint is not the pinned one")
    world = manifest["world"]
    split = manifest.get("expert_split", "whole")
    if manifest.get("format") != fmt.FORMAT_VERSION:
        raise CheckpointValidationError(f"the checkpoint was packed as {manifest.get('format')!r}; this loader reads {fmt.FORMAT_VERSION!r}")
    if sorted(manifest["files"]) != sorted(manifest_mod.expected_files(world)):
        raise CheckpointValidationError("the manifest does not list exactly the files of this world size")
    checked = []
    for name in files if files is not None else sorted(manifest["files"]):
        record = manifest["files"].get(name)
        if record is None:
            raise CheckpointValidationError(f"{name} is not part of this checkpoint")
        path = target / name
        if not path.is_file() or path.stat().st_size != record["size"]:
            raise CheckpointValidationError(f"{name}: missing or wrong size")
        header, _ = fmt.read_header(path)
        meta = header.get("__metadata__", {})
        if (meta.get("format") != fmt.FORMAT_VERSION or meta.get("geometry_sha256") != geometry.geometry_hash or meta.get("world") != str(world)
                or meta.get("expert_split") != split):
            raise CheckpointValidationError(f"{name}: foreign or stale file (metadata differs)")
        rank = None if name == fmt.SHARED_FILE else int(name.split("rank")[1].split("of")[0])
        want = placement.packed_tensor_shapes(geometry, world, rank, split)
        have = {n: (e["dtype"], tuple(e["shape"])) for n, e in header.items() if n != "__metadata__"}
        if have != {n: (d, tuple(s)) for n, (d, s) in want.items()}:
            raise CheckpointValidationError(f"{name}: tensor list differs from the placement plan")
        recorded = {n: (t["dtype"], tuple(t["shape"])) for n, t in record["tensors"].items()}
        if recorded != have or any(not t.get("sha256") for t in record["tensors"].values()):
            raise CheckpointValidationError(f"{name}: the manifest's tensor records differ from the header")
        head, _, _ = fmt.layout({n: (e["dtype"], e["shape"]) for n, e in header.items() if n != "__metadata__"}, meta)
        import hashlib

        if hashlib.sha256(head).hexdigest() != record.get("header_sha256"):
            raise CheckpointValidationError(f"{name}: the header is not the canonical one the manifest recorded")
        if rehash and fmt.file_sha256(path) != record["sha256"]:
            raise CheckpointValidationError(f"{name}: content digest differs from the manifest")
        checked.append(name)
    return {"ok": True, "files": checked, "manifest_sha256": seal["manifest_sha256"], "world": world, "geometry_sha256": geometry.geometry_hash,
            "expert_split": split, "manifest_files": manifest["files"]}
