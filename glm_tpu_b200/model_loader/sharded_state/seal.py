"""The ``SUCCESS`` seal: a self-hashed record that names the manifest it closes.

A checkpoint directory is usable only if ``SUCCESS`` exists, its own digest matches its body, and the manifest it
names is the one on disk.  The seal is installed last and create-once; a failed pack therefore never looks complete.

Parity: reference ``glm_tpu/model_loader/sharded_state/seal.py:43-241``.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.utils.io_utils import create_private_exclusive
from glm_tpu_b200.utils.json_utils import canonical_hash_bytes, canonical_wire_bytes


def success_record(manifest: dict) -> dict:
    body = {"schema": "glm_b200_seal_v1", "manifest_sha256": hashlib.sha256(canonical_hash_bytes(manifest)).hexdigest(),
            "geometry_sha256": manifest["geometry_sha256"], "world": manifest["world"], "total_bytes": manifest["total_bytes"]}
    return dict(body, seal_sha256=hashlib.sha256(canonical_hash_bytes(body)).hexdigest())


def install(target: Path, geometry, manifest: dict) -> dict:
    target = Path(target)
    create_private_exclusive(target / fmt.GEOMETRY_FILE, canonical_wire_bytes(geometry.as_dict()) + b"\n")
    create_private_exclusive(target / fmt.MANIFEST_FILE, canonical_wire_bytes(manifest) + b"\n")
    seal = success_record(manifest)
    create_private_exclusive(target / fmt.SEAL_FILE, canonical_wire_bytes(seal) + b"\n")
    return seal


SEAL_KEYS = ("schema", "manifest_sha256", "geometry_sha256", "world", "total_bytes", "seal_sha256")


def read_json_object(path: Path, what: str) -> dict:
    """A JSON object from ``path``; anything else (absent, unreadable, not JSON, not an object) is a validation error."""
    try:
        value = json.loads(path.read_text())
    except FileNotFoundError:
        raise CheckpointValidationError(f"{what} is missing") from None
    except (OSError, UnicodeDecodeError, ValueError) as exc:
        raise CheckpointValidationError(f"{what} cannot be read as JSON: {exc}") from None
    if not isinstance(value, dict):
        raise CheckpointValidationError(f"{what} is not a JSON object")
    return value


def read_seal(target: Path) -> tuple[dict, dict]:
    """``(seal, manifest)`` after checking that both are self-consistent and belong together: the seal has exactly its keys and
    hashes to its own digest, the manifest on disk hashes to the digest the seal names, and the facts both state (geometry,
    GPU count, total bytes) are equal."""
    target = Path(target)
    if not (target / fmt.SEAL_FILE).exists():
        raise CheckpointValidationError("no SUCCESS seal: the checkpoint was never completed")
    seal = read_json_object(target / fmt.SEAL_FILE, "the SUCCESS seal")
    if sorted(seal) != sorted(SEAL_KEYS) or seal["schema"] != "glm_b200_seal_v1":
        raise CheckpointValidationError("the SUCCESS seal is not a glm_b200_seal_v1 record")
    body = {k: v for k, v in seal.items() if k != "seal_sha256"}
    if seal["seal_sha256"] != hashlib.sha256(canonical_hash_bytes(body)).hexdigest():
        raise CheckpointValidationError("the SUCCESS seal does not match its own digest")
    manifest = read_json_object(target / fmt.MANIFEST_FILE, "the manifest")
    if hashlib.sha256(canonical_hash_bytes(manifest)).hexdigest() != seal["manifest_sha256"]:
        raise CheckpointValidationError("the manifest on disk is not the one the seal closes")
    for key in ("geometry_sha256", "world", "total_bytes"):
        if manifest.get(key) != seal[key]:
            raise CheckpointValidationError(f"seal and manifest state different {key}")
    return seal, manifest
