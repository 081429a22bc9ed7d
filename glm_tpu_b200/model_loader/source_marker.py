"""``SOURCE_COMPLETE.json``: the marker that a downloaded source checkpoint is whole.

``mark_source`` re-reads the inventory, checks every shard against the expected sizes / SHA-256 digests when a
``checksums.json`` (``{file: {"size": n, "sha256": hex}}``, e.g. exported from the hub's LFS pointers) is present, hashes
the small configuration files, and writes the marker create-once.  Packing refuses a source without a valid marker.

Parity: reference ``glm_tpu/model_loader/source_marker.py:138-243``.
"""

from __future__ import annotations

import json
from pathlib import Path

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader import source_inventory
from glm_tpu_b200.model_loader.sharded_state.format import file_sha256
from glm_tpu_b200.utils.io_utils import create_private_exclusive
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

MARKER_FILE = "SOURCE_COMPLETE.json"
CHECKSUMS_FILE = "checksums.json"
SMALL_FILES = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "chat_template.jinja",
               source_inventory.INDEX_FILE)


def compute_marker(root: Path, *, hash_shards: bool = False) -> dict:
    """The marker record of ``root`` as it is now; nothing is written."""
    root = Path(root)
    inv = source_inventory.read_source_inventory(root)
    expected = json.loads((root / CHECKSUMS_FILE).read_text()) if (root / CHECKSUMS_FILE).exists() else {}
    files = {}
    for shard, size in inv.shards.items():
        record = {"size": size}
        want = expected.get(shard)
        if want is not None and want.get("size") not in (None, size):
            raise CheckpointValidationError(f"{shard}: size {size} differs from the expected {want['size']}")
        if hash_shards or (want is not None and want.get("sha256")):
            record["sha256"] = file_sha256(root / shard)
            if want is not None and want.get("sha256") not in (None, record["sha256"]):
                raise CheckpointValidationError(f"{shard}: content differs from the expected digest")
        files[shard] = record
    small = {name: file_sha256(root / name) for name in SMALL_FILES if (root / name).exists()}
    return {"schema": "glm_b200_source_marker_v1", "inventory_sha256": inv.sha256, "tensor_count": len(inv.tensors),
            "total_bytes": sum(inv.shards.values()), "shards": files, "small_files": small}


def mark_source(root: Path, *, hash_shards: bool = False) -> dict:
    marker = compute_marker(root, hash_shards=hash_shards)
    create_private_exclusive(Path(root) / MARKER_FILE, canonical_wire_bytes(marker) + b"\n")
    return marker


def differences(mine: dict, upstream: dict) -> list[str]:
    """In which respects this copy of a source differs from the copy another marker describes: the tensor inventory, the shard
    list and sizes, shard digests where both markers carry one, and the small files.  An empty list: the same source."""
    if not isinstance(upstream, dict) or upstream.get("schema") != "glm_b200_source_marker_v1":
        return ["the upstream file is not a glm_b200_source_marker_v1 record"]
    out = []
    for key in ("inventory_sha256", "tensor_count", "total_bytes"):
        if mine.get(key) != upstream.get(key):
            out.append(f"{key}: {mine.get(key)} here, {upstream.get(key)} upstream")
    theirs = upstream.get("shards") if isinstance(upstream.get("shards"), dict) else {}
    for name in sorted(set(mine["shards"]) | set(theirs)):
        a, b = mine["shards"].get(name), theirs.get(name)
        if a is None or b is None:
            out.append(f"{name}: only {'upstream' if a is None else 'here'}")
        elif a.get("size") != b.get("size"):
            out.append(f"{name}: {a.get('size')} bytes here, {b.get('size')} upstream")
        elif a.get("sha256") and b.get("sha256") and a["sha256"] != b["sha256"]:
            out.append(f"{name}: content differs")
    small = upstream.get("small_files") if isinstance(upstream.get("small_files"), dict) else {}
    for name in sorted(set(mine["small_files"]) | set(small)):
        if mine["small_files"].get(name) != small.get(name):
            out.append(f"{name}: {'differs' if name in mine['small_files'] and name in small else 'present on one side only'}")
    return out


def check_against_upstream(root: Path, upstream_marker: Path, *, output: Path | None = None, hash_shards: bool = False) -> dict:
    """Compare the source in ``root`` with the one ``upstream_marker`` (a ``SOURCE_COMPLETE.json`` made elsewhere) describes;
    refuses on any difference.  The record computed here goes to ``output`` (create-once) when one is given; the source
    directory itself is not written to."""
    try:
        upstream = json.loads(Path(upstream_marker).read_text())
    except (OSError, UnicodeDecodeError, ValueError) as exc:
        raise CheckpointValidationError(f"the upstream marker cannot be read as JSON: {exc}") from None
    wants_digests = isinstance(upstream, dict) and isinstance(upstream.get("shards"), dict) and any(
        isinstance(r, dict) and r.get("sha256") for r in upstream["shards"].values())
    mine = compute_marker(root, hash_shards=hash_shards or wants_digests)
    found = differences(mine, upstream)
    if found:
        raise CheckpointValidationError(f"this source differs from the upstream marker in {len(found)} respect(s): " + "; ".join(found[:5]))
    if output is not None:
        create_private_exclusive(Path(output), canonical_wire_bytes(mine) + b"\n")
    return {"matches_upstream": True, "upstream_marker_sha256": file_sha256(Path(upstream_marker)), "shards_compared_by_content": bool(wants_digests),
            "marker": mine}


def marker_sha256(root: Path) -> str:
    """SHA-256 of the marker file's bytes: what a site file pins as ``[checkpoint] source_marker_sha256``."""
    return file_sha256(Path(root) / MARKER_FILE)


def require_marker(root: Path, pin: str = "") -> dict:
    """The marker of ``root`` after checking it against ``pin`` (the digest of the marker file, when one is pinned) and against
    what is on disk now: the inventory (every tensor, every shard size) and
    the digests of the small files (configuration, tokenizer, template, index) it recorded.  The shards' contents are not read
    again here: their sizes and headers are part of the inventory, their bytes are hashed when they are packed."""
    root = Path(root)
    path = root / MARKER_FILE
    if not path.exists():
        raise CheckpointValidationError("the source has no SOURCE_COMPLETE.json: run `checkpoint mark-source` first")
    try:
        marker = json.loads(path.read_text())
    except (OSError, UnicodeDecodeError, ValueError) as exc:
        raise CheckpointValidationError(f"SOURCE_COMPLETE.json cannot be read as JSON: {exc}") from None
    if not isinstance(marker, dict) or marker.get("schema") != "glm_b200_source_marker_v1":
        raise CheckpointValidationError("SOURCE_COMPLETE.json is not a glm_b200_source_marker_v1 record")
    if pin and marker_sha256(root) != pin:
        raise CheckpointValidationError("the source's marker is not the pinned one ([checkpoint] source_marker_sha256)")
    inv = source_inventory.read_source_inventory(root)
    if marker.get("inventory_sha256") != inv.sha256:
        raise CheckpointValidationError("the source changed after it was marked complete")
    shards = marker.get("shards")
    if not isinstance(shards, dict) or {n: r.get("size") if isinstance(r, dict) else None for n, r in shards.items()} != dict(inv.shards):
        raise CheckpointValidationError("the marker's shard list differs from the source")
    small = marker.get("small_files")
    if not isinstance(small, dict):
        raise CheckpointValidationError("the marker lists no small files")
    present = {name for name in SMALL_FILES if (root / name).exists()}
    if present != set(small):
        raise CheckpointValidationError("configuration files were added or removed after the source was marked: "
                                        + ", ".join(sorted(present ^ set(small))))
    for name, digest in sorted(small.items()):
        if file_sha256(root / name) != digest:
            raise CheckpointValidationError(f"{name} changed after the source was marked complete")
    return marker
