"""Inventory of a Hugging Face source checkpoint, read from the safetensors headers only.

``read_source_inventory(dir)`` opens ``model.safetensors.index.json`` (if present) and every ``*.safetensors`` shard,
reads only the headers and returns every tensor with its dtype, shape, shard and byte range, the shard sizes, and a
content address: the SHA-256 of the canonical JSON of that listing.  Nothing of the payload is read, so a 756 GB
checkpoint is inventoried in seconds.  ``authenticated_inventory`` re-reads and refuses a drift from a pinned digest.

Parity: reference ``glm_tpu/model_loader/source_inventory.py:429-561``.
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from pathlib import Path

from glm_tpu_b200.exceptions import CheckpointValidationError
from glm_tpu_b200.model_loader.sharded_state import format as fmt
from glm_tpu_b200.utils.json_utils import canonical_hash_bytes

INDEX_FILE = "model.safetensors.index.json"


@dataclass(frozen=True)
class SourceTensor:
    name: str
    dtype: str
    shape: tuple
    shard: str
    begin: int  # absolute file offset
    end: int


@dataclass(frozen=True)
class SourceInventory:
    root: Path
    tensors: dict  # name -> SourceTensor
    shards: dict  # file name -> size in bytes
    sha256: str

    def listing(self) -> dict:
        return {"tensors": {n: [t.dtype, list(t.shape), t.shard, t.begin, t.end] for n, t in sorted(self.tensors.items())},
                "shards": dict(sorted(self.shards.items()))}


def read_source_inventory(root: Path) -> SourceInventory:
    root = Path(root)
    index = root / INDEX_FILE
    if index.exists():
        weight_map = json.loads(index.read_text())["weight_map"]
        shard_names = sorted(set(weight_map.values()))
    else:
        weight_map = None
        shard_names = sorted(p.name for p in root.glob("*.safetensors"))
    if not shard_names:
        raise CheckpointValidationError(f"{root} holds no safetensors shards")
    tensors, shards = {}, {}
    for shard in shard_names:
        path = root / shard
        if not path.is_file():
            raise CheckpointValidationError(f"shard {shard} named by the index is missing")
        header, start = fmt.read_header(path)
        shards[shard] = path.stat().st_size
        for name, entry in header.items():
            if name == "__metadata__":
                continue
            if name in tensors:
                raise CheckpointValidationError(f"tensor {name!r} appears in two shards")
            if weight_map is not None and weight_map.get(name) != shard:
                raise CheckpointValidationError(f"tensor {name!r} is not where the index says")
            begin, end = entry["data_offsets"]
            tensors[name] = SourceTensor(name, entry["dtype"], tuple(entry["shape"]), shard, start + begin, start + end)
    if weight_map is not None and set(weight_map) != set(tensors):
        missing = sorted(set(weight_map) - set(tensors))[:3]
        raise CheckpointValidationError(f"the index names tensors that no shard holds: {missing}")
    listing = {"tensors": {n: [t.dtype, list(t.shape), t.shard, t.begin, t.end] for n, t in sorted(tensors.items())},
               "shards": dict(sorted(shards.items()))}
    return SourceInventory(root, tensors, shards, hashlib.sha256(canonical_hash_bytes(listing)).hexdigest())


def authenticated_inventory(root: Path, expected_sha256: str) -> SourceInventory:
    inv = read_source_inventory(root)
    if inv.sha256 != expected_sha256:
        raise CheckpointValidationError("the source checkpoint differs from the pinned inventory")
    return inv


def read_source_tensor(inv: SourceInventory, name: str):
    import torch

    t = inv.tensors[name]
    dtype = fmt.DTYPES[t.dtype][0]
    with (inv.root / t.shard).open("rb") as f:
        f.seek(t.begin)
        raw = f.read(t.end - t.begin)
    if len(raw) != t.end - t.begin:
        raise CheckpointValidationError(f"short read for {name!r}")
    return torch.frombuffer(bytearray(raw), dtype=dtype).reshape(t.shape) if raw else torch.empty(t.shape, dtype=dtype)
