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


def read_source_pieces(inv: SourceInventory, name: str, piece_bytes: int | None = None, rows: tuple | None = None):
    """The source tensor ``name`` (or its rows ``[rows[0], rows[1])``) as a sequence of flat CPU tensors of at most
    ``piece_bytes`` bytes each (whole elements), front to back: a large table passes through without ever being whole in memory."""
    import os

    import torch

    t = inv.tensors[name]
    dtype, item = fmt.DTYPES[t.dtype]
    cap = piece_bytes or fmt.PIECE_BYTES
    cap -= cap % item
    first, last = t.begin, t.end
    if rows is not None:
        row_bytes = (t.end - t.begin) // max(t.shape[0], 1)
        if not 0 <= rows[0] <= rows[1] <= t.shape[0]:
            raise CheckpointValidationError(f"rows {rows} outside {name!r}")
        first, last = t.begin + rows[0] * row_bytes, t.begin + rows[1] * row_bytes
    fd = os.open(inv.root / t.shard, os.O_RDONLY)
    try:
        at = first
        while at < last:
            n = min(cap, last - at)
            buf = bytearray(n)
            view, got = memoryview(buf), 0
            while got < n:
                k = os.preadv(fd, [view[got:]], at + got)
                if k <= 0:
                    raise CheckpointValidationError(f"short read for {name!r}")
                got += k
            yield torch.frombuffer(buf, dtype=dtype)
            at += n
    finally:
        os.close(fd)


def read_source_tensor(inv: SourceInventory, name: str, rows: tuple | None = None):
    """One whole source tensor, or a run of its rows (an expert's table, a scale table: tens of megabytes at most)."""
    import torch

    t = inv.tensors[name]
    parts = list(read_source_pieces(inv, name, rows=rows))
    flat = parts[0] if len(parts) == 1 else (torch.cat(parts) if parts else torch.empty(0, dtype=fmt.DTYPES[t.dtype][0]))
    shape = t.shape if rows is None else (rows[1] - rows[0], *t.shape[1:])
    return flat.reshape(shape)
