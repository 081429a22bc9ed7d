"""The on-disk tensor container (safetensors layout) with a canonical header, and the packed-checkpoint file names.

A file is ``u64 little-endian header length | JSON header | raw tensor bytes``.  The header maps each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header) plus ``__metadata__``
(string to string).  Files written here are *canonical*: names sorted, tensors laid out in that order without gaps,
header JSON compact with sorted keys and padded with spaces to a multiple of 8 bytes -- so equal contents give equal
bytes and equal hashes on every machine.

A packed checkpoint directory holds ``shared.safetensors`` (every non-routed tensor, FP8 pairs kept as stored),
``experts.rank<r>of<w>.safetensors`` (the routed experts of GPU r, stacked ``[experts_local, N, K]``), ``geometry.json``,
``manifest.json`` and the ``SUCCESS`` seal.  FP8 payloads containing an e4m3fn NaN code (0x7F / 0xFF) are refused.

Parity: reference ``glm_tpu/model_loader/sharded_state/format.py:195-324`` (canonical header, metadata, NaN refusal).
"""

from __future__ import annotations

import hashlib
import json
import struct
from pathlib import Path

import torch

from glm_tpu_b200.exceptions import CheckpointValidationError

FORMAT_VERSION = "glm_b200_packed_v1"
SHARED_FILE = "shared.safetensors"
GEOMETRY_FILE = "geometry.json"
MANIFEST_FILE = "manifest.json"
SEAL_FILE = "SUCCESS"
HEADER_CAP = 100 << 20

DTYPES = {
    "F8_E4M3": (torch.uint8, 1),  # kept as raw bits
    "U8": (torch.uint8, 1),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
TORCH_TO_NAME = {torch.uint8: "U8", torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32",
                 torch.int64: "I64"}


def expert_file(rank: int, world: int) -> str:
    return f"experts.rank{rank}of{world}.safetensors"


def read_header(path: Path) -> tuple[dict, int]:
    """``(header, data_start)``; bounded and validated (offsets contiguous, inside the file, sizes match shapes)."""
    path = Path(path)
    size = path.stat().st_size
    with path.open("rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise CheckpointValidationError(f"{path.name}: truncated header length")
        (n,) = struct.unpack("<Q", raw)
        if not 2 <= n <= min(HEADER_CAP, size - 8):
            raise CheckpointValidationError(f"{path.name}: implausible header length {n}")
        try:
            header = json.loads(f.read(n))
        except ValueError as exc:
            raise CheckpointValidationError(f"{path.name}: header is not JSON") from exc
    if type(header) is not dict:
        raise CheckpointValidationError(f"{path.name}: header must be an object")
    start = 8 + n
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (begin, end) = entry["dtype"], entry["shape"], entry["data_offsets"]
        except (KeyError, TypeError, ValueError) as exc:
            raise CheckpointValidationError(f"{path.name}: malformed entry for {name!r}") from exc
        if dtype not in DTYPES:
            raise CheckpointValidationError(f"{path.name}: unsupported dtype {dtype} for {name!r}")
        count = 1
        for d in shape:
            if type(d) is not int or d < 0:
                raise CheckpointValidationError(f"{path.name}: bad shape for {name!r}")
            count *= d
        if end - begin != count * DTYPES[dtype][1] or begin < 0 or start + end > size:
            raise CheckpointValidationError(f"{path.name}: data range of {name!r} does not match its shape or the file")
    return header, start


def read_tensor(path: Path, header: dict, start: int, name: str) -> torch.Tensor:
    entry = header[name]
    begin, end = entry["data_offsets"]
    dtype = DTYPES[entry["dtype"]][0]
    with Path(path).open("rb") as f:
        f.seek(start + begin)
        raw = f.read(end - begin)
    if len(raw) != end - begin:
        raise CheckpointValidationError(f"{Path(path).name}: short read for {name!r}")
    t = torch.frombuffer(bytearray(raw), dtype=dtype) if raw else torch.empty(0, dtype=dtype)
    return t.reshape(entry["shape"])


def refuse_fp8_nan(name: str, bits: torch.Tensor) -> None:
    if bool(((bits & 0x7F) == 0x7F).any()):
        raise CheckpointValidationError(f"{name}: the FP8 payload contains an e4m3fn NaN code")


def write_file(path: Path, tensors: dict, metadata: dict, fp8_names: set | None = None) -> dict:
    """Write ``tensors`` canonically to ``path + '.partial'``, fsync, rename.  Returns ``{"sha256", "size", "tensors"}``."""
    path = Path(path)
    fp8_names = fp8_names or set()
    names = sorted(tensors)
    header: dict = {"__metadata__": {str(k): str(v) for k, v in sorted(metadata.items())}}
    offset = 0
    for name in names:
        t = tensors[name]
        dtype = "F8_E4M3" if name in fp8_names else TORCH_TO_NAME[t.dtype]
        if name in fp8_names:
            refuse_fp8_nan(name, t)
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": dtype, "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, sort_keys=True, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    partial = path.with_name(path.name + ".partial")
    digest = hashlib.sha256()
    with partial.open("wb") as f:
        for chunk in (struct.pack("<Q", len(raw)), raw):
            f.write(chunk)
            digest.update(chunk)
        for name in names:
            data = tensors[name].contiguous().cpu()
            buf = data.view(torch.uint8).numpy().tobytes() if data.numel() else b""
            f.write(buf)
            digest.update(buf)
        f.flush()
        import os

        os.fsync(f.fileno())
    partial.replace(path)
    return {"sha256": digest.hexdigest(), "size": 8 + len(raw) + offset,
            "tensors": {n: {"dtype": header[n]["dtype"], "shape": header[n]["shape"]} for n in names}}


def file_sha256(path: Path, chunk: int = 8 << 20) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as f:
        while True:
            buf = f.read(chunk)
            if not buf:
                break
            digest.update(buf)
    return digest.hexdigest()
