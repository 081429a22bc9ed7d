"""The on-disk tensor container (safetensors layout) with a canonical header, and the packed-checkpoint file names.

A file is ``u64 little-endian header length | JSON header | raw tensor bytes``.  The header maps each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the header) plus ``__metadata__``
(string to string).  Files written here are *canonical*: names sorted, tensors laid out in that order without gaps,
header JSON compact with sorted keys and padded with spaces to a multiple of 8 bytes -- so equal contents give equal
bytes and equal hashes on every machine.

Nothing here holds a whole file, or even a whole large tensor, in host memory.  ``FileWriter`` lays the file out from
the shapes alone, then takes each tensor as a sequence of pieces that are checked (FP8 NaN codes, finiteness), hashed
and written at their final offset as they arrive; ``TensorReader`` streams a tensor in pieces of at most ``PIECE_BYTES``
through one reusable (pinned, when a GPU is the destination) buffer, hashing and checking every piece on its way, and
compares the digest with the one the manifest recorded for that tensor.  A checkpoint is therefore read exactly once
on its way to the device and every byte of it is authenticated by the chain pin -> manifest -> tensor digest.

A packed checkpoint directory holds ``shared.safetensors`` (every non-routed tensor, FP8 pairs kept as stored),
``experts.rank<r>of<w>.safetensors`` (the routed experts' part of GPU r: whole experts ``[experts_local, N, K]`` or a
column slice of every expert), ``geometry.json``, ``manifest.json`` and the ``SUCCESS`` seal.  FP8 payloads containing
an e4m3fn NaN code (0x7F / 0xFF) are refused.

Parity: reference ``glm_tpu/model_loader/sharded_state/format.py:195-324`` (canonical header, metadata, NaN refusal).
"""

from __future__ import annotations

import hashlib
import json
import os
import struct
from pathlib import Path

import torch

from glm_tpu_b200.exceptions import CheckpointValidationError

FORMAT_VERSION = "glm_b200_packed_v2"
SHARED_FILE = "shared.safetensors"
GEOMETRY_FILE = "geometry.json"
MANIFEST_FILE = "manifest.json"
SEAL_FILE = "SUCCESS"
HEADER_CAP = 100 << 20
PIECE_BYTES = 256 << 20  # the most that is read, checked or written in one go

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
FLOAT_NAMES = ("BF16", "F16", "F32")


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
    ranges = []
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
        ranges.append((begin, end, name))
    # the payload is the tensors back to back: no overlap, no gap, nothing after the last one
    at = 0
    for begin, end, name in sorted(ranges):
        if begin != at:
            raise CheckpointValidationError(f"{path.name}: {name!r} starts at {begin}, {'overlapping' if begin < at else 'leaving a gap after'} byte {at}")
        at = end
    if start + at != size:
        raise CheckpointValidationError(f"{path.name}: {size - start - at} bytes follow the last tensor")
    return header, start


def refuse_fp8_nan(name: str, bits: torch.Tensor) -> None:
    if bool(((bits & 0x7F) == 0x7F).any()):
        raise CheckpointValidationError(f"{name}: the FP8 payload contains an e4m3fn NaN code")


def check_piece(name: str, dtype_name: str, piece: torch.Tensor) -> None:
    """``piece``: raw bytes (uint8, any device) of a run of whole elements of ``name``."""
    if dtype_name == "F8_E4M3":
        refuse_fp8_nan(name, piece)
    elif dtype_name in FLOAT_NAMES and piece.numel():
        if not bool(torch.isfinite(piece.view(DTYPES[dtype_name][0]).float()).all()):
            raise CheckpointValidationError(f"{name}: non-finite values")


def layout(specs: dict, metadata: dict) -> tuple[bytes, dict, int]:
    """The canonical header of a file holding ``specs`` (``name -> (dtype name, shape)``): ``(header bytes incl. the length
    word, name -> (begin, end) relative to the end of the header, payload bytes)``."""
    header: dict = {"__metadata__": {str(k): str(v) for k, v in sorted(metadata.items())}}
    ranges, offset = {}, 0
    for name in sorted(specs):
        dtype, shape = specs[name]
        count = 1
        for d in shape:
            count *= int(d)
        nbytes = count * DTYPES[dtype][1]
        header[name] = {"dtype": dtype, "shape": [int(d) for d in shape], "data_offsets": [offset, offset + nbytes]}
        ranges[name] = (offset, offset + nbytes)
        offset += nbytes
    raw = json.dumps(header, sort_keys=True, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    return struct.pack("<Q", len(raw)) + raw, ranges, offset


class FileWriter:
    """Writes one canonical file piece by piece: ``FileWriter(path, specs, metadata)``, then for every tensor any number of
    ``append(name, piece)`` calls that together cover it front to back, then ``close()`` -> the receipt.

    The bytes go to ``path + '.partial'`` (created exclusively, sized up front) at their final offsets, so tensors may be
    filled in any order and nothing is stacked in memory first.  Every piece is checked and enters its tensor's running
    SHA-256.  ``close`` refuses an incompletely covered tensor, syncs, re-reads the file from disk for the whole-file digest
    and only then renames it into place."""

    def __init__(self, path: Path, specs: dict, metadata: dict):
        self.path = Path(path)
        self.partial = self.path.with_name(self.path.name + ".partial")
        self.specs = {n: (d, tuple(int(x) for x in shape)) for n, (d, shape) in specs.items()}
        self.head, self.ranges, self.payload = layout(self.specs, metadata)
        self._fd = os.open(self.partial, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o600)
        os.pwrite(self._fd, self.head, 0)
        os.ftruncate(self._fd, len(self.head) + self.payload)
        self._filled = {n: 0 for n in self.specs}
        self._digests = {n: hashlib.sha256() for n in self.specs}

    def append(self, name: str, piece: torch.Tensor) -> None:
        dtype, _ = self.specs[name]
        begin, end = self.ranges[name]
        data = piece.contiguous().cpu()
        if DTYPES[dtype][0] != data.dtype:
            raise CheckpointValidationError(f"{name}: a {data.dtype} piece for a {dtype} tensor")
        raw_all = data.reshape(-1).view(torch.uint8)
        if self._filled[name] + raw_all.numel() > end - begin:
            raise CheckpointValidationError(f"{name}: more bytes than its shape holds")
        for lo in range(0, raw_all.numel(), PIECE_BYTES):
            raw = raw_all[lo : lo + PIECE_BYTES]
            check_piece(name, dtype, raw)
            buf = memoryview(raw.numpy())
            self._digests[name].update(buf)
            at = len(self.head) + begin + self._filled[name]
            done = 0
            while done < len(buf):
                done += os.pwrite(self._fd, buf[done:], at + done)
            self._filled[name] += len(buf)

    def close(self) -> dict:
        try:
            short = [n for n, (b, e) in self.ranges.items() if self._filled[n] != e - b]
            if short:
                raise CheckpointValidationError(f"{self.path.name}: {len(short)} tensors were not written completely, e.g. {short[:3]}")
            os.fsync(self._fd)
        finally:
            os.close(self._fd)
        sha = file_sha256(self.partial)  # what reached the disk
        self.partial.replace(self.path)
        return {"sha256": sha, "size": len(self.head) + self.payload, "header_sha256": hashlib.sha256(self.head).hexdigest(),
                "tensors": {n: {"dtype": d, "shape": list(shape), "sha256": self._digests[n].hexdigest()} for n, (d, shape) in sorted(self.specs.items())}}

    def abort(self) -> None:
        try:
            os.close(self._fd)
        except OSError:
            pass
        self.partial.unlink(missing_ok=True)


def write_file(path: Path, tensors: dict, metadata: dict, fp8_names: set | None = None) -> dict:
    """Write whole in-memory ``tensors`` canonically (fixtures, exports).  Returns the receipt of ``FileWriter.close``."""
    fp8_names = fp8_names or set()
    specs = {n: ("F8_E4M3" if n in fp8_names else TORCH_TO_NAME[t.dtype], tuple(t.shape)) for n, t in tensors.items()}
    w = FileWriter(path, specs, metadata)
    try:
        for name in sorted(tensors):
            w.append(name, tensors[name])
        return w.close()
    except BaseException:
        w.abort()
        raise


class TensorReader:
    """Streams tensors out of one file.  ``read(name, device=..., expect_sha256=...)`` allocates the destination, then moves
    the tensor there in pieces of at most ``PIECE_BYTES`` through one reusable staging buffer (pinned when the destination is
    a GPU); every piece is hashed on the host and checked (FP8 NaN codes, finiteness) where it lands."""

    def __init__(self, path: Path, header: dict | None = None, start: int | None = None):
        self.path = Path(path)
        if header is None:
            header, start = read_header(self.path)
        self.header, self.start = header, start
        self._fd = os.open(self.path, os.O_RDONLY)
        self._stage = None
        self.bytes_read = 0
        self.largest_piece = 0

    def names(self) -> list:
        return [n for n in self.header if n != "__metadata__"]

    def close(self) -> None:
        if self._fd is not None:
            os.close(self._fd)
            self._fd = None
        self._stage = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    def _staging(self, nbytes: int, pinned: bool) -> torch.Tensor:
        want = min(PIECE_BYTES, max(nbytes, 1))
        if self._stage is None or self._stage.numel() < want or (pinned and not self._stage.is_pinned()):
            self._stage = torch.empty(want, dtype=torch.uint8, pin_memory=pinned)
        return self._stage

    def read(self, name: str, *, device=None, expect_sha256: str | None = None, check: bool = True) -> torch.Tensor:
        entry = self.header[name]
        begin, end = entry["data_offsets"]
        dtype_name = entry["dtype"]
        dtype, item = DTYPES[dtype_name]
        dev = torch.device(device) if device is not None else torch.device("cpu")
        nbytes = end - begin
        out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        digest = hashlib.sha256()
        piece_cap = PIECE_BYTES - PIECE_BYTES % item
        on_gpu = dev.type == "cuda"
        stage = self._staging(nbytes, on_gpu) if on_gpu else None
        done = 0
        while done < nbytes:
            n = min(piece_cap, nbytes - done)
            target = stage[:n] if on_gpu else out[done : done + n]
            view = memoryview(target.numpy())
            got = 0
            while got < n:
                k = os.preadv(self._fd, [view[got:]], self.start + begin + done + got)
                if k <= 0:
                    raise CheckpointValidationError(f"{self.path.name}: short read for {name!r}")
                got += k
            digest.update(view)
            if on_gpu:
                out[done : done + n].copy_(target, non_blocking=True)
                if check and (dtype_name == "F8_E4M3" or dtype_name in FLOAT_NAMES):
                    check_piece(name, dtype_name, out[done : done + n])  # on the device; reading the verdict also waits for the copy
                else:
                    torch.cuda.current_stream(dev).synchronize()  # the staging buffer is reused by the next piece
            elif check:
                check_piece(name, dtype_name, target)
            done += n
            self.bytes_read += n
            self.largest_piece = max(self.largest_piece, n)
        if expect_sha256 is not None and digest.hexdigest() != expect_sha256:
            raise CheckpointValidationError(f"{self.path.name}: content digest of {name!r} differs from the manifest")
        return out.view(dtype).reshape(entry["shape"])


def read_tensor(path: Path, header: dict, start: int, name: str) -> torch.Tensor:
    """One tensor on the CPU (small files and tests; the loader streams through a ``TensorReader`` it keeps open)."""
    reader = TensorReader(path, header, start)
    try:
        return reader.read(name)
    finally:
        reader.close()


def file_sha256(path: Path, chunk: int = 8 << 20) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as f:
        while True:
            buf = f.read(chunk)
            if not buf:
                break
            digest.update(buf)
    return digest.hexdigest()
