"""Owner-only, create-once file I/O for run directories and checkpoints.

* ``create_private_exclusive``: 0600, ``O_EXCL | O_NOFOLLOW``; never replaces anything.
* ``write_collected``: store a record fetched from a rank exactly once; an equal record is
  skipped, a different one is kept beside it under ``final/`` and reported as divergent.
* ``read_bounded``: read a regular file of 1..cap bytes without following symlinks or blocking.
* ``atomic_json`` / ``persist_json``: write-to-temp, fsync, rename.
* ``require_private``: refuse a path that others can read or write.

Parity: reference ``glm_tpu/utils/io_utils.py:28-148``.
"""

from __future__ import annotations

import json
import os
import stat
from pathlib import Path

FINAL_DIR = "final"


def create_private_exclusive(path: Path, payload: bytes) -> None:
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL | os.O_NOFOLLOW, 0o600)
    try:
        done = 0
        while done < len(payload):
            done += os.write(fd, payload[done:])
        os.fsync(fd)
    finally:
        os.close(fd)


def _holds(path: Path, payload: bytes) -> bool:
    try:
        if not stat.S_ISREG(os.lstat(path).st_mode):
            return False
        current = path.read_bytes()
    except FileNotFoundError:
        return False
    if current == payload:
        return True
    try:
        return json.loads(current) == json.loads(payload)
    except ValueError:
        return False


def write_collected(root: Path, name: str, payload: bytes, divergent: list[str]) -> None:
    if not name or name in (".", "..") or "/" in name or "\0" in name:
        raise ValueError(f"collected record name {name!r} must be a plain file name")
    root = Path(root)
    try:
        create_private_exclusive(root / name, payload)
        return
    except FileExistsError:
        if _holds(root / name, payload):
            return
    keep = root / FINAL_DIR
    keep.mkdir(mode=0o700, exist_ok=True)
    index = 0
    while True:
        candidate = keep / (name if index == 0 else f"{name}.{index}")
        try:
            create_private_exclusive(candidate, payload)
            break
        except FileExistsError:
            if _holds(candidate, payload):
                break
            index += 1
    if name not in divergent:
        divergent.append(name)


def plain_path(path: Path) -> Path:
    path = Path(path).absolute()
    for part in (path, *path.parents):
        if part.is_symlink():
            raise ValueError("paths must not traverse symlinks")
    return path


def read_bounded(path: Path, cap: int) -> bytes:
    path = plain_path(path)
    fd = os.open(path, os.O_RDONLY | os.O_NOFOLLOW | os.O_NONBLOCK)
    try:
        facts = os.fstat(fd)
        if not stat.S_ISREG(facts.st_mode) or not 0 < facts.st_size <= cap:
            raise ValueError("input is not a bounded regular file")
        chunks, total = [], 0
        while total <= cap:
            chunk = os.read(fd, min(1 << 20, cap + 1 - total))
            if not chunk:
                break
            chunks.append(chunk)
            total += len(chunk)
    finally:
        os.close(fd)
    raw = b"".join(chunks)
    if not 0 < len(raw) <= cap:
        raise ValueError("input changed beyond its byte cap")
    return raw


def atomic_json(path: Path, value) -> None:
    path = Path(path)
    tmp = path.with_name(path.name + ".tmp")
    fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
    with os.fdopen(fd, "w", encoding="utf-8") as stream:
        json.dump(value, stream, ensure_ascii=False)
        stream.flush()
        os.fsync(stream.fileno())
    tmp.replace(path)


def persist_json(path: Path, value) -> None:
    path = Path(path)
    tmp = path.with_name(path.name + ".tmp")
    with tmp.open("w", encoding="utf-8") as stream:
        json.dump(value, stream, sort_keys=True, indent=2)
        stream.write("\n")
        stream.flush()
        os.fsync(stream.fileno())
    tmp.replace(path)


def require_private(path: Path) -> None:
    plain_path(path)
    info = Path(path).stat()
    if info.st_uid != os.geteuid() or stat.S_IMODE(info.st_mode) & 0o077:
        raise ValueError(f"{path} must be owned by this user and closed to group and others")
