"""File discipline of run directories and state directories: owner-only, create-once, never follow a link.

* ``create_private_exclusive`` makes a new 0600 file or fails; it cannot replace, truncate or follow anything that is already there.
* ``write_collected`` files a record that may arrive more than once (a resident run already holds its first records when the final
  collection brings the same names again).  The first arrival keeps the name.  A later arrival with the same bytes, or the same JSON
  value, changes nothing.  A later arrival that differs is kept beside it under ``final/`` and its name is reported, because a worker
  that failed late rewrites its record and both versions are evidence.
* ``read_bounded`` reads a regular file of 1..cap bytes through a descriptor opened without following links and without blocking on a
  FIFO; ``plain_path`` refuses a path that passes through a symbolic link anywhere.
* ``atomic_json`` / ``persist_json`` replace a JSON document by writing a sibling and renaming it.

Standard library only.  Behaviour parity: reference ``glm_tpu/utils/io_utils.py``.
"""

from __future__ import annotations

import json
import os
import stat
from pathlib import Path

FINAL_DIR = "final"
_CREATE_ONCE = os.O_WRONLY | os.O_CREAT | os.O_EXCL | os.O_NOFOLLOW
_READ_PLAIN = os.O_RDONLY | os.O_NOFOLLOW | os.O_NONBLOCK


def create_private_exclusive(path: Path, payload: bytes) -> None:
    """A new file with mode 0600 holding ``payload``, flushed to disk; ``FileExistsError`` if the name is taken by anything."""
    with os.fdopen(os.open(path, _CREATE_ONCE, 0o600), "wb", buffering=0) as stream:
        remaining = memoryview(payload)
        while len(remaining):
            remaining = remaining[stream.write(remaining):]
        os.fsync(stream.fileno())


# ---------------------------------------------------------------------------------------------------------------------- collected records
def _holds(path: Path, payload: bytes) -> bool:
    """Does the regular file ``path`` already say what ``payload`` says (byte for byte, or as a JSON value)?"""
    try:
        if not stat.S_ISREG(path.lstat().st_mode):
            return False
        present = path.read_bytes()
    except FileNotFoundError:
        return False
    if present == payload:
        return True
    try:
        return json.loads(present) == json.loads(payload)
    except ValueError:  # one of them is not JSON: only identical bytes would have counted
        return False


def _places(root: Path, name: str):
    """Where a record may go, in order of preference: its own name, then ``final/name``, ``final/name.1``, ..."""
    yield root / name
    keep = root / FINAL_DIR
    keep.mkdir(mode=0o700, exist_ok=True)
    yield keep / name
    number = 0
    while True:
        number += 1
        yield keep / f"{name}.{number}"


def write_collected(root: Path, name: str, payload: bytes, divergent: list[str]) -> None:
    """File ``payload`` as ``root/name`` without ever overwriting; a differing later arrival goes to ``final/`` and ``name`` is added to
    ``divergent`` (once).  Errors of the file system itself (full disk, permissions) propagate."""
    if name in ("", ".", "..") or "/" in name or "\0" in name:
        raise ValueError(f"collected record name {name!r} must be a plain file name")
    for rank, place in enumerate(_places(Path(root), name)):
        try:
            create_private_exclusive(place, payload)
        except FileExistsError:
            if not _holds(place, payload):
                continue  # taken by something else: try the next place
        if rank > 0 and name not in divergent:
            divergent.append(name)
        return


# ---------------------------------------------------------------------------------------------------------------------- guarded reads
def plain_path(path: Path) -> Path:
    """``path`` made absolute; refused when it, or any directory above it, is a symbolic link."""
    absolute = Path(os.path.abspath(path))
    for ancestor in (absolute, *absolute.parents):
        if os.path.islink(ancestor):
            raise ValueError("paths must not traverse symlinks")
    return absolute


def read_bounded(path: Path, cap: int) -> bytes:
    """The 1..``cap`` bytes of the regular file ``path``.  ``ValueError`` for a path through a link, for anything that is not a regular
    file of that size (checked on the open descriptor, before reading) and for a file that grows past the cap while it is read."""
    descriptor = os.open(plain_path(path), _READ_PLAIN)
    try:
        facts = os.fstat(descriptor)
        if not (stat.S_ISREG(facts.st_mode) and 1 <= facts.st_size <= cap):
            raise ValueError("input is not a bounded regular file")
        collected = bytearray()
        while len(collected) <= cap:
            piece = os.read(descriptor, min(1 << 20, cap + 1 - len(collected)))
            if not piece:
                break
            collected += piece
    finally:
        os.close(descriptor)
    if not 1 <= len(collected) <= cap:
        raise ValueError("input changed beyond its byte cap")
    return bytes(collected)


def require_private(path: Path) -> None:
    """``ValueError`` unless ``path`` belongs to this user, is closed to group and others, and is reached without links."""
    facts = plain_path(path).stat()
    if facts.st_uid != os.geteuid() or stat.S_IMODE(facts.st_mode) & (stat.S_IRWXG | stat.S_IRWXO):
        raise ValueError(f"{path} must be owned by this user and closed to group and others")


# ---------------------------------------------------------------------------------------------------------------------- replaced documents
def _replace_with(path: Path, write) -> None:
    """Write a 0600 sibling ``<name>.tmp`` with ``write(stream)``, flush it to disk and rename it over ``path``."""
    path = Path(path)
    sibling = path.with_name(path.name + ".tmp")
    with os.fdopen(os.open(sibling, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600), "w", encoding="utf-8") as stream:
        write(stream)
        stream.flush()
        os.fsync(stream.fileno())
    os.replace(sibling, path)


def atomic_json(path: Path, value) -> None:
    """State documents (compact, UTF-8 as is)."""
    _replace_with(path, lambda stream: json.dump(value, stream, ensure_ascii=False))


def persist_json(path: Path, value) -> None:
    """Reports meant to be read by people: sorted keys, indented, newline at the end."""
    _replace_with(path, lambda stream: stream.write(json.dumps(value, sort_keys=True, indent=2) + "\n"))
