"""The source manifest: a digest of every file of the package a worker will import, taken by the controller and re-checked
by each worker before it opens a device.

The controller and its workers share one filesystem on a single box, so nothing is copied; what the manifest catches is a
tree that changed between the moment the controller recorded its identity and the moment a worker starts (an edit, a
rebuild of the CUDA library, a different checkout on ``PYTHONPATH``).  ``build`` lists ``relative path -> sha256`` for the
Python sources, the CUDA sources and the built library; ``digest`` is the SHA-256 of its canonical JSON (what the worker is
given on its command line); ``verify`` re-hashes.

Parity: reference ``glm_tpu/worker/tpu_worker.py:57-67`` (worker re-hashes every staged source file against
``source_manifest.json``), ``glm_tpu/executor/staging.py:15-50``.
"""

from __future__ import annotations

import hashlib
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

PACKAGE = "glm_tpu_b200"
SUFFIXES = (".py", ".cu", ".cuh", ".h", ".so", ".json", ".js", ".css", ".html")
MANIFEST_FILE = "source_manifest.json"


def _sha(path: Path) -> str:
    digest = hashlib.sha256()
    with path.open("rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            digest.update(chunk)
    return digest.hexdigest()


def build(repo: Path) -> dict[str, str]:
    root = Path(repo) / PACKAGE
    if not root.is_dir():
        raise ConfigValidationError(f"{root} is not the package directory")
    out = {}
    for path in sorted(root.rglob("*")):
        if path.is_file() and path.suffix in SUFFIXES and "__pycache__" not in path.parts and "build" not in path.relative_to(root).parts[:-1]:
            out[path.relative_to(repo).as_posix()] = _sha(path)
    return out


def to_bytes(manifest: dict[str, str]) -> bytes:
    return canonical_wire_bytes(manifest)


def digest(manifest: dict[str, str]) -> str:
    return hashlib.sha256(to_bytes(manifest)).hexdigest()


def verify(repo: Path, manifest: dict, *, must_contain: str | None = None) -> None:
    """Every listed file must exist under ``repo`` with the listed digest; ``must_contain``: a path that has to be listed."""
    repo = Path(repo).resolve()
    if type(manifest) is not dict or not manifest:
        raise ConfigValidationError("the source manifest is empty or not an object")
    if must_contain is not None and must_contain not in manifest:
        raise ConfigValidationError(f"the source manifest does not list {must_contain}")
    for name, want in manifest.items():
        path = (repo / name).resolve()
        if not path.is_relative_to(repo) or not path.is_file() or _sha(path) != want:
            raise ConfigValidationError(f"deployed source differs from the controller's: {name}")
