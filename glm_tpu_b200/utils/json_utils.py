"""Two canonical JSON encodings of one value.

Both sort keys, use the most compact separators and refuse NaN / infinity.  They differ in how text leaves the process: the *wire* form
keeps characters as UTF-8 (what is written to files, pipes and sockets), the *hash* form escapes everything outside ASCII (what is fed to
SHA-256, so that a digest never depends on an encoding choice).  ``fingerprint`` is the SHA-256 of the hash form.

Parity: reference ``glm_tpu/utils/json_utils.py`` (the same two contracts).
"""

from __future__ import annotations

import hashlib
import json
from typing import Any


def _canonical_text(value: Any, *, ascii_only: bool) -> str:
    return json.dumps(value, ensure_ascii=ascii_only, allow_nan=False, sort_keys=True, separators=(",", ":"))


def canonical_wire_bytes(value: Any) -> bytes:
    return _canonical_text(value, ascii_only=False).encode("utf-8")


def canonical_hash_bytes(value: Any) -> bytes:
    return _canonical_text(value, ascii_only=True).encode("ascii")


def fingerprint(value: Any) -> str:
    return hashlib.sha256(canonical_hash_bytes(value)).hexdigest()
