"""Two canonical JSON encodings.

``canonical_wire_bytes`` is what goes over a wire or into a file that another process reads
(sorted keys, compact, UTF-8, NaN refused).  ``canonical_hash_bytes`` is the input of every
content hash (same, but ASCII-escaped so the digest does not depend on an encoding choice).

Parity: reference ``glm_tpu/utils/json_utils.py:13-34``.
"""

from __future__ import annotations

import hashlib
import json
from typing import Any


def canonical_wire_bytes(value: Any) -> bytes:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=False, allow_nan=False).encode("utf-8")


def canonical_hash_bytes(value: Any) -> bytes:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=True, allow_nan=False).encode("ascii")


def fingerprint(value: Any) -> str:
    return hashlib.sha256(canonical_hash_bytes(value)).hexdigest()
