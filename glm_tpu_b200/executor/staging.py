"""Run-directory staging: a fresh, owner-only directory with the request the workers will validate.

Parity: reference ``glm_tpu/executor/staging.py:15-50`` (bundle staged to every host; here all workers share one
filesystem, so staging is a directory and a canonical request file).
"""

from __future__ import annotations

import os
import time
from pathlib import Path

from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.utils.io_utils import create_private_exclusive
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

REQUEST_FILE = "request.json"


def new_run_dir(run_root: Path, tag: str = "") -> Path:
    run_root = Path(run_root)
    run_root.mkdir(parents=True, exist_ok=True, mode=0o700)
    stamp = time.strftime("%Y%m%d-%H%M%S")
    for attempt in range(100):
        name = f"run-{stamp}-{os.getpid()}" + (f"-{tag}" if tag else "") + (f".{attempt}" if attempt else "")
        path = run_root / name
        try:
            path.mkdir(mode=0o700)
        except FileExistsError:
            continue
        (path / proto.INBOX_DIR).mkdir(mode=0o700)
        return path
    raise RuntimeError("could not create a fresh run directory")


def stage_request(run_dir: Path, payload: dict | None) -> Path | None:
    if payload is None:
        return None
    path = Path(run_dir) / REQUEST_FILE
    create_private_exclusive(path, canonical_wire_bytes(payload))
    return path
