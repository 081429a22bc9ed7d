"""The run-directory protocol shared by the controller, the per-GPU workers and the front ends.

A run directory holds ``inbox/NNNN.json`` (prepared requests published by a producer with ``os.link``, never
overwritten), ``inbox/stop.json`` (``{"stop":true}``), ``resident-ready.json`` (``{"sequence": n}`` once request n is
done and the model is idle), one result directory per sequence (``resident-NNNN/``; the run directory itself for
sequence 0) with ``tokens.jsonl``, ``answer.txt`` and ``runner.rank<r>.json``, and ``resident-measurement.json``.
A worker receives each request as one canonical JSON line on stdin: ``{"request": ..., "sequence": n}``.

Parity: reference ``glm_tpu/engine/resident_protocol.py:26-71``.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

# ---- who runs what: `python -m` targets, and the flag a controller sets so that a worker started by hand refuses to run
CONTROLLER_MODULE = "glm_tpu_b200.executor.multiproc_executor"
WORKER_MODULE = "glm_tpu_b200.worker.gpu_worker"
PACK_WORKER_MODULE = "glm_tpu_b200.model_loader.pack_worker"
WORKER_ENV_FLAG = "GLM_B200_WORKER"

# ---- lines on a controller's stdout that front ends look for
STDOUT_RUN = "RUN "
STDOUT_RESIDENT_RESULT = "RESIDENT_RESULT "

# ---- names inside a run directory
INBOX_DIR = "inbox"
STOP_FILE, STOP_COMMAND = "stop.json", b'{"stop":true}\n'
PRODUCER_LOCK = "producer.lock"
READY_FILE = "resident-ready.json"
MEASUREMENT_FILE = "resident-measurement.json"
SUMMARY_FILE = "summary.json"
CONTROLLER_IDENTITY_FILE, CONTROLLER_TERMINAL_FILE = "controller_identity.json", "controller_terminal.json"
TOKENS_FILE, ANSWER_FILE = "tokens.jsonl", "answer.txt"
SEQUENCE_DIGITS = 4


def _numbered(sequence: int) -> str:
    if sequence < 0:
        raise ValueError("sequence numbers start at 0")
    return str(sequence).zfill(SEQUENCE_DIGITS)


def inbox_name(sequence: int) -> str:
    """File name of request ``sequence`` in the inbox."""
    return _numbered(sequence) + ".json"


def result_dir(root: Path, sequence: int) -> Path:
    """Where a sequence's records go: the first request (0) writes into the run directory itself."""
    root = Path(root)
    return root / ("resident-" + _numbered(sequence)) if sequence else root


def runner_file(rank: int) -> str:
    return "runner.rank%d.json" % rank


def worker_started_file(rank: int) -> str:
    return "worker_started.rank%d.json" % rank


def encode_command(sequence: int, request: Any) -> bytes:
    """One line for a worker's stdin."""
    return canonical_wire_bytes({"request": request, "sequence": sequence}) + b"\n"
