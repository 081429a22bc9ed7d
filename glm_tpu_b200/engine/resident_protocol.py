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

CONTROLLER_MODULE = "glm_tpu_b200.executor.multiproc_executor"
WORKER_MODULE = "glm_tpu_b200.worker.gpu_worker"
PACK_WORKER_MODULE = "glm_tpu_b200.model_loader.pack_worker"
WORKER_ENV_FLAG = "GLM_B200_WORKER"

INBOX_DIR = "inbox"
STOP_FILE = "stop.json"
STOP_COMMAND = b'{"stop":true}\n'
READY_FILE = "resident-ready.json"
MEASUREMENT_FILE = "resident-measurement.json"
CONTROLLER_IDENTITY_FILE = "controller_identity.json"
CONTROLLER_TERMINAL_FILE = "controller_terminal.json"
SUMMARY_FILE = "summary.json"
TOKENS_FILE = "tokens.jsonl"
ANSWER_FILE = "answer.txt"
PRODUCER_LOCK = "producer.lock"
STDOUT_RUN = "RUN "
STDOUT_RESIDENT_RESULT = "RESIDENT_RESULT "


def inbox_name(sequence: int) -> str:
    return f"{sequence:04d}.json"


def result_dir(root: Path, sequence: int) -> Path:
    return Path(root) if sequence == 0 else Path(root) / f"resident-{sequence:04d}"


def runner_file(rank: int) -> str:
    return f"runner.rank{rank}.json"


def worker_started_file(rank: int) -> str:
    return f"worker_started.rank{rank}.json"


def encode_command(sequence: int, request: Any) -> bytes:
    return canonical_wire_bytes({"sequence": sequence, "request": request}) + b"\n"
