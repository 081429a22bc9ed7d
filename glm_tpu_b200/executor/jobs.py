"""Fleet jobs: the lease every controller holds while it uses the GPUs, and the common shape of a job.

``fleet_job`` is a context manager: take the workload lease (``flock``, non-blocking: a second controller is refused
instead of queued), record the source identity, run the idle probe, yield a ``Job`` that starts workers and always
cleans up its own process groups.

Parity: reference ``glm_tpu/executor/jobs.py:268-292`` (``fleet_job``), ``multihost_executor.py:288-296`` (locks).
"""

from __future__ import annotations

import contextlib
import fcntl
import os
from dataclasses import dataclass, field
from pathlib import Path

from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.executor import fleet as fleet_mod
from glm_tpu_b200.executor import launch_policy
from glm_tpu_b200.utils.io_utils import persist_json

LEASE_FILE = "workload.lock"


class LeaseHeld(ConfigValidationError):
    pass


@contextlib.contextmanager
def workload_lease(run_root: Path):
    run_root = Path(run_root)
    run_root.mkdir(parents=True, exist_ok=True, mode=0o700)
    fd = os.open(run_root / LEASE_FILE, os.O_RDWR | os.O_CREAT, 0o600)
    try:
        try:
            fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except BlockingIOError as exc:
            raise LeaseHeld(f"another controller holds {run_root / LEASE_FILE}") from exc
        os.ftruncate(fd, 0)
        os.write(fd, f"{os.getpid()}\n".encode())
        yield
    finally:
        os.close(fd)


@dataclass
class Job:
    run_root: Path
    identity: dict
    idle: dict
    fleets: list = field(default_factory=list)

    def start(self, specs, keep_stdin=False) -> fleet_mod.Fleet:
        fl = fleet_mod.Fleet(specs, keep_stdin=keep_stdin)
        self.fleets.append(fl)
        fl.start()
        return fl


@contextlib.contextmanager
def fleet_job(run_root: Path, *, repo: Path, policy: str = "record", require_idle: bool = True, idle_query=None):
    with workload_lease(run_root):
        identity = launch_policy.source_identity(repo)
        launch_policy.check(identity, policy)
        idle = fleet_mod.gpu_idle_report(idle_query) if require_idle else {"available": False, "busy": [], "skipped": True}
        if require_idle and idle["available"] and idle["busy"]:
            raise ConfigValidationError(f"GPUs are busy: {idle['busy']}")
        job = Job(Path(run_root), identity, idle)
        try:
            yield job
        finally:
            for fl in job.fleets:
                fl.cleanup()


def write_identity(run_dir: Path, job: Job, extra: dict | None = None) -> None:
    persist_json(Path(run_dir) / "controller_identity.json", {"source": job.identity, "idle_probe": job.idle, "pid": os.getpid(), **(extra or {})})
