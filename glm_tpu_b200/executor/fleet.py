"""The local fleet: building worker commands, probing that the GPUs are idle, starting and supervising workers.

On the TPU reference the fleet is eight hosts reached over SSH with authenticated helper programs
(``glm_tpu/executor/fleet.py:88-259``, ``executor/remote/*``).  On one 8-GPU box the fleet is N child processes of the
controller; what is kept is the discipline: one controller at a time (lease file), workers only run when started by a
controller (environment flag), an idle probe before anything is launched, supervision by exit code and wall deadline,
and cleanup that only ever signals the process groups this controller started.
"""

from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path

from glm_tpu_b200.engine import resident_protocol as proto


@dataclass
class WorkerSpec:
    rank: int
    world: int
    argv: list[str]
    env: dict
    log: Path


def worker_specs(*, world: int, run_dir: Path, worker_args: list[str], master_port: int, module: str = proto.WORKER_MODULE,
                 python: str = sys.executable, extra_env: dict | None = None) -> list[WorkerSpec]:
    specs = []
    for rank in range(world):
        env = dict(os.environ)
        env.update({
            "RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1",
            "MASTER_PORT": str(master_port), proto.WORKER_ENV_FLAG: "1", "NCCL_NVLS_ENABLE": env.get("NCCL_NVLS_ENABLE", "0"),
            "PYTHONPATH": os.pathsep.join([str(Path(__file__).resolve().parents[2]), env.get("PYTHONPATH", "")]).rstrip(os.pathsep),
        })
        env.update(extra_env or {})
        specs.append(WorkerSpec(rank, world, [python, "-m", module, *worker_args], env, Path(run_dir) / f"worker.rank{rank}.log"))
    return specs


def gpu_idle_report(query=None) -> dict:
    """Which GPUs already run compute processes (``nvidia-smi``).  ``query`` is injectable for tests."""
    if query is None:
        def query():
            done = subprocess.run(["nvidia-smi", "--query-compute-apps=gpu_uuid,pid,used_memory", "--format=csv,noheader"],
                                  capture_output=True, text=True, timeout=30)
            if done.returncode != 0:
                raise RuntimeError(done.stderr.strip() or "nvidia-smi failed")
            return done.stdout
    try:
        lines = [ln for ln in query().splitlines() if ln.strip()]
    except (OSError, RuntimeError, subprocess.TimeoutExpired) as exc:
        return {"available": False, "error": str(exc), "busy": []}
    return {"available": True, "busy": [ln.split(",")[0].strip() for ln in lines], "processes": len(lines)}


@dataclass
class Fleet:
    specs: list[WorkerSpec]
    keep_stdin: bool = False
    procs: list = field(default_factory=list)

    def start(self) -> None:
        for spec in self.specs:
            log = spec.log.open("wb")
            proc = subprocess.Popen(spec.argv, env=spec.env, stdin=subprocess.PIPE if self.keep_stdin else subprocess.DEVNULL,
                                    stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
            log.close()
            self.procs.append(proc)

    def send_all(self, line: bytes) -> None:
        for proc in self.procs:
            if proc.stdin is not None and proc.poll() is None:
                proc.stdin.write(line)
                proc.stdin.flush()

    def poll(self) -> list:
        return [p.poll() for p in self.procs]

    def wait(self, deadline: float | None, on_tick=None, tick: float = 0.2) -> list:
        """Until every worker exited, one failed, or the deadline passed.  Returns the exit codes (None = still running)."""
        while True:
            codes = self.poll()
            if all(c is not None for c in codes) or any(c not in (None, 0) for c in codes):
                return codes
            if deadline is not None and time.monotonic() > deadline:
                return codes
            if on_tick is not None and on_tick() is False:
                return self.poll()
            time.sleep(tick)

    def cleanup(self, grace: float = 5.0) -> list:
        """Terminate the process groups this controller started (nothing else is ever signalled)."""
        for proc in self.procs:
            if proc.stdin is not None:
                try:
                    proc.stdin.close()
                except OSError:
                    pass
        end = time.monotonic() + grace
        for proc in self.procs:
            if proc.poll() is None:
                try:
                    os.killpg(proc.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        for proc in self.procs:
            try:
                proc.wait(max(0.1, end - time.monotonic()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(proc.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
                proc.wait()
        return self.poll()
