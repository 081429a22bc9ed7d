"""Controller + workers end to end on the CPU (oracle backend): one-shot, two ranks, resident session, lease."""

import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import pytest

from tests.conftest import scaled

from glm_tpu_b200.config.model import tiny_geometry
from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.executor import jobs, launch_policy, multiproc_executor
from glm_tpu_b200.exceptions import ConfigValidationError
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

ROOT = Path(__file__).resolve().parents[1]
G = tiny_geometry()
PROFILE = rq.RequestProfile.for_geometry(G, (64,), concurrent_capacity=64)


def prepared(tmp_path, name="req.json", rid="q1", ids=(5, 6, 7, 8), n=3):
    req = rq.from_token_ids(list(ids), request_id=rid, max_new_tokens=n, context_capacity=64, profile=PROFILE)
    path = tmp_path / name
    path.write_bytes(canonical_wire_bytes(req))
    return req, path


def run_controller(args, timeout=240):
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    return subprocess.run([sys.executable, "-m", "glm_tpu_b200.executor.multiproc_executor", *args], env=env, capture_output=True,
                          text=True, timeout=scaled(timeout))


def run_dir_of(stdout):
    return Path(next(ln for ln in stdout.splitlines() if ln.startswith(proto.STDOUT_RUN))[len(proto.STDOUT_RUN):])


def test_one_shot_single_rank(tmp_path):
    req, path = prepared(tmp_path)
    done = run_controller(["--request", str(path), "--run-root", str(tmp_path / "runs"), "--backend", "oracle", "--gpus", "1",
                           "--model", "random:tiny", "--context", "64", "--print-answers"])
    assert done.returncode == 0, done.stdout + done.stderr
    run_dir = run_dir_of(done.stdout)
    events = [json.loads(ln) for ln in (run_dir / proto.TOKENS_FILE).read_text().splitlines()]
    assert [e["index"] for e in events] == [0, 1, 2] and events[-1]["finish_reason"] in ("length", "eos")
    summary = json.loads((run_dir / proto.SUMMARY_FILE).read_text())
    assert summary["agree"] and summary["requests"][0]["emitted"] == len(events)
    assert json.loads((run_dir / proto.CONTROLLER_TERMINAL_FILE).read_text())["ok"]
    assert "q1" in json.loads((run_dir / proto.ANSWER_FILE).read_text())
    ident = json.loads((run_dir / "controller_identity.json").read_text())
    assert "source" in ident and ident["idle_probe"].get("skipped")


def test_two_ranks_agree_over_gloo(tmp_path):
    req, path = prepared(tmp_path, n=2)
    done = run_controller(["--request", str(path), "--run-root", str(tmp_path / "runs"), "--backend", "oracle", "--gpus", "2",
                           "--model", "random:tiny", "--context", "64", "--master-port", "29591"])
    assert done.returncode == 0, done.stdout + done.stderr
    summary = json.loads((run_dir_of(done.stdout) / proto.SUMMARY_FILE).read_text())
    assert summary["ranks"] == 2 and summary["agree"]


def test_resident_session_serves_the_inbox(tmp_path):
    req0, path0 = prepared(tmp_path, n=2)
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    proc = subprocess.Popen([sys.executable, "-m", "glm_tpu_b200.executor.multiproc_executor", "--request", str(path0), "--run-root",
                             str(tmp_path / "runs"), "--backend", "oracle", "--gpus", "1", "--model", "random:tiny", "--context", "64",
                             "--keep-loaded", "--poll-seconds", "0.1", "--wall-seconds", "200"], env=env, stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT, text=True)
    lines = []
    reader = threading.Thread(target=lambda: lines.extend(iter(proc.stdout.readline, "")), daemon=True)
    reader.start()
    try:
        deadline = time.time() + 120
        while time.time() < deadline and not any(ln.startswith(proto.STDOUT_RUN) for ln in lines):
            time.sleep(0.1)
        run_dir = run_dir_of("".join(lines))
        while time.time() < deadline and not (run_dir / proto.READY_FILE).exists():
            time.sleep(0.1)
        assert (run_dir / proto.READY_FILE).exists(), "".join(lines)
        req1, path1 = prepared(tmp_path, name="next.json", rid="q2", ids=(9, 10, 11), n=2)
        os.link(path1, run_dir / proto.INBOX_DIR / proto.inbox_name(1))  # publish: never overwrites
        def results():
            return [json.loads(ln[len(proto.STDOUT_RESIDENT_RESULT):]) for ln in lines if ln.startswith(proto.STDOUT_RESIDENT_RESULT)]

        while time.time() < deadline and len(results()) < 2:
            time.sleep(0.1)
        first, result = results()[:2]
        assert first["sequence"] == 0 and first["agree"]  # the request the session was started with is reported at once
        assert result["sequence"] == 1 and result["agree"] and result["requests"][0]["request_id"] == "q2"
        assert (proto.result_dir(run_dir, 1) / proto.TOKENS_FILE).exists()
        (run_dir / proto.INBOX_DIR / proto.STOP_FILE).write_text('{"stop":true}')
        assert proc.wait(60) == 0, "".join(lines)
    finally:
        if proc.poll() is None:
            proc.terminate()


def test_worker_refuses_to_start_without_the_controller_flag(tmp_path):
    env = {k: v for k, v in os.environ.items() if k != proto.WORKER_ENV_FLAG}
    env["PYTHONPATH"] = str(ROOT)
    done = subprocess.run([sys.executable, "-m", "glm_tpu_b200.worker.gpu_worker", "--run-dir", str(tmp_path)], env=env,
                          capture_output=True, text=True, timeout=scaled(60))
    assert done.returncode != 0 and proto.WORKER_ENV_FLAG in done.stderr


def test_second_controller_is_refused_while_the_lease_is_held(tmp_path):
    with jobs.workload_lease(tmp_path):
        with pytest.raises(jobs.LeaseHeld):
            with jobs.workload_lease(tmp_path):
                pass
    with jobs.workload_lease(tmp_path):  # released on exit
        pass


def test_busy_gpus_and_strict_policy_refuse(tmp_path):
    with pytest.raises(ConfigValidationError):
        with jobs.fleet_job(tmp_path, repo=ROOT, idle_query=lambda: "GPU-abc, 123, 1000 MiB\n"):
            pass
    ident = launch_policy.source_identity(tmp_path)
    assert ident["git"] is False
    with pytest.raises(ConfigValidationError):
        launch_policy.check(ident, "strict")
    launch_policy.check(ident, "record")


def test_summarize_detects_disagreement(tmp_path):
    rec = {"requests": [{"request_id": "a", "token_sha256": "x", "emitted": 1, "finish_reason": "length", "decode_tokens_per_second": 1.0,
                         "prefill_seconds": 0.1}], "programs": [{"name": "decode", "kind": "host"}]}
    (tmp_path / proto.runner_file(0)).write_text(json.dumps(rec))
    other = json.loads(json.dumps(rec))
    other["requests"][0]["token_sha256"] = "y"
    (tmp_path / proto.runner_file(1)).write_text(json.dumps(other))
    assert not multiproc_executor.summarize(tmp_path, 2)["agree"]
    (tmp_path / proto.runner_file(1)).write_text(json.dumps(rec))
    assert multiproc_executor.summarize(tmp_path, 2)["agree"]
    assert multiproc_executor.summarize(tmp_path, 3)["missing_ranks"] == [2]
