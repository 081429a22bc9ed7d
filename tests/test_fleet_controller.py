"""The local fleet and the controller's resident loop without a model: tiny child processes as workers, a scripted fleet for the
loop.  What is checked is the discipline: workers carry the controller's flag and rendezvous, supervision ends on the first
failure or on the deadline, cleanup reaches the whole process group and nothing else, run directories are fresh and private,
and the resident loop ends in order whatever arrives in its inbox.

Reference counterparts: ``tests/executor/test_multihost_executor.py``, ``tests/executor/test_remote_helpers.py``."""

import json
import os
import signal
import stat
import subprocess
import sys
import time
from pathlib import Path

import pytest

from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.executor import fleet as fleet_mod
from glm_tpu_b200.executor import multiproc_executor as controller
from glm_tpu_b200.executor import staging
from glm_tpu_b200.executor.fleet import Fleet, WorkerSpec, gpu_idle_report, worker_specs


def spec(tmp_path, rank, code: str, world=2) -> WorkerSpec:
    return WorkerSpec(rank, world, [sys.executable, "-c", code], dict(os.environ), tmp_path / f"worker.rank{rank}.log")


# ------------------------------------------------------------------------------------------------ commands and probes
def test_worker_commands_carry_the_rendezvous_and_the_controller_flag(tmp_path, monkeypatch):
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "1")
    monkeypatch.setenv("PYTHONPATH", "/somewhere/else")
    specs = worker_specs(world=4, run_dir=tmp_path, worker_args=["--run-dir", str(tmp_path)], master_port=29611, extra_env={"X": "y"})
    assert [s.rank for s in specs] == [0, 1, 2, 3] and all(s.world == 4 for s in specs)
    for s in specs:
        assert s.argv == [sys.executable, "-m", proto.WORKER_MODULE, "--run-dir", str(tmp_path)]
        assert s.env["RANK"] == s.env["LOCAL_RANK"] == str(s.rank) and s.env["WORLD_SIZE"] == "4"
        assert s.env["MASTER_ADDR"] == "127.0.0.1" and s.env["MASTER_PORT"] == "29611"  # never a host name that may not resolve
        assert s.env[proto.WORKER_ENV_FLAG] == "1" and s.env["X"] == "y" and s.env["NCCL_NVLS_ENABLE"] == "1"  # the caller's choice is kept
        assert s.env["PYTHONPATH"].split(os.pathsep) == [str(Path(fleet_mod.__file__).resolve().parents[2]), "/somewhere/else"]
        assert s.log == tmp_path / f"worker.rank{s.rank}.log"
    monkeypatch.delenv("NCCL_NVLS_ENABLE")
    assert worker_specs(world=1, run_dir=tmp_path, worker_args=[], master_port=1)[0].env["NCCL_NVLS_ENABLE"] == "0"  # off unless asked for


def test_idle_probe():
    assert gpu_idle_report(lambda: "") == {"available": True, "busy": [], "processes": 0}
    busy = gpu_idle_report(lambda: "GPU-aaa, 4242, 1024 MiB\nGPU-bbb, 4243, 10 MiB\n\n")
    assert busy == {"available": True, "busy": ["GPU-aaa", "GPU-bbb"], "processes": 2}

    def broken():
        raise RuntimeError("NVIDIA-SMI has failed")

    assert gpu_idle_report(broken) == {"available": False, "error": "NVIDIA-SMI has failed", "busy": []}

    def absent():
        raise FileNotFoundError("nvidia-smi")

    assert gpu_idle_report(absent)["available"] is False  # no driver on this machine: reported, not raised


# ------------------------------------------------------------------------------------------------ supervision
def test_wait_ends_when_all_workers_are_done(tmp_path):
    fl = Fleet([spec(tmp_path, r, f"print('rank {r} says hello')") for r in range(2)])
    fl.start()
    assert fl.wait(time.monotonic() + 60) == [0, 0]
    assert (tmp_path / "worker.rank1.log").read_text() == "rank 1 says hello\n"
    assert fl.cleanup() == [0, 0]


def test_the_first_failure_ends_the_wait_and_cleanup_stops_the_rest(tmp_path):
    fl = Fleet([spec(tmp_path, 0, "import time; time.sleep(600)"), spec(tmp_path, 1, "import sys; sys.exit(3)")])
    fl.start()
    started = time.monotonic()
    codes = fl.wait(time.monotonic() + 60)
    assert codes[1] == 3 and codes[0] is None and time.monotonic() - started < 30  # did not sit out the sleeping worker
    assert fl.cleanup(grace=5) == [-signal.SIGTERM, 3]


def test_the_deadline_ends_the_wait(tmp_path):
    fl = Fleet([spec(tmp_path, 0, "import time; time.sleep(600)")])
    fl.start()
    assert fl.wait(time.monotonic() + 0.5) == [None]
    ticks = []
    assert fl.wait(None, on_tick=lambda: ticks.append(1) or len(ticks) < 3, tick=0.01) == [None]  # the caller's tick may end it too
    assert len(ticks) == 3 and fl.cleanup(grace=5) == [-signal.SIGTERM]


def test_cleanup_reaches_grandchildren_and_workers_that_ignore_sigterm(tmp_path):
    pid_file = tmp_path / "grandchild.pid"
    parent = ("import subprocess, sys, time\n"
              f"child = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(600)'])\n"
              f"open({str(pid_file)!r}, 'w').write(str(child.pid))\n"
              "time.sleep(600)\n")
    stubborn = "import signal, time\nsignal.signal(signal.SIGTERM, signal.SIG_IGN)\nprint('ready', flush=True)\ntime.sleep(600)\n"
    fl = Fleet([spec(tmp_path, 0, parent), spec(tmp_path, 1, stubborn)])
    fl.start()
    for _ in range(200):
        if pid_file.exists() and pid_file.read_text() and (tmp_path / "worker.rank1.log").read_text().startswith("ready"):
            break
        time.sleep(0.05)
    grandchild = int(pid_file.read_text())
    assert fl.cleanup(grace=1.0) == [-signal.SIGTERM, -signal.SIGKILL]  # asked first, then made to
    for _ in range(100):
        try:
            os.kill(grandchild, 0)
        except ProcessLookupError:
            break
        time.sleep(0.05)
    else:
        pytest.fail("the worker's own child survived the cleanup of its process group")
    assert all(p.pid != os.getpgid(0) for p in fl.procs)  # each worker leads a group of its own: the controller's group is never signalled


def test_lines_reach_only_workers_that_listen(tmp_path):
    echo = "import sys\nfor line in sys.stdin:\n    print('got', line.strip(), flush=True)\n    if 'stop' in line: break\n"
    fl = Fleet([spec(tmp_path, 0, echo), spec(tmp_path, 1, "pass")], keep_stdin=True)
    fl.start()
    fl.procs[1].wait(30)
    fl.send_all(proto.encode_command(1, {"a": 1}))  # the worker that exited is skipped, not written to
    fl.send_all(proto.STOP_COMMAND)
    assert fl.wait(time.monotonic() + 30) == [0, 0]
    assert (tmp_path / "worker.rank0.log").read_text() == 'got {"request":{"a":1},"sequence":1}\ngot {"stop":true}\n'
    silent = Fleet([spec(tmp_path, 0, "pass")])  # one-shot workers get no stdin at all
    silent.start()
    assert silent.procs[0].stdin is None and silent.wait(time.monotonic() + 30) == [0]
    silent.send_all(b"ignored\n")


# ------------------------------------------------------------------------------------------------ staging
def test_run_directories_are_fresh_and_private(tmp_path):
    root = tmp_path / "runs"
    first, second = staging.new_run_dir(root), staging.new_run_dir(root)
    tagged = staging.new_run_dir(root, "pack")
    assert len({first, second, tagged}) == 3 and tagged.name.endswith("-pack") or "-pack." in tagged.name
    for path in (root, first, second, first / proto.INBOX_DIR):
        assert stat.S_IMODE(path.stat().st_mode) == 0o700
    payload = {"b": 1, "a": "ü"}
    staged = staging.stage_request(first, payload)
    assert staged == first / staging.REQUEST_FILE and staged.read_bytes() == '{"a":"ü","b":1}'.encode() and stat.S_IMODE(staged.stat().st_mode) == 0o600
    with pytest.raises(FileExistsError):
        staging.stage_request(first, {"other": True})  # a run has one request; it is never replaced
    assert staging.stage_request(second, None) is None and not (second / staging.REQUEST_FILE).exists()


# ------------------------------------------------------------------------------------------------ the resident loop
class ScriptedFleet:
    """Stands in for ``Fleet``: records what the controller tells the workers and answers ``poll`` from a script."""

    def __init__(self, run_dir, world=2):
        self.run_dir, self.world, self.sent, self.codes, self.broken = run_dir, world, [], [None] * world, False

    def poll(self):
        return list(self.codes)

    def send_all(self, line):
        if self.broken:
            raise BrokenPipeError("worker gone")
        self.sent.append(line)
        command = json.loads(line)
        if "sequence" in command:  # the workers answer at once: records for the sequence, then the ready file
            finish(self.run_dir, self.world, command["sequence"], command["request"]["request_id"])


def finish(run_dir, world, sequence, rid, digest="d" * 64):
    out = proto.result_dir(run_dir, sequence)
    out.mkdir(exist_ok=True)
    for rank in range(world):
        (out / proto.runner_file(rank)).write_text(json.dumps({
            "programs": [{"name": "decode", "kind": "cuda_graph"}],
            "requests": [{"request_id": rid, "token_sha256": digest if rank == 0 or digest != "split" else "other", "emitted": 3, "finish_reason": "eos",
                          "decode_tokens_per_second": 100.0 + rank, "prefill_seconds": 0.1 * (rank + 1)}]}))
    (run_dir / proto.READY_FILE).write_text(json.dumps({"sequence": sequence}))


def loop(run_dir, fl, seconds=5.0, check=lambda payload: None, **kw):
    return controller.resident_controller(fl, run_dir, fl.world, check, time.monotonic() + seconds, 0.01, **kw)


@pytest.fixture
def run_dir(tmp_path):
    return staging.new_run_dir(tmp_path / "runs")


def publish(run_dir, sequence, payload):
    (run_dir / proto.INBOX_DIR / proto.inbox_name(sequence)).write_text(json.dumps(payload) if not isinstance(payload, str) else payload)


def test_requests_are_served_in_sequence_until_the_stop_file(run_dir, capsys):
    fl = ScriptedFleet(run_dir)
    (run_dir / proto.READY_FILE).write_text(json.dumps({"sequence": 0}))  # loaded, nothing asked yet
    publish(run_dir, 1, {"request_id": "one"})
    publish(run_dir, 2, {"request_id": "two"})
    publish(run_dir, 4, {"request_id": "four"})  # a gap: never reached
    (run_dir / proto.INBOX_DIR / proto.STOP_FILE).write_bytes(proto.STOP_COMMAND)
    result = loop(run_dir, fl)
    # the stop file is honoured when the model is idle, before the next request is taken
    assert result == {"stopped": "stop_file", "served": []} and fl.sent == [proto.STOP_COMMAND]

    (run_dir / proto.INBOX_DIR / proto.STOP_FILE).unlink()
    fl = ScriptedFleet(run_dir)
    result = loop(run_dir, fl, seconds=3.0)
    assert result == {"stopped": "deadline", "served": [1, 2]}
    assert [json.loads(x).get("sequence") for x in fl.sent] == [1, 2, None] and fl.sent[-1] == proto.STOP_COMMAND
    lines = [json.loads(x[len(proto.STDOUT_RESIDENT_RESULT):]) for x in capsys.readouterr().out.splitlines() if x.startswith(proto.STDOUT_RESIDENT_RESULT)]
    assert [x["sequence"] for x in lines] == [1, 2] and all(x["agree"] and x["ranks"] == 2 for x in lines)
    measurement = json.loads((proto.result_dir(run_dir, 2) / proto.MEASUREMENT_FILE).read_text())
    assert measurement["requests"] == [{"request_id": "two", "emitted": 3, "finish_reason": "eos", "decode_tokens_per_second": 100.0,
                                        "prefill_seconds": 0.2, "token_sha256": "d" * 64}]  # the slowest rank's figures


def test_an_invalid_request_ends_the_session_in_order(run_dir):
    (run_dir / proto.READY_FILE).write_text(json.dumps({"sequence": 0}))
    for content, error in (("{not json", "JSONDecodeError"), ("", "ValueError"), (json.dumps({"request_id": "bad"}), "RequestValidationError")):
        fl = ScriptedFleet(run_dir)
        publish(run_dir, 1, content)

        def check(payload):
            from glm_tpu_b200.exceptions import RequestValidationError

            raise RequestValidationError("missing request fields")

        result = loop(run_dir, fl, check=check)
        assert result["stopped"] == "invalid_request" and result["sequence"] == 1 and result["served"] == [] and result["error"].startswith(error)
        assert fl.sent == [proto.STOP_COMMAND]  # the workers never saw it; they were told to stop
    link_target = run_dir / "elsewhere.json"
    link_target.write_text(json.dumps({"request_id": "x"}))
    (run_dir / proto.INBOX_DIR / proto.inbox_name(1)).unlink()
    (run_dir / proto.INBOX_DIR / proto.inbox_name(1)).symlink_to(link_target)
    result = loop(run_dir, ScriptedFleet(run_dir))
    assert result["stopped"] == "invalid_request" and "symlink" in result["error"]  # a planted link is not a request


def test_a_worker_that_exits_ends_the_session(run_dir):
    (run_dir / proto.READY_FILE).write_text(json.dumps({"sequence": 0}))
    fl = ScriptedFleet(run_dir)
    fl.codes = [None, 1]
    assert loop(run_dir, fl) == {"stopped": "worker_exit", "exit_codes": [None, 1], "served": []}
    fl = ScriptedFleet(run_dir)
    fl.broken = True  # alive at the poll, gone at the write
    publish(run_dir, 1, {"request_id": "one"})
    assert loop(run_dir, fl) == {"stopped": "worker_exit", "exit_codes": [None, None], "served": []}


def test_the_initial_request_is_reported_once_the_model_is_idle(run_dir, capsys):
    fl = ScriptedFleet(run_dir)
    finish(run_dir, 2, 0, "question-01")
    (run_dir / proto.ANSWER_FILE).write_text("Four.")
    result = loop(run_dir, fl, seconds=0.3, initial=True, print_answers=True)
    out = capsys.readouterr().out
    assert result == {"stopped": "deadline", "served": []} and out.startswith("Four.\n" + proto.STDOUT_RESIDENT_RESULT)
    assert json.loads(out.splitlines()[1][len(proto.STDOUT_RESIDENT_RESULT):])["sequence"] == 0 and out.count(proto.STDOUT_RESIDENT_RESULT) == 1


def test_ranks_that_disagree_are_reported_as_such(run_dir):
    finish(run_dir, 2, 0, "q", digest="split")
    summary = controller.summarize(run_dir, 2)
    assert summary["agree"] is False and summary["requests"] == [] and summary["ranks"] == 2
    finish(run_dir, 2, 0, "q")
    assert controller.summarize(run_dir, 2)["agree"] is True
    assert controller.summarize(run_dir, 3) == {"ranks": 2, "missing_ranks": [2], "agree": False, "failures": [], "requests": []}
    record = json.loads((run_dir / proto.runner_file(1)).read_text())
    (run_dir / proto.runner_file(1)).write_text(json.dumps(dict(record, failure_type="DeviceStatusError")))
    failed = controller.summarize(run_dir, 2)
    assert failed["agree"] is False and failed["failures"] == ["DeviceStatusError"]


def test_a_record_that_cannot_be_read_counts_as_missing(run_dir):
    finish(run_dir, 2, 0, "q")
    (run_dir / proto.runner_file(1)).write_text('{"requests": [')  # a worker died while writing
    assert controller.summarize(run_dir, 2) == {"ranks": 1, "missing_ranks": [1], "agree": False, "failures": [], "requests": []}
    (run_dir / proto.runner_file(1)).write_text("[]")
    assert controller.summarize(run_dir, 2)["missing_ranks"] == [1]


def test_an_idle_session_has_no_deadline_and_every_request_its_own(run_dir):
    """``--wall-seconds`` bounds the start-up with the first request, then each later request; waiting for the inbox costs nothing.
    (The budgets are generous against a loaded machine: what matters is their order, not their size.)"""
    import threading

    def wait_for(condition, seconds=20.0):
        end = time.monotonic() + seconds
        while not condition() and time.monotonic() < end:
            time.sleep(0.01)
        return condition()

    (run_dir / proto.READY_FILE).write_text(json.dumps({"sequence": 0}))
    fl = ScriptedFleet(run_dir)
    result = {}
    worker = threading.Thread(target=lambda: result.update(controller.resident_controller(
        fl, run_dir, 2, lambda payload: None, time.monotonic() + 1.0, 0.01, wall_seconds=0.3)))
    worker.start()
    time.sleep(1.6)  # longer than the start-up budget and than a request's budget, idle: still waiting
    assert worker.is_alive() and fl.sent == []
    publish(run_dir, 1, {"request_id": "one"})
    assert wait_for(lambda: [json.loads(x).get("sequence") for x in fl.sent] == [1])
    time.sleep(0.6)  # answered within its own budget; idle again, and again without a deadline
    assert worker.is_alive()
    (run_dir / proto.INBOX_DIR / proto.STOP_FILE).write_bytes(proto.STOP_COMMAND)
    worker.join(20)
    assert result == {"stopped": "stop_file", "served": [1]}

    class Stuck(ScriptedFleet):  # takes the request and never finishes it
        def send_all(self, line):
            self.sent.append(line)

    (run_dir / proto.INBOX_DIR / proto.STOP_FILE).unlink()
    stuck = Stuck(run_dir)
    (run_dir / proto.READY_FILE).write_text(json.dumps({"sequence": 0}))
    started = time.monotonic()
    outcome = controller.resident_controller(stuck, run_dir, 2, lambda payload: None, time.monotonic() + 60.0, 0.01, wall_seconds=0.3)
    # sequence 1 is handed over at once and never answered: its own budget runs out, long before the start-up one would
    assert outcome == {"stopped": "deadline", "served": []} and 0.25 < time.monotonic() - started < 30.0
    assert json.loads(stuck.sent[0])["sequence"] == 1 and stuck.sent[-1] == proto.STOP_COMMAND
