"""The job queue on top of the real resident client, against a run directory that a scripted "session" serves: what reaches the
inbox, in which order, under which sequence numbers, across restarts of the server and across a halt.

Reference counterparts: ``tests/entrypoints/serve/test_job_queue.py``, ``tests/engine/test_resident_client.py``."""

import hashlib
import json
import os
import stat
import struct

import pytest

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.engine.resident_client import Resident
from glm_tpu_b200.entrypoints.serve import job_queue
from glm_tpu_b200.entrypoints.serve.job_queue import API_HISTORY, PENDING, JobQueue
from glm_tpu_b200.exceptions import ApiError
from glm_tpu_b200.tokenizer import ByteTokenizer

EOS = (1021, 1022, 1023)
PROFILE = rq.RequestProfile(vocab_size=1024, eos_ids=EOS, capacities=(512,), prompt_limits={512: 512}, concurrent_capacity=512, max_new=128)


class Session:
    """The far side of the run directory: answers what is in the inbox the way a controller and its workers would."""

    def __init__(self, tmp_path, world=2):
        self.run, self.world, self.tok = tmp_path / "run", world, ByteTokenizer(1024, EOS)
        (self.run / proto.INBOX_DIR).mkdir(parents=True)
        (self.run / proto.CONTROLLER_IDENTITY_FILE).write_text(json.dumps({"pid": os.getpid()}))
        (self.run / proto.READY_FILE).write_text(json.dumps({"sequence": 0}))
        self.served = []

    def client(self):
        return Resident(self.run, self.tok, PROFILE, capacity=512, world=self.world)

    def inbox(self):
        return sorted(p.name for p in (self.run / proto.INBOX_DIR).iterdir())

    def serve(self, sequence, text="</think>Four.", *, tokens_only=False):
        payload = json.loads((self.run / proto.INBOX_DIR / proto.inbox_name(sequence)).read_text())
        rq.validate(payload, PROFILE)  # what arrives is a whole, valid request
        ids = self.tok.encode(text) + [EOS[0]]
        root = proto.result_dir(self.run, sequence)
        root.mkdir(exist_ok=True)
        rid = payload["request_id"]
        (root / proto.TOKENS_FILE).write_text("".join(json.dumps({"request_id": rid, "index": i, "token_id": t, "finish_reason": None}) + "\n"
                                                       for i, t in enumerate(ids)))
        if tokens_only:
            return rid
        digest = hashlib.sha256(struct.pack(f"<{len(ids)}i", *ids)).hexdigest()
        (root / proto.MEASUREMENT_FILE).write_text(json.dumps({"agree": True, "ranks": self.world, "requests": [
            {"request_id": rid, "finish_reason": "eos", "emitted": len(ids), "token_sha256": digest, "decode_tokens_per_second": 150.0, "prefill_seconds": 0.02}]}))
        (self.run / proto.READY_FILE).write_text(json.dumps({"sequence": sequence}))
        self.served.append(sequence)
        return rid


def ask(client, queue, key, text="2+2?"):
    payload = client.prepare_api([{"role": "user", "content": text}], key, tools=None, effort="max", max_new_tokens=16)
    return queue.submit(payload, key, label="api")


def test_one_request_at_a_time_in_submission_order(tmp_path):
    session = Session(tmp_path)
    client = session.client()
    queue = JobQueue(tmp_path / "state", client)
    for key in ("a", "b", "c"):
        ask(client, queue, key, text=f"question {key}")
    queue.step()
    assert session.inbox() == ["0001.json"] and queue.job("a")["sequence"] == 1 and queue.job("a")["status"] == "generating"
    queue.step()
    queue.step()
    assert session.inbox() == ["0001.json"] and queue.job("b")["sequence"] is None  # nothing else is published while one is in flight
    session.serve(1, tokens_only=True)
    queue.step()
    assert queue.job("a")["status"] == "generating" and queue.job("a")["answer"] == "Four." and session.inbox() == ["0001.json"]
    session.serve(1)
    queue.step()
    done = queue.job("a")
    assert done["status"] == "complete" and done["answer"] == "Four." and done["decode_tps"] == 150.0 and done["stop_cause"] == "eos"
    queue.step()
    assert session.inbox() == ["0001.json", "0002.json"] and queue.job("b")["sequence"] == 2 and queue.job("c")["sequence"] is None
    assert json.loads((session.run / proto.INBOX_DIR / "0002.json").read_text())["request_id"] == "api-b"
    session.serve(2, "thinking</think>Zwei.")
    queue.step()
    queue.step()
    session.serve(3)
    queue.step()
    assert [queue.job(k)["status"] for k in "abc"] == ["complete"] * 3 and queue.job("b")["thinking"] == "thinking" and session.served == [1, 2, 3]
    assert queue.pending() == 0 and queue.error is None


def test_a_restart_reconciles_the_same_request_under_the_same_number(tmp_path):
    session = Session(tmp_path)
    client = session.client()
    queue = JobQueue(tmp_path / "state", client)
    ask(client, queue, "a")
    ask(client, queue, "b")
    queue.step()
    assert session.inbox() == ["0001.json"]
    published = (session.run / proto.INBOX_DIR / "0001.json").read_bytes()

    restarted = JobQueue(tmp_path / "state", session.client())  # the server process went away and came back
    assert restarted.job("a")["sequence"] == 1 and restarted.job("a")["status"] == "generating" and restarted.job("b")["status"] == "queued"
    restarted.step()
    assert session.inbox() == ["0001.json"] and (session.run / proto.INBOX_DIR / "0001.json").read_bytes() == published  # not published twice
    session.serve(1)
    restarted.step()
    restarted.step()
    assert restarted.job("a")["status"] == "complete" and restarted.job("b")["sequence"] == 2 and session.inbox() == ["0001.json", "0002.json"]
    assert ask(client, restarted, "a")["status"] == "complete"  # a client that retries its key gets the finished job, not a second run


def test_a_number_made_durable_before_publication_is_used_after_a_crash(tmp_path):
    """The process dies between writing the sequence number and publishing: the next start publishes under that number."""
    session = Session(tmp_path)
    client = session.client()
    queue = JobQueue(tmp_path / "state", client)
    ask(client, queue, "a")
    real_publish = client.publish

    def crash(job, state):
        raise KeyboardInterrupt  # not an Exception: nothing is recorded, as when the process is killed

    client.publish = crash
    with pytest.raises(KeyboardInterrupt):
        queue.step()
    assert session.inbox() == [] and json.loads((tmp_path / "state" / "chats.json").read_text())["jobs"][0]["sequence"] == 1
    client.publish = real_publish
    restarted = JobQueue(tmp_path / "state", session.client())
    restarted.step()
    assert session.inbox() == ["0001.json"] and restarted.job("a")["sequence"] == 1 and restarted.error is None


def test_a_halt_keeps_the_identity_and_refuses_everything_after(tmp_path):
    session = Session(tmp_path)
    client = session.client()
    queue = JobQueue(tmp_path / "state", client)
    ask(client, queue, "a")
    queue.step()
    other = client.prepare_api([{"role": "user", "content": "someone else's"}], "x", tools=None, effort="max", max_new_tokens=4)
    os.unlink(session.run / proto.INBOX_DIR / "0001.json")
    (session.run / proto.INBOX_DIR / "0001.json").write_text(json.dumps(other))  # another producer took the number
    queue.step()
    assert queue.error == "Resident sequence belongs to a different request." and queue.job("a")["sequence"] == 1
    halt = json.loads((tmp_path / "state" / job_queue.HALT_RECORD).read_text())
    assert halt["job"] == "a" and halt["error"] == queue.error
    queue.step()
    assert queue.job("a")["status"] == "generating" and session.inbox() == ["0001.json"]  # nothing is retried under a new number
    with pytest.raises(ApiError) as refused:
        ask(client, queue, "b")
    assert refused.value.status == 503 and refused.value.kind == "server_error"
    assert queue.job("b") is None


def test_a_session_that_is_gone_halts_the_queue_without_publishing(tmp_path):
    session = Session(tmp_path)
    client = session.client()
    queue = JobQueue(tmp_path / "state", client)
    ask(client, queue, "a")
    (session.run / proto.CONTROLLER_TERMINAL_FILE).write_text("{}")
    queue.step()
    assert "has ended" in queue.error and session.inbox() == [] and queue.job("a")["sequence"] is None


def test_limits(tmp_path, monkeypatch):
    session = Session(tmp_path)
    client = session.client()
    queue = JobQueue(tmp_path / "state", client)
    for i in range(PENDING):
        ask(client, queue, f"k{i}")
    with pytest.raises(ApiError) as refused:
        ask(client, queue, "one-too-many")
    assert refused.value.status == 429 and queue.pending() == PENDING and queue.job("one-too-many") is None
    assert ask(client, queue, "k3")["id"] == "k3"  # a key that is already queued is not a new admission

    monkeypatch.setattr(job_queue, "API_HISTORY", 3)
    for job in queue.db["jobs"]:
        job["status"] = "complete"
    for i in range(3):
        ask(client, queue, f"late{i}")
    finished = [j["id"] for j in queue.db["jobs"] if j["status"] == "complete"]
    assert finished == ["k7", "k8", "k9"]  # the oldest finished stateless jobs are forgotten, the newest three stay
    assert [j["id"] for j in queue.db["jobs"] if j["status"] == "queued"] == ["late0", "late1", "late2"]
    assert API_HISTORY == 50


def test_the_state_directory_is_private_and_the_job_view_is_detached(tmp_path):
    open_dir = tmp_path / "open"
    open_dir.mkdir(mode=0o755)
    with pytest.raises(ValueError, match="must be private"):
        JobQueue(open_dir, None)
    session = Session(tmp_path)
    client = session.client()
    queue = JobQueue(tmp_path / "fresh" / "state", client)
    assert stat.S_IMODE((tmp_path / "fresh" / "state").stat().st_mode) == 0o700
    ask(client, queue, "a")
    assert stat.S_IMODE((tmp_path / "fresh" / "state" / "chats.json").stat().st_mode) == 0o600
    view = queue.job("a")
    assert "payload" not in view and view["prompt_tokens"] > 0
    view["status"] = "complete"
    assert queue.job("a")["status"] == "queued" and queue.job("missing") is None


def test_one_server_per_session(tmp_path):
    """The inbox has one producer: a second server on the same run directory is refused, in this process or another."""
    import subprocess
    import sys

    from glm_tpu_b200.entrypoints.serve.server import ProducerBusy, hold_producer_lock

    session = Session(tmp_path)
    first = hold_producer_lock(session.run)
    lock = session.run / proto.INBOX_DIR / proto.PRODUCER_LOCK
    assert lock.read_text().strip() == str(os.getpid()) and stat.S_IMODE(lock.stat().st_mode) == 0o600
    with pytest.raises(ProducerBusy, match="one producer per session"):
        hold_producer_lock(session.run)
    probe = ("import sys; from pathlib import Path; from glm_tpu_b200.entrypoints.serve.server import hold_producer_lock, ProducerBusy\n"
             "try:\n    hold_producer_lock(Path(sys.argv[1])); print('held')\nexcept ProducerBusy as e:\n    print('busy')\n")
    done = subprocess.run([sys.executable, "-c", probe, str(session.run)], capture_output=True, text=True, timeout=120)
    assert done.stdout.strip() == "busy", done.stderr
    os.close(first)
    done = subprocess.run([sys.executable, "-c", probe, str(session.run)], capture_output=True, text=True, timeout=120)
    assert done.stdout.strip() == "held", done.stderr  # released with the descriptor (or the process): the next server gets it
    with pytest.raises(ProducerBusy, match="no inbox"):
        hold_producer_lock(tmp_path / "not-a-run")
    # the lock file is not a request: the client still claims the next number, and the controller's loop never reads it as one
    assert session.client().next_sequence() == 1 and proto.PRODUCER_LOCK not in (proto.inbox_name(n) for n in range(3))
