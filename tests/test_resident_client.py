"""The client side of a resident session against a run directory made by hand: liveness, claiming a sequence number, create-once
publication, and the completion check that accepts an answer only when the controller's measurement agrees with the token
stream that was read.

Reference counterparts: ``tests/engine/test_resident_client.py``, ``tests/engine/test_resident_protocol.py``."""

import hashlib
import json
import os
import struct
import subprocess
import sys

import pytest

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.engine.resident_client import Resident, ResidentUnavailable
from glm_tpu_b200.exceptions import ApiError, RequestValidationError
from glm_tpu_b200.tokenizer import ByteTokenizer

EOS = (1021, 1022, 1023)
PROFILE = rq.RequestProfile(vocab_size=1024, eos_ids=EOS, capacities=(512,), prompt_limits={512: 512}, concurrent_capacity=512, max_new=256)


def session(tmp_path, *, pid=None, ready=None, world=2):
    run = tmp_path / "run"
    (run / proto.INBOX_DIR).mkdir(parents=True)
    (run / proto.CONTROLLER_IDENTITY_FILE).write_text(json.dumps({"pid": os.getpid() if pid is None else pid}))
    if ready is not None:
        (run / proto.READY_FILE).write_text(json.dumps({"sequence": ready}))
    return run, Resident(run, ByteTokenizer(1024, EOS), PROFILE, capacity=512, world=world)


def finished(run, sequence, payload, ids, *, finish="eos", agree=True, ranks=2, emitted=None, digest=None, extra_reports=()):
    """Write the records a finished request leaves: the rank-0 token stream and the controller's measurement."""
    root = proto.result_dir(run, sequence)
    root.mkdir(exist_ok=True)
    rid = payload["request_id"]
    (root / proto.TOKENS_FILE).write_text("".join(json.dumps({"request_id": rid, "index": i, "token_id": t, "finish_reason": None}) + "\n"
                                                   for i, t in enumerate(ids)))
    report = {"request_id": rid, "finish_reason": finish, "emitted": len(ids) if emitted is None else emitted,
              "token_sha256": digest or hashlib.sha256(struct.pack(f"<{len(ids)}i", *ids)).hexdigest(), "decode_tokens_per_second": 123.0,
              "prefill_seconds": 0.05}
    (root / proto.MEASUREMENT_FILE).write_text(json.dumps({"agree": agree, "ranks": ranks, "requests": [report, *extra_reports]}))


# ------------------------------------------------------------------------------------------------ protocol names
def test_names_in_a_run_directory(tmp_path):
    assert proto.inbox_name(0) == "0000.json" and proto.inbox_name(12) == "0012.json" and proto.inbox_name(12345) == "12345.json"
    assert proto.result_dir(tmp_path, 0) == tmp_path and proto.result_dir(tmp_path, 3) == tmp_path / "resident-0003"
    assert proto.runner_file(5) == "runner.rank5.json" and proto.worker_started_file(0) == "worker_started.rank0.json"
    with pytest.raises(ValueError):
        proto.inbox_name(-1)
    line = proto.encode_command(2, {"b": 1, "a": "ü"})
    assert line == '{"request":{"a":"ü","b":1},"sequence":2}\n'.encode("utf-8") and line.count(b"\n") == 1
    assert proto.STOP_COMMAND == b'{"stop":true}\n' and json.loads(proto.STOP_COMMAND) == {"stop": True}


# ------------------------------------------------------------------------------------------------ liveness
def test_a_session_must_look_alive(tmp_path):
    run, client = session(tmp_path)
    client.check()
    (run / proto.CONTROLLER_TERMINAL_FILE).write_text("{}")
    with pytest.raises(ResidentUnavailable, match="has ended"):
        client.check()
    (run / proto.CONTROLLER_TERMINAL_FILE).unlink()
    (run / proto.CONTROLLER_IDENTITY_FILE).unlink()
    with pytest.raises(ResidentUnavailable, match="unavailable"):
        client.check()
    with pytest.raises(ResidentUnavailable, match="unavailable"):
        Resident(tmp_path / "nowhere", client.tokenizer, PROFILE, capacity=512).check()


def test_a_dead_controller_is_noticed(tmp_path):
    child = subprocess.Popen([sys.executable, "-c", "pass"])
    child.wait()
    run, client = session(tmp_path, pid=child.pid)  # that process has exited and was reaped: its pid names nobody
    with pytest.raises(ResidentUnavailable, match="controller is gone"):
        client.check()
    with pytest.raises(ResidentUnavailable):
        client.prepare([{"role": "user", "content": "hi"}], "k")
    with pytest.raises(ResidentUnavailable):
        client.next_sequence()


# ------------------------------------------------------------------------------------------------ preparing
def test_prepared_turns_fit_the_loaded_context(tmp_path):
    run, client = session(tmp_path, ready=0)
    messages = [{"role": "user", "content": "What is two plus two?"}]
    turn = client.prepare(messages, "abc")
    rq.validate(turn, PROFILE)
    assert turn["request_id"] == "ui-abc" and turn["context_capacity"] == 512
    assert turn["max_new_tokens"] == min(PROFILE.max_new, 512 - len(turn["prompt_ids"]))
    api = client.prepare_api(messages, "abc", tools=None, effort="max", max_new_tokens=7)
    assert api["request_id"] == "api-abc" and api["max_new_tokens"] == 7 and api["prompt_ids"] == turn["prompt_ids"]
    assert client.prepare_api(messages, "abc", tools=None, effort="max", max_new_tokens=None)["max_new_tokens"] == PROFILE.max_new
    assert client.prepare_api(messages, "abc", tools=None, effort="max", max_new_tokens=10**9)["max_new_tokens"] == PROFILE.max_new
    long = [{"role": "user", "content": "x" * 600}]
    with pytest.raises(ApiError, match="fills the 512-slot context; start a new one"):
        client.prepare(long, "abc")
    with pytest.raises(ApiError, match="send less history"):
        client.prepare_api(long, "abc", tools=None, effort="max", max_new_tokens=5)


# ------------------------------------------------------------------------------------------------ claiming and publishing
def test_the_next_sequence_follows_the_ready_file(tmp_path):
    run, client = session(tmp_path)
    with pytest.raises(ValueError, match="still loading"):
        client.next_sequence()
    (run / proto.READY_FILE).write_text(json.dumps({"sequence": 0}))
    assert client.next_sequence() == 1
    (run / proto.READY_FILE).write_text(json.dumps({"sequence": 2}))
    with pytest.raises(ValueError, match="still collecting"):
        client.next_sequence()  # request 2 is done on the GPUs, its measurement is not filed yet
    proto.result_dir(run, 2).mkdir()
    (proto.result_dir(run, 2) / proto.MEASUREMENT_FILE).write_text("{}")
    assert client.next_sequence() == 3
    (run / proto.INBOX_DIR / proto.inbox_name(3)).write_text("{}")
    with pytest.raises(ValueError, match="another request owner"):
        client.next_sequence()
    (run / proto.INBOX_DIR / proto.inbox_name(3)).unlink()
    (run / proto.INBOX_DIR / proto.inbox_name(1)).write_text("{}")  # answered requests stay in the inbox: they do not block
    (run / proto.INBOX_DIR / proto.STOP_FILE).write_text("{}")  # nor does a name that is not a number
    assert client.next_sequence() == 3


def test_publication_is_create_once(tmp_path):
    run, client = session(tmp_path, ready=0)
    state = tmp_path / "state"
    state.mkdir()
    payload = client.prepare([{"role": "user", "content": "first"}], "one")
    job = {"id": "job-1", "sequence": 1, "payload": payload}
    client.publish(job, state)
    target = run / proto.INBOX_DIR / "0001.json"
    assert json.loads(target.read_text()) == payload
    assert os.stat(target).st_ino == os.stat(state / "job-1.request.json").st_ino  # a hard link: published whole or not at all
    client.publish(job, state)  # the same request again (a restart of the server): nothing changes

    other = client.prepare([{"role": "user", "content": "second"}], "two")
    with pytest.raises(ValueError, match="belongs to a different request"):
        client.publish({"id": "job-2", "sequence": 1, "payload": other}, state)
    assert json.loads(target.read_text()) == payload  # the first producer's request is untouched
    with pytest.raises(ValueError, match="Saved request identity differs"):
        client.publish({"id": "job-1", "sequence": 2, "payload": other}, state)
    assert not (run / proto.INBOX_DIR / "0002.json").exists()

    tampered = dict(payload, max_new_tokens=payload["max_new_tokens"] - 1)  # identity no longer matches the body
    with pytest.raises(RequestValidationError):
        client.publish({"id": "job-3", "sequence": 3, "payload": tampered}, state)
    assert not (state / "job-3.request.json").exists() and not (run / proto.INBOX_DIR / "0003.json").exists()

    outside = tmp_path / "outside.json"
    outside.write_text(json.dumps(other))
    (run / proto.INBOX_DIR / "0004.json").symlink_to(outside)  # a planted link with the right content is still not ours
    with pytest.raises(ValueError, match="belongs to a different request"):
        client.publish({"id": "job-4", "sequence": 4, "payload": other}, state)


# ------------------------------------------------------------------------------------------------ observing
def test_progress_and_completion(tmp_path):
    run, client = session(tmp_path, ready=0)
    payload = client.prepare([{"role": "user", "content": "2+2?"}], "q")
    job = {"id": "j", "sequence": 1, "payload": payload}
    tok = client.tokenizer
    assert client.observe(job) == {"thinking": "", "answer": "", "output_tokens": 0, "status": "generating"}

    ids = tok.encode("adding</think>Four.") + [EOS[0]]
    root = proto.result_dir(run, 1)
    root.mkdir()
    lines = [json.dumps({"request_id": payload["request_id"], "index": i, "token_id": t, "finish_reason": None}) + "\n" for i, t in enumerate(ids)]
    (root / proto.TOKENS_FILE).write_text("".join(lines[:6]) + lines[6][:-5])  # the seventh line is still being written
    seen = client.observe(job)
    assert seen["output_tokens"] == 6 and seen["status"] == "generating" and seen["thinking"] == "adding"[:6] and seen["answer"] == ""

    finished(run, 1, payload, ids)
    done = client.observe(job)
    assert done["status"] == "complete" and done["answer"] == "Four." and done["thinking"] == "adding" and done["output_tokens"] == len(ids)
    assert done["finish_reason"] == "eos" and done["stop_cause"] == "eos" and done["decode_tps"] == 123.0 and done["prefill_seconds"] == 0.05

    finished(run, 1, payload, ids[:-1], finish="length")  # the output cap ended it: an answer, but not a complete one
    cut = client.observe(job)
    assert cut["status"] == "incomplete" and cut["stop_cause"] == "output_cap" and cut["answer"] == "Four."
    finished(run, 1, payload, tok.encode("still thinking") + [EOS[1]])  # ended without ever leaving the reasoning section
    assert client.observe(job)["status"] == "incomplete"


@pytest.mark.parametrize("change,match", [
    ({"agree": False}, "completion check failed"),
    ({"ranks": 1}, "completion check failed"),
    ({"extra_reports": ({"request_id": "ui-q", "finish_reason": "eos", "emitted": 1, "token_sha256": "0" * 64},)}, "completion check failed"),
    ({"digest": "0" * 64}, "agreement failed"),
    ({"emitted": 3}, "agreement failed"),
])
def test_a_measurement_that_does_not_match_the_stream_is_refused(tmp_path, change, match):
    run, client = session(tmp_path, ready=0)
    payload = client.prepare([{"role": "user", "content": "2+2?"}], "q")
    ids = client.tokenizer.encode("</think>Four.") + [EOS[0]]
    finished(run, 1, payload, ids, **change)
    with pytest.raises(ValueError, match=match):
        client.observe({"id": "j", "sequence": 1, "payload": payload})


def test_a_foreign_or_reordered_token_stream_is_refused(tmp_path):
    run, client = session(tmp_path, ready=0)
    payload = client.prepare([{"role": "user", "content": "2+2?"}], "q")
    job = {"id": "j", "sequence": 1, "payload": payload}
    root = proto.result_dir(run, 1)
    root.mkdir()
    event = lambda rid, i: json.dumps({"request_id": rid, "index": i, "token_id": 65, "finish_reason": None}) + "\n"  # noqa: E731
    (root / proto.TOKENS_FILE).write_text(event("ui-other", 0))
    with pytest.raises(ValueError, match="Token stream identity differs"):
        client.observe(job)
    (root / proto.TOKENS_FILE).write_text(event("ui-q", 0) + event("ui-q", 2))
    with pytest.raises(ValueError, match="Token stream identity differs"):
        client.observe(job)
    (root / proto.TOKENS_FILE).write_text(event("ui-q", 0) + event("ui-q", 1))
    assert client.observe(job)["output_tokens"] == 2


def test_observing_notices_a_session_that_died_mid_answer(tmp_path):
    run, client = session(tmp_path, ready=0)
    payload = client.prepare([{"role": "user", "content": "2+2?"}], "q")
    (run / proto.CONTROLLER_TERMINAL_FILE).write_text("{}")
    with pytest.raises(ResidentUnavailable, match="has ended"):
        client.observe({"id": "j", "sequence": 1, "payload": payload})
    finished(run, 1, payload, client.tokenizer.encode("</think>Four.") + [EOS[0]])
    assert client.observe({"id": "j", "sequence": 1, "payload": payload})["status"] == "complete"  # a filed answer outlives its session


# ------------------------------------------------------------------------------------------------ preparing a conversation by hand
def test_a_whole_conversation_becomes_one_prepared_request():
    tok = ByteTokenizer(1024, EOS)
    chat = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "4"},
            {"role": "user", "content": "and 3+3?"}]
    prepared = rq.from_messages(chat, tokenizer=tok, request_id="follow-up", context_capacity=512, profile=PROFILE)
    rq.validate(prepared, PROFILE)
    text = tok.decode(prepared["prompt_ids"])
    assert text.startswith("[gMASK]<sop><|system|>Reasoning Effort: Max<|system|>Be brief.<|user|>2+2?") and text.endswith("<|user|>and 3+3?<|assistant|><think>")
    assert prepared["max_new_tokens"] == min(PROFILE.max_new, 512 - len(prepared["prompt_ids"])) and prepared["request_id"] == "follow-up"
    capped = rq.from_messages(chat, tokenizer=tok, request_id="r", max_new_tokens=5, context_capacity=512, profile=PROFILE, reasoning_effort="low")
    assert capped["max_new_tokens"] == 5 and "Reasoning Effort: Low" in tok.decode(capped["prompt_ids"])
    user = {"role": "user", "content": "q"}
    for bad, sentence in (([], "non-empty list"), ("hi", "non-empty list"), ([user, {"role": "assistant", "content": "a"}], "a user message last"),
                          ([user, {"role": "system", "content": "s"}, user], "first place only"), ([{"role": "tool", "content": "r"}, user], "exactly a role"),
                          ([{"role": "user", "content": ["q"]}], "exactly a role"), ([dict(user, name="n")], "exactly a role"), ([{"role": "user"}], "exactly a role"),
                          ([{"role": "user", "content": "x" * (rq.MESSAGES_CAP + 1)}], "bytes of messages")):
        with pytest.raises(RequestValidationError, match=sentence):
            rq.from_messages(bad, tokenizer=tok, request_id="r", context_capacity=512, profile=PROFILE)
    with pytest.raises(RequestValidationError, match="fills the 512-slot context; nothing is truncated"):
        rq.from_messages([{"role": "user", "content": "x" * 600}], tokenizer=tok, request_id="r", context_capacity=512, profile=PROFILE)  # never truncated
    with pytest.raises(RequestValidationError, match="unsupported context capacity"):
        rq.from_messages([user], tokenizer=tok, request_id="r", context_capacity=4096, profile=PROFILE)


def test_reading_a_prepared_request_from_a_file(tmp_path):
    import hashlib as hl

    tok = ByteTokenizer(1024, EOS)
    prepared = rq.from_messages([{"role": "user", "content": "q"}], tokenizer=tok, request_id="r", context_capacity=512, profile=PROFILE)
    path = tmp_path / "request.json"
    path.write_text(json.dumps(prepared))
    digest = hl.sha256(path.read_bytes()).hexdigest()
    assert rq.read(path, PROFILE) == prepared and rq.read(path, PROFILE, expected_sha256=digest) == prepared
    batch = rq.batch([prepared], profile=PROFILE)
    (tmp_path / "batch.json").write_text(json.dumps(batch))
    assert rq.read(tmp_path / "batch.json", PROFILE) == batch
    for make, sentence in ((lambda: rq.read(path, PROFILE, expected_sha256="0" * 64), "not the pinned one"),
                           (lambda: rq.read(tmp_path / "absent.json", PROFILE), "cannot be read"),
                           (lambda: rq.read(tmp_path, PROFILE), "cannot be read")):
        with pytest.raises(RequestValidationError, match=sentence):
            make()
    (tmp_path / "link.json").symlink_to(path)
    with pytest.raises(RequestValidationError, match="cannot be read.*symlink"):
        rq.read(tmp_path / "link.json", PROFILE)
    path.write_text("{not json")
    with pytest.raises(RequestValidationError, match="not JSON"):
        rq.read(path, PROFILE)
    path.write_text(json.dumps(dict(prepared, max_new_tokens=prepared["max_new_tokens"] - 1)))
    with pytest.raises(RequestValidationError, match="identity or fixed profile differs"):
        rq.read(path, PROFILE)


def test_prepare_request_refuses_to_write_into_the_checkout(tmp_path, capsys):
    from pathlib import Path

    from glm_tpu_b200.entrypoints.cli import main as cli

    messages = tmp_path / "m.json"
    messages.write_text(json.dumps([{"role": "user", "content": "hi"}]))
    inside = Path(cli.__file__).resolve().parents[3] / "tests" / "would-be-private.json"
    code = cli.main(["prepare-request", "--messages", str(messages), "--output", str(inside), "--model", "random:tiny", "--capacity", "256"])
    assert code == 2 and "outside the source checkout" in capsys.readouterr().err and not inside.exists()
    code = cli.main(["prepare-request", "--messages", str(messages), "--output", str(tmp_path / "p.json"), "--model", "random:tiny", "--capacity", "256"])
    assert code == 0 and (tmp_path / "p.json").stat().st_mode & 0o077 == 0
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps([{"role": "assistant", "content": "I speak first"}]))
    code = cli.main(["prepare-request", "--messages", str(bad), "--output", str(tmp_path / "q.json"), "--model", "random:tiny", "--capacity", "256"])
    assert code == 2 and "a user message last" in capsys.readouterr().err and not (tmp_path / "q.json").exists()
