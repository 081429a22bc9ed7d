"""Request schema, sessions, the vote schedule and the engine's failure model (CPU, fake device)."""

import json

import pytest

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.engine.llm_engine import LLMEngine
from glm_tpu_b200.engine.outputs import TokenEvent, final_channel
from glm_tpu_b200.engine.request_session import LocalVote
from glm_tpu_b200.exceptions import EngineFailure, RequestValidationError
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes
from tests.fakes import FakeRunner, Script, StrandedVote, ThreadFleet

PROFILE = rq.RequestProfile(vocab_size=1000, eos_ids=(997, 998, 999), capacities=(64, 128), prompt_limits={64: 64, 128: 128},
                            concurrent_capacity=64, max_new=100)


def make(ids=(1, 2, 3), rid="r1", n=5, cap=64):
    return rq.from_token_ids(list(ids), request_id=rid, max_new_tokens=n, context_capacity=cap, profile=PROFILE)


# ---------------------------------------------------------------------------------------- schema
def test_request_is_self_hashed_and_validates():
    r = make()
    rq.validate(r, PROFILE)
    body = {k: v for k, v in r.items() if k != "request_sha256"}
    import hashlib

    assert r["request_sha256"] == hashlib.sha256(canonical_wire_bytes(body)).hexdigest()
    assert r["decode_policy"] == "greedy" and r["eos_ids"] == [997, 998, 999]
    tampered = dict(r, max_new_tokens=6)
    with pytest.raises(RequestValidationError):
        rq.validate(tampered, PROFILE)


@pytest.mark.parametrize("kw", [dict(ids=[]), dict(ids=[1000]), dict(ids=[1, -1]), dict(n=0), dict(cap=63), dict(ids=list(range(60)), n=5),
                                dict(rid=""), dict(ids=[True])])
def test_request_refusals(kw):
    with pytest.raises(RequestValidationError):
        make(**kw)


def test_production_profile_constants():
    assert rq.CAPACITIES == (8192, 32768, 166912, 262144)
    assert rq.GLM53_PROFILE.vocab_size == 154880 and rq.GLM53_PROFILE.eos_ids == (154820, 154827, 154829)
    assert rq.default_max_new_tokens(200, 8192) == 8192 - 200
    assert rq.default_max_new_tokens(200, 262144) == rq.MAX_NEW


def test_batches():
    a, b = make(rid="a"), make(rid="b")
    seq = rq.batch([a, b], profile=PROFILE)
    assert seq["schema"] == rq.BATCH_SCHEMA and rq.requests_of(seq, PROFILE) == [a, b]
    con = rq.batch([a, b], concurrent=True, profile=PROFILE)
    assert rq.is_concurrent(con)
    with pytest.raises(RequestValidationError):
        rq.batch([a, a], profile=PROFILE)  # duplicate ids
    with pytest.raises(RequestValidationError):
        rq.batch([make(rid=str(i)) for i in range(5)], concurrent=True, profile=PROFILE)  # more than four chats
    with pytest.raises(RequestValidationError):
        rq.batch([make(rid="c", cap=128)], concurrent=True, profile=PROFILE)  # wrong profile for concurrency
    with pytest.raises(RequestValidationError):
        rq.validate_payload(dict(seq, context_capacity=128), PROFILE)


def test_stop_causes():
    assert rq.stop_cause(make(), "eos") == "eos"
    assert rq.stop_cause(make(n=5), "length") == "output_cap"
    assert rq.stop_cause(make(ids=range(10), n=54), "length") == "context_exhausted"


def test_final_channel():
    assert final_channel("<think>a b</think> answer <|user|> more") == ("a b", "answer")
    assert final_channel("<think>still thinking") == ("still thinking", "")
    assert TokenEvent("r", 0, 5, None).wire() == {"request_id": "r", "index": 0, "token_id": 5, "finish_reason": None}
    assert "batch_round" in TokenEvent("r", 0, 5, None, batch_round=2).wire()


# ---------------------------------------------------------------------------------------- engine
def test_generate_schedule_and_report():
    runner, vote, events = FakeRunner(), LocalVote(), []
    engine = LLMEngine(runner, vote=vote, profile=PROFILE)
    report = engine.generate(make(n=4), events.append)
    assert [e.index for e in events] == [0, 1, 2, 3] and events[-1].finish_reason == "length"
    assert report["emitted"] == 4 and report["timed_decode_tokens"] == 3 and report["stop_cause"] == "output_cap"
    # memory admission first, the prefill pair, then (validity, delivery) per decode step, in this exact order
    assert [p for p, _ in vote.log] == ["admission", "prefill_validity", "prefill_delivery"] + ["validity", "delivery"] * 3
    assert ("deactivate", 0) in runner.log
    assert report["token_sha256"] and report["prompt_tokens"] == 3


def test_eos_stops_early_and_fresh_cache_per_request():
    runner = FakeRunner(script=Script(eos_at={0: 2}))
    engine = LLMEngine(runner, profile=PROFILE)
    report = engine.generate(make(n=10))
    assert report["finish_reason"] == "eos" and report["emitted"] == 3
    again = engine.generate(make(n=10, rid="r2"))
    assert again["token_sha256"] == report["token_sha256"]  # same prompt, fresh state -> same tokens


@pytest.mark.parametrize("script", [Script(bad_status_at=1), Script(bad_token_at=0), Script(fail_prefill=True)])
def test_failure_poisons_the_engine(script):
    engine = LLMEngine(FakeRunner(script=script), profile=PROFILE)
    with pytest.raises(EngineFailure):
        engine.generate(make(n=6))
    assert engine.poisoned
    with pytest.raises(EngineFailure):
        engine.generate(make(n=6, rid="next"))


def test_failed_delivery_is_voted_not_retried():
    events = []

    def sink(ev):
        if ev.index == 2:
            raise OSError("disk full")
        events.append(ev)

    engine = LLMEngine(FakeRunner(), profile=PROFILE)
    with pytest.raises(EngineFailure):
        engine.generate(make(n=6), sink)
    assert [e.index for e in events] == [0, 1] and engine.poisoned


def test_deadline_is_folded_into_the_vote():
    now = [0.0]
    engine = LLMEngine(FakeRunner(), profile=PROFILE, clock=lambda: now.__setitem__(0, now[0] + 1.0) or now[0])
    with pytest.raises(EngineFailure):
        engine.generate(make(n=50), deadline=10.0)


def test_wrong_capacity_is_refused_without_poisoning():
    engine = LLMEngine(FakeRunner(capacity=64), profile=PROFILE)
    with pytest.raises(RequestValidationError):
        engine.generate(make(cap=128))
    assert not engine.poisoned


def test_concurrent_lanes_freeze_independently():
    runner = FakeRunner(lanes=4, script=Script(eos_at={1: 2}))
    events = []
    engine = LLMEngine(runner, profile=PROFILE)
    reqs = [make(rid=f"c{i}", ids=(i + 1, 2, 3), n=5) for i in range(3)]
    reports = engine.generate_concurrent(rq.batch(reqs, concurrent=True, profile=PROFILE), events.append)
    assert [r["emitted"] for r in reports] == [5, 3, 5] and reports[1]["finish_reason"] == "eos"
    # the unused fourth lane and the finished lane are frozen while the others continue
    assert ("deactivate", 3) in runner.log and ("deactivate", 1) in runner.log
    last = [e for e in runner.log if e[0] == "decode"][-1]
    assert last[2] == (True, False, True, False)
    solo = LLMEngine(FakeRunner(), profile=PROFILE).generate(make(rid="solo", ids=(1, 2, 3), n=5))
    assert solo["token_sha256"] == reports[0]["token_sha256"]  # a lane's tokens do not depend on its neighbours
    assert all(e.batch_round is not None for e in events)


# ---------------------------------------------------------------------------------------- several ranks
def test_ranks_fail_together_when_one_rank_sees_a_dirty_status():
    fleet = ThreadFleet(2)

    def body(rank):
        script = Script(bad_status_at=1) if rank == 1 else Script()
        engine = LLMEngine(FakeRunner(rank=rank, script=script), vote=fleet.vote(rank), profile=PROFILE)
        return engine.generate(make(n=6))

    out = fleet.run(body)
    assert all(isinstance(o, EngineFailure) for o in out), out
    assert fleet.log[-1] == ("validity", False)


def test_token_disagreement_is_caught_by_the_digest_consensus():
    fleet = ThreadFleet(2)
    digests = {}

    def body(rank):
        def consensus(d):
            digests[rank] = d
            ok = fleet.vote(rank + 100).all(True, "noop") if False else True
            return ok and (len(digests) < 2 or len(set(digests.values())) == 1)

        engine = LLMEngine(FakeRunner(rank=rank, script=Script(rank_token_skew_at=1)), vote=fleet.vote(rank), profile=PROFILE,
                           digest_consensus=consensus)
        return engine.generate(make(n=4))

    out = fleet.run(body)
    assert any(isinstance(o, EngineFailure) for o in out)


def test_a_rank_that_never_votes_strands_its_peer_loudly():
    fleet = ThreadFleet(2, timeout=0.5)

    def body(rank):
        if rank == 1:
            return "left early"
        return LLMEngine(FakeRunner(), vote=fleet.vote(rank), profile=PROFILE).generate(make(n=3))

    out = fleet.run(body)
    assert isinstance(out[0], StrandedVote)


def test_token_events_are_json_lines():
    events = []
    LLMEngine(FakeRunner(), profile=PROFILE).generate(make(n=2), events.append)
    line = json.dumps(events[0].wire(), sort_keys=True, separators=(",", ":"))
    assert line.startswith('{"finish_reason":null,"index":0,"request_id":"r1","token_id":')
