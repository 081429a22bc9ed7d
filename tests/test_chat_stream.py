"""The event stream of ``/v1/chat/completions`` driven by scripted job snapshots: the channels never mix, nothing is sent twice or
lost, text that turns out to be a tool call is never sent as content, and every way a job can end maps to its finish reason.

Reference counterpart: ``tests/entrypoints/openai/test_serving_chat.py`` (stream separation, finish reasons, deadlines)."""

import json

import pytest

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.entrypoints.openai import serving_chat
from glm_tpu_b200.entrypoints.openai.serving_chat import OpenAIServingChat, _content_so_far
from glm_tpu_b200.exceptions import ApiError
from glm_tpu_b200.tokenizer import ByteTokenizer

PROFILE = rq.RequestProfile(vocab_size=1024, eos_ids=(1021, 1022, 1023), capacities=(4096,), prompt_limits={4096: 4096}, concurrent_capacity=4096)
CALL = "<tool_call>read<arg_key>path</arg_key><arg_value>a.txt</arg_value></tool_call>"


class Backend:
    def __init__(self):
        self.tokenizer = ByteTokenizer(1024, PROFILE.eos_ids)

    def prepare_api(self, messages, key, *, tools, effort, max_new_tokens, context_capacity):
        ids = self.tokenizer.apply_chat_template(messages, tools=tools, reasoning_effort=effort)
        return rq.from_token_ids(ids, request_id="api-" + key, max_new_tokens=max_new_tokens or 64, context_capacity=context_capacity, profile=PROFILE)


class ScriptedQueue:
    """``submit`` accepts; ``job`` plays the given snapshots in order and repeats the last one."""

    def __init__(self, snapshots):
        self.snapshots, self.reads, self.submitted = snapshots, 0, []

    def submit(self, payload, key, *, label):
        self.submitted.append((key, label, payload["request_id"]))

    def job(self, key):
        snap = self.snapshots[min(self.reads, len(self.snapshots) - 1)]
        self.reads += 1
        if snap is None:
            return None
        base = {"id": key, "status": "generating", "thinking": "", "answer": "", "prompt_tokens": 11, "output_tokens": 0, "created": 1700000000.0}
        return {**base, **snap}


def run(snapshots, body=None, **kw):
    queue = ScriptedQueue(snapshots)
    chat = OpenAIServingChat(queue, Backend(), capacity=4096, wait_seconds=kw.pop("wait_seconds", 30), poll_seconds=0.0)
    body = body or {"messages": [{"role": "user", "content": "hi"}], "stream": True}
    chunks = list(chat.stream(body))
    assert chunks[-1] == b"data: [DONE]\n\n" and all(c.startswith(b"data: ") and c.endswith(b"\n\n") for c in chunks)
    events = [json.loads(c[6:]) for c in chunks[:-1]]
    assert len({e["id"] for e in events}) == 1 and all(e["object"] == "chat.completion.chunk" and len(e["choices"]) == 1 for e in events)
    return events, queue


def deltas(events, channel):
    return [e["choices"][0]["delta"][channel] for e in events if channel in e["choices"][0]["delta"]]


def test_channels_grow_separately_and_nothing_is_sent_twice():
    events, queue = run([
        {"thinking": "Let", "output_tokens": 1},
        {"thinking": "Let me add", "output_tokens": 3},
        {"thinking": "Let me add", "output_tokens": 3},  # a poll without growth sends nothing
        {"thinking": "Let me add.", "answer": "Fo", "output_tokens": 5},
        {"thinking": "Let me add.", "answer": "Four.", "output_tokens": 7, "status": "complete", "stop_cause": "eos"},
    ])
    assert events[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""} and events[0]["choices"][0]["finish_reason"] is None
    assert deltas(events, "reasoning_content") == ["Let", " me add", "."] and deltas(events[1:], "content") == ["Fo", "ur."]
    assert all(len(e["choices"][0]["delta"]) <= 1 for e in events[1:])  # one channel per event
    last = events[-1]
    assert last["choices"][0] == {"index": 0, "delta": {}, "logprobs": None, "finish_reason": "stop"}
    assert last["usage"] == {"prompt_tokens": 11, "completion_tokens": 7, "total_tokens": 18}
    assert queue.submitted[0][1] == "api" and queue.submitted[0][2] == "api-" + queue.submitted[0][0]
    assert events[0]["model"] == "glm-5.3"


def test_text_that_becomes_a_tool_call_is_never_content():
    events, _ = run([
        {"answer": "I will look.", "output_tokens": 4},
        {"answer": "I will look.<tool_c", "output_tokens": 5},               # may be the beginning of a call: held back
        {"answer": "I will look." + CALL[:30], "output_tokens": 9},          # it is one
        {"answer": "I will look." + CALL + " Then I continue.", "output_tokens": 20, "status": "complete", "stop_cause": "eos"},
    ])
    content = "".join(deltas(events[1:], "content"))
    assert content == "I will look. Then I continue." and "<" not in content
    calls = [e["choices"][0]["delta"]["tool_calls"][0] for e in events if "tool_calls" in e["choices"][0]["delta"]]
    assert len(calls) == 1 and calls[0]["index"] == 0 and calls[0]["function"] == {"name": "read", "arguments": '{"path": "a.txt"}'}
    assert calls[0]["id"].startswith("call_") and calls[0]["type"] == "function"
    assert events[-1]["choices"][0]["finish_reason"] == "tool_calls"
    order = ["tool_calls" if "tool_calls" in e["choices"][0]["delta"] else "content" for e in events[1:-1]]
    assert order.index("tool_calls") == len(order) - 1  # the calls come after all content


def test_a_tail_that_only_looked_like_a_tag_is_sent_once_it_is_decided():
    events, _ = run([
        {"answer": "a <", "output_tokens": 2},
        {"answer": "a <tool", "output_tokens": 3},
        {"answer": "a <tools> b", "output_tokens": 5, "status": "complete", "stop_cause": "eos"},
    ])
    assert "".join(deltas(events[1:], "content")) == "a <tools> b"
    assert _content_so_far("x<tool_call>y") == "x" and _content_so_far("x<tool_call") == "x" and _content_so_far("x<") == "x"
    assert _content_so_far("x<tool_calls") == "x<tool_calls" and _content_so_far("x < y") == "x < y" and _content_so_far("") == ""
    assert _content_so_far("<tool_call>") == "" and _content_so_far("a<b<tool") == "a<b"


@pytest.mark.parametrize("final,reason", [
    ({"status": "complete", "stop_cause": "eos", "answer": "ok"}, "stop"),
    ({"status": "incomplete", "stop_cause": "output_cap", "answer": "cut"}, "length"),
    ({"status": "incomplete", "stop_cause": "context_exhausted", "answer": "cut"}, "length"),
    ({"status": "incomplete", "stop_cause": "eos", "answer": ""}, "stop"),  # ended inside its reasoning: no answer, but not cut short
    ({"status": "incomplete", "stop_cause": "output_cap", "answer": CALL}, "tool_calls"),  # a call that made it out whole is a call
])
def test_finish_reasons(final, reason):
    events, _ = run([{**final, "thinking": "t", "output_tokens": 3}])
    assert events[-1]["choices"][0]["finish_reason"] == reason
    chat = OpenAIServingChat(ScriptedQueue([{**final, "thinking": "t", "output_tokens": 3}]), Backend(), capacity=4096, poll_seconds=0.0)
    reply = chat.completion({"messages": [{"role": "user", "content": "hi"}]})
    assert reply["choices"][0]["finish_reason"] == reason and reply["object"] == "chat.completion" and reply["created"] == 1700000000
    message = reply["choices"][0]["message"]
    assert message["reasoning_content"] == "t" and (message["content"] is None) == (final["answer"] in ("", CALL))


def test_a_job_that_fails_or_vanishes_ends_the_stream_with_its_status():
    queue = ScriptedQueue([{"thinking": "x", "output_tokens": 1}, {"error": "The resident controller is gone. No model was restarted."}])
    chat = OpenAIServingChat(queue, Backend(), capacity=4096, poll_seconds=0.0)
    stream = chat.stream({"messages": [{"role": "user", "content": "hi"}], "stream": True})
    next(stream), next(stream)
    with pytest.raises(ApiError) as failed:
        next(stream)
    assert failed.value.status == 503 and "controller is gone" in str(failed.value)
    chat = OpenAIServingChat(ScriptedQueue([None]), Backend(), capacity=4096, poll_seconds=0.0)
    with pytest.raises(ApiError) as lost:
        chat.completion({"messages": [{"role": "user", "content": "hi"}]})
    assert lost.value.status == 500


def test_the_server_deadline(monkeypatch):
    chat = OpenAIServingChat(ScriptedQueue([{"thinking": "still", "output_tokens": 1}]), Backend(), capacity=4096, wait_seconds=0.05, poll_seconds=0.01)
    with pytest.raises(ApiError) as late:
        chat.completion({"messages": [{"role": "user", "content": "hi"}]})
    assert late.value.status == 504 and late.value.kind == "timeout" and "use stream=true" in str(late.value)
    stream = chat.stream({"messages": [{"role": "user", "content": "hi"}], "stream": True})
    with pytest.raises(ApiError) as late:
        list(stream)
    assert late.value.status == 504 and "use stream=true" not in str(late.value)  # no such hint to a client that already streams


def test_fields_of_a_request():
    queue = ScriptedQueue([{"status": "complete", "stop_cause": "eos", "answer": "ok", "output_tokens": 1}])
    chat = OpenAIServingChat(queue, Backend(), capacity=4096, poll_seconds=0.0)
    ok = {"messages": [{"role": "user", "content": "hi"}]}
    for extra in ({"temperature": 0.3, "top_p": 0.9, "seed": 7, "presence_penalty": 1}, {"n": 1}, {"n": None}, {"max_tokens": 5}, {"model": None},
                  {"reasoning_effort": "low"}, {"tool_choice": "required"}, {"stream": False}, {"user": "someone"}):
        assert chat.completion({**ok, **extra})["choices"][0]["message"]["content"] == "ok"  # sampling fields are accepted and ignored
    for bad, status in (({**ok, "n": 2}, 400), ({**ok, "max_tokens": 0}, 400), ({**ok, "max_tokens": 2.5}, 400), ({**ok, "max_tokens": True}, 400),
                        ({**ok, "reasoning_effort": "medium"}, 400), ({**ok, "model": "gpt-4o"}, 404), ({"messages": []}, 400), ("hi", 400),
                        ({**ok, "tools": []}, 400), ({**ok, "tools": [{"function": {"name": "f"}}], "tool_choice": "sometimes"}, 400)):
        with pytest.raises(ApiError) as refused:
            chat.completion(bad)
        assert refused.value.status == status, bad
    assert serving_chat.ALIASES[serving_chat.MODEL_NAME] is None  # the plain name leaves the effort to the request
    prepared, key, model = chat.prepare({**ok, "model": "glm-5.3-low", "reasoning_effort": "max"})
    assert model == "glm-5.3-low" and "Reasoning Effort: Low" in Backend().tokenizer.decode(prepared["prompt_ids"])  # the alias outranks the field
