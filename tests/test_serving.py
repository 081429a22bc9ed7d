"""Job queue, conversation store, /v1 shaping, HTTP boundaries and the chat format (CPU, fake resident session)."""

import json
import threading
import urllib.error
import urllib.request
from http.server import ThreadingHTTPServer

import pytest

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.entrypoints.openai import chat_utils, tool_parser
from glm_tpu_b200.entrypoints.openai.protocol import ApiError
from glm_tpu_b200.entrypoints.openai.serving_chat import OpenAIServingChat
from glm_tpu_b200.entrypoints.openai.serving_models import OpenAIServingModels
from glm_tpu_b200.entrypoints.serve.http_handler import handler
from glm_tpu_b200.entrypoints.serve.job_queue import PENDING, JobQueue
from glm_tpu_b200.entrypoints.serve.security import api_token
from glm_tpu_b200.entrypoints.ui.conversations import ConversationStore
from glm_tpu_b200.tokenizer import ByteTokenizer, chat_template

PROFILE = rq.RequestProfile(vocab_size=1024, eos_ids=(1020, 1021, 1022), capacities=(4096,), prompt_limits={4096: 4096},
                            concurrent_capacity=4096, max_new=2000)


class FakeResident:
    """prepare / next_sequence / publish / observe without a model: answers are scripted per request."""

    def __init__(self, answers=None):
        self.capacity, self.profile = 4096, PROFILE
        self.tokenizer = ByteTokenizer(1024, PROFILE.eos_ids)
        self.answers = answers or {}
        self.published, self.sequence, self.polls = [], 0, {}
        self.fail_publish = False
        self.available = True

    def check(self):
        if not self.available:
            raise ValueError("The resident model is unavailable. No model was restarted.")

    def prepare(self, messages, key):
        ids = self.tokenizer.apply_chat_template(messages)
        return rq.from_token_ids(ids, request_id="ui-" + key, max_new_tokens=100, context_capacity=4096, profile=PROFILE)

    def prepare_api(self, messages, key, *, tools, effort, max_new_tokens, context_capacity):
        ids = self.tokenizer.apply_chat_template(messages, tools=tools, reasoning_effort=effort)
        self.last_prompt = self.tokenizer.decode(ids)
        return rq.from_token_ids(ids, request_id="api-" + key, max_new_tokens=max_new_tokens or 100, context_capacity=4096, profile=PROFILE)

    def next_sequence(self):
        self.sequence += 1
        return self.sequence

    def publish(self, job, state):
        if self.fail_publish:
            raise ValueError("Resident sequence belongs to a different request.")
        if job["sequence"] not in self.published:
            self.published.append(job["sequence"])

    def observe(self, job):
        n = self.polls[job["id"]] = self.polls.get(job["id"], 0) + 1
        thinking, answer = self.answers.get("default", ("because", "forty-two"))
        if n < 2:
            return {"thinking": thinking[:3], "answer": "", "output_tokens": 1, "status": "generating"}
        return {"thinking": thinking, "answer": answer, "output_tokens": 7, "status": "complete", "stop_cause": "eos",
                "decode_tps": 123.0, "prefill_seconds": 0.01}


def drain(queue, rounds=6):
    for _ in range(rounds):
        queue.step()


# ------------------------------------------------------------------------------------------ chat format
def test_chat_format_matches_the_published_layout():
    text = chat_template.render([{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"}])
    assert text == "[gMASK]<sop><|system|>Reasoning Effort: Max<|system|>Be brief.<|user|>Hi<|assistant|><think>"
    text = chat_template.render([{"role": "user", "content": "Hi"}], reasoning_effort="low")
    assert "Reasoning Effort: Low" in text
    tools = [{"type": "function", "function": {"name": "add", "parameters": {"type": "object"}}}]
    text = chat_template.render([{"role": "user", "content": "1+1"},
                                 {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "add", "arguments": {"a": 1, "b": "x"}}}]},
                                 {"role": "tool", "content": "2", "tool_call_id": "c1"}], tools=tools)
    assert "# Tools" in text and '{"name": "add", "parameters": {"type": "object"}}' in text
    assert "<tool_call>add<arg_key>a</arg_key><arg_value>1</arg_value><arg_key>b</arg_key><arg_value>x</arg_value></tool_call>" in text
    assert "<|observation|><tool_response>2</tool_response><|assistant|><think>" in text


def test_byte_tokenizer_round_trip():
    tok = ByteTokenizer(1024, (1020,))
    text = "[gMASK]<sop><|user|>héllo <think>x</think>"
    ids = tok.encode(text)
    assert tok.decode(ids) == text and max(ids) < 1024
    assert len(tok.encode("<|user|>")) == 1


# ------------------------------------------------------------------------------------------ openai shaping
def test_message_conversion_and_refusals():
    out = chat_utils.convert([{"role": "user", "content": [{"type": "text", "text": "a"}, {"type": "text", "text": "b"}]},
                              {"role": "assistant", "content": None, "tool_calls": [{"id": "c", "function": {"name": "f", "arguments": '{"x": 1}'}}]},
                              {"role": "tool", "tool_call_id": "c", "content": "ok"}])
    assert out[0]["content"] == "ab" and out[1]["tool_calls"][0]["function"]["arguments"] == {"x": 1}
    for bad in ([], [{"role": "robot", "content": "x"}], [{"role": "user", "content": [{"type": "image_url"}]}],
                [{"role": "tool", "content": "x"}], [{"role": "user", "content": "  "}],
                [{"role": "assistant", "tool_calls": [{"function": {"name": "f", "arguments": "[1]"}}]}]):
        with pytest.raises(ApiError):
            chat_utils.convert(bad)
    with pytest.raises(ApiError):
        chat_utils.check_tools([{"type": "retrieval"}])
    msgs = chat_utils.instruct([{"role": "user", "content": "x"}], "required", [{"function": {"name": "f"}}])
    assert msgs[0]["role"] == "system" and "must answer this turn by calling" in msgs[0]["content"]
    msgs = chat_utils.instruct([{"role": "system", "content": "S"}, {"role": "user", "content": "x"}], {"type": "function", "function": {"name": "f"}},
                               [{"function": {"name": "f"}}])
    assert msgs[0]["content"].startswith("S\n\n") and "named f" in msgs[0]["content"]


def test_tool_call_parsing():
    content, calls = tool_parser.parse('Sure.<tool_call>get_weather<arg_key>city</arg_key><arg_value>Paris</arg_value>'
                                       '<arg_key>days</arg_key><arg_value>3</arg_value></tool_call>')
    assert content == "Sure." and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris", "days": 3}
    assert tool_parser.parse("plain")[1] == []


def test_models_listing():
    data = OpenAIServingModels(capacity=32768, wait_seconds=1800).models()["data"]
    assert [m["id"] for m in data] == ["glm-5.3", "glm-5.3-low", "glm-5.3-high"]
    assert data[0]["context_window"] == 32768 and data[0]["max_input_tokens"] == 32767 and data[1]["reasoning_effort"] == "low"
    assert data[0]["supports"]["parallel_requests"] is False and data[0]["supports"]["sampling"] is False


def test_completion_and_stream(tmp_path):
    backend = FakeResident({"default": ("thinking hard", "Answer<tool_call>f<arg_key>a</arg_key><arg_value>1</arg_value></tool_call>")})
    queue = JobQueue(tmp_path / "state", backend)
    worker = threading.Thread(target=queue.work, daemon=True)
    worker.start()
    chat = OpenAIServingChat(queue, backend, capacity=4096, wait_seconds=20, poll_seconds=0.01)
    try:
        out = chat.completion({"model": "glm-5.3-high", "messages": [{"role": "user", "content": "hi"}], "temperature": 0.7})
        assert "Reasoning Effort: High" in backend.last_prompt  # the alias forces the effort
        msg = out["choices"][0]["message"]
        assert msg["content"] == "Answer" and msg["reasoning_content"] == "thinking hard"
        assert out["choices"][0]["finish_reason"] == "tool_calls" and msg["tool_calls"][0]["function"]["name"] == "f"
        assert out["usage"]["completion_tokens"] == 7
        chunks = [c for c in chat.stream({"messages": [{"role": "user", "content": "hi"}], "stream": True})]
        assert chunks[-1] == b"data: [DONE]\n\n"
        bodies = [json.loads(c[6:]) for c in chunks[:-1]]
        assert bodies[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}
        text = "".join(b["choices"][0]["delta"].get("content", "") for b in bodies)
        assert text == "Answer" and "<tool_call>" not in text  # held back once a tool call opens
        assert any("tool_calls" in b["choices"][0]["delta"] for b in bodies)
        assert bodies[-1]["choices"][0]["finish_reason"] == "tool_calls" and "usage" in bodies[-1]
    finally:
        queue.stopping.set()
        worker.join(2)
    for bad, status in (({"model": "gpt-4", "messages": [{"role": "user", "content": "x"}]}, 404), ({"n": 2, "messages": []}, 400),
                        ({"messages": [{"role": "user", "content": "x"}], "reasoning_effort": "extreme"}, 400),
                        ({"messages": [{"role": "user", "content": "x"}], "max_tokens": 0}, 400)):
        with pytest.raises(ApiError) as err:
            chat.prepare(bad)
        assert err.value.status == status


# ------------------------------------------------------------------------------------------ queue + conversations
def test_queue_is_sequential_bounded_and_idempotent(tmp_path):
    backend = FakeResident()
    queue = JobQueue(tmp_path / "state", backend)
    payload = backend.prepare_api([{"role": "user", "content": "x"}], "k", tools=None, effort="max", max_new_tokens=5, context_capacity=4096)
    first = queue.submit(payload, "k1", label="api")
    assert queue.submit(payload, "k1", label="api") is first  # duplicate suppression
    for i in range(2, PENDING + 1):
        queue.submit(payload, f"k{i}", label="api")
    with pytest.raises(ApiError) as err:
        queue.submit(payload, "overflow", label="api")
    assert err.value.status == 429
    drain(queue, 3)
    assert queue.job("k1")["status"] == "complete" and queue.job("k2")["status"] in ("queued", "generating")
    assert backend.published[0] == 1
    reloaded = JobQueue(tmp_path / "state", backend)  # persisted document survives a restart
    assert reloaded.job("k1")["status"] == "complete" and "payload" not in reloaded.job("k1")


def test_uncertain_failure_stops_the_queue_and_keeps_identity(tmp_path):
    backend = FakeResident()
    queue = JobQueue(tmp_path / "state", backend)
    payload = backend.prepare([{"role": "user", "content": "x"}], "a" * 32)
    queue.submit(payload, "j1", label="api")
    backend.fail_publish = True
    queue.step()
    assert queue.error and queue.db["jobs"][0]["sequence"] == 1 and (tmp_path / "state" / "error.json").exists()
    backend.fail_publish = False
    queue.step()  # stays stopped: never resubmits under a fresh sequence
    assert backend.sequence == 1 and queue.db["jobs"][0]["status"] == "queued"
    with pytest.raises(ApiError) as err:
        queue.submit(payload, "j2", label="api")
    assert err.value.status == 503


def test_conversations(tmp_path):
    backend = FakeResident()
    queue = JobQueue(tmp_path / "state", backend)
    store = ConversationStore(queue)
    chat_id = store.change({"action": "create"})["id"]
    key = "ab" * 16
    assert store.change({"action": "send", "chat": chat_id, "id": key, "text": "What is 6 x 7?"}) == {"ok": True}
    assert store.change({"action": "send", "chat": chat_id, "id": key, "text": "What is 6 x 7?"}) == {"id": key}  # idempotent
    with pytest.raises(ValueError):
        store.change({"action": "send", "chat": chat_id, "id": key, "text": "other text"})
    with pytest.raises(ValueError):
        store.change({"action": "send", "chat": chat_id, "id": "cd" * 16, "text": "second turn too early"})
    with pytest.raises(ValueError):
        store.change({"action": "delete", "chat": chat_id})
    drain(queue, 3)
    snap = store.snapshot()
    assert snap["chats"][0]["title"] == "What is 6 x 7?" and snap["chats"][0]["messages"][1]["content"] == "forty-two"
    assert snap["jobs"][0]["status"] == "complete" and "payload" not in snap["jobs"][0] and snap["capacity"] == 4096
    store.change({"action": "rename", "chat": chat_id, "title": "  Maths "})
    assert store.snapshot()["chats"][0]["title"] == "Maths"
    backend.available = False
    assert "unavailable" in store.snapshot()["error"]
    store.change({"action": "delete", "chat": chat_id})
    assert store.snapshot()["chats"] == []
    for bad in ({"action": "send", "chat": "nope"}, {"action": "explode", "chat": chat_id}):
        with pytest.raises(ValueError):
            store.change(bad)


# ------------------------------------------------------------------------------------------ HTTP
@pytest.fixture
def http(tmp_path):
    backend = FakeResident()
    queue = JobQueue(tmp_path / "state", backend)
    store = ConversationStore(queue)
    token = api_token(tmp_path / "state" / "api-key")
    chat = OpenAIServingChat(queue, backend, capacity=4096, wait_seconds=20, poll_seconds=0.01)
    server = ThreadingHTTPServer(("127.0.0.1", 0), handler(store, chat, OpenAIServingModels(capacity=4096, wait_seconds=20), token))
    threads = [threading.Thread(target=server.serve_forever, daemon=True), threading.Thread(target=queue.work, daemon=True)]
    for t in threads:
        t.start()
    yield server.server_port, token, tmp_path
    queue.stopping.set()
    server.shutdown()
    server.server_close()


def call(port, path, *, method="GET", body=None, headers=None):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", method=method, data=None if body is None else json.dumps(body).encode(),
                                 headers=headers or {})
    try:
        with urllib.request.urlopen(req, timeout=30) as res:
            return res.status, res.read(), dict(res.headers)
    except urllib.error.HTTPError as err:
        return err.code, err.read(), dict(err.headers)


def test_http_boundaries(http):
    port, token, tmp_path = http
    status, body, headers = call(port, "/")
    assert status == 200 and b"<title>" in body and "frame-ancestors 'none'" in headers["Content-Security-Policy"]
    assert call(port, "/app.js")[0] == 200 and call(port, "/style.css")[0] == 200 and call(port, "/secret")[0] == 404
    assert call(port, "/", headers={"Host": "evil.example:80"})[0] == 403  # DNS rebinding
    assert call(port, "/api/state", headers={"Origin": "http://evil.example"})[0] == 403  # cross-site
    assert json.loads(call(port, "/api/state")[1])["scheduling"] == "sequential"
    assert call(port, "/api/chat", method="POST", body={"action": "create"})[0] == 403  # missing X-GLM-UI
    status, body, _ = call(port, "/api/chat", method="POST", body={"action": "create"}, headers={"X-GLM-UI": "1", "Content-Type": "application/json"})
    assert status == 200 and "id" in json.loads(body)
    assert call(port, "/api/chat", method="POST", body={"action": "nope", "chat": "x"}, headers={"X-GLM-UI": "1"})[0] == 400
    assert call(port, "/v1/models")[0] == 401
    assert call(port, "/v1/models", headers={"Authorization": "Bearer wrong"})[0] == 401
    auth = {"Authorization": "Bearer " + token}
    assert json.loads(call(port, "/v1/models", headers=auth)[1])["data"][0]["id"] == "glm-5.3"
    assert call(port, "/v1/files", headers=auth)[0] == 404
    status, body, _ = call(port, "/v1/chat/completions", method="POST", headers=auth, body={"messages": [{"role": "user", "content": "hi"}]})
    assert status == 200 and json.loads(body)["choices"][0]["message"]["content"] == "forty-two"
    status, body, _ = call(port, "/v1/chat/completions", method="POST", headers=auth, body={"model": "nope", "messages": [{"role": "user", "content": "x"}]})
    assert status == 404 and json.loads(body)["error"]["type"] == "model_not_found"
    status, body, headers = call(port, "/v1/chat/completions", method="POST", headers=auth,
                                 body={"stream": True, "messages": [{"role": "user", "content": "hi"}]})
    assert status == 200 and headers["Content-Type"].startswith("text/event-stream") and body.endswith(b"data: [DONE]\n\n")
    assert (tmp_path / "state" / "api-key").stat().st_mode & 0o077 == 0
