"""``POST /v1/chat/completions``: stateless request shaping in front of the sequential resident queue.

Supported fields: ``model`` (``glm-5.3`` or an alias that forces the reasoning effort), ``messages``, ``tools``,
``tool_choice`` (rendered as an in-band system instruction), ``max_tokens``, ``stream``, ``reasoning_effort``
(low / high / max), ``n`` (must be 1).  Sampling parameters are accepted and ignored: decoding is greedy.  The answer
separates ``reasoning_content`` from ``content``; ``finish_reason`` is ``stop``, ``tool_calls`` or ``length``; streaming
sends SSE chunks (role, reasoning deltas, content deltas -- held back once a ``<tool_call>`` opens -- tool calls, the
finish chunk with ``usage``) and ``[DONE]``.  Errors: 400 invalid request, 404 unknown model, 429 ten jobs waiting,
503 queue stopped, 504 server deadline.

Parity: reference ``glm_tpu/entrypoints/openai/serving_chat.py:18-163``.
"""

from __future__ import annotations

import json
import time
import uuid

from glm_tpu_b200.entrypoints.openai.chat_utils import check_tools, convert, instruct
from glm_tpu_b200.entrypoints.openai.protocol import ALIASES, EFFORTS, MODEL_NAME, ApiError
from glm_tpu_b200.entrypoints.openai.tool_parser import OPEN, parse
from glm_tpu_b200.entrypoints.serve.job_queue import DONE


def finish_reason(job: dict, calls: list) -> str:
    if calls:
        return "tool_calls"
    if job["status"] == "complete":
        return "stop"
    return "length" if job.get("stop_cause") in ("context_exhausted", "output_cap") else "stop"


def usage(job: dict) -> dict:
    return {"prompt_tokens": job["prompt_tokens"], "completion_tokens": job["output_tokens"],
            "total_tokens": job["prompt_tokens"] + job["output_tokens"]}


class OpenAIServingChat:
    def __init__(self, queue, backend, *, capacity: int, wait_seconds: float = 1800, poll_seconds: float = 0.2):
        self.queue, self.backend = queue, backend
        self.capacity, self.wait_seconds, self.poll_seconds = capacity, wait_seconds, poll_seconds

    def prepare(self, data):
        if type(data) is not dict:
            raise ApiError("expected a JSON object")
        name = data.get("model") or MODEL_NAME
        if name not in ALIASES:
            raise ApiError("unknown model: " + str(name), status=404, kind="model_not_found")
        if data.get("n") not in (None, 1):
            raise ApiError("only one choice per request is supported")
        effort = data.get("reasoning_effort", "max")
        if effort not in EFFORTS:
            raise ApiError("reasoning_effort must be low, high or max")
        effort = ALIASES[name] or effort  # the alias wins, for clients that cannot send the field
        budget = data.get("max_tokens")
        if budget is not None and (type(budget) is not int or budget <= 0):
            raise ApiError("max_tokens must be a positive integer")
        tools = check_tools(data.get("tools"))
        messages = instruct(convert(data.get("messages")), data.get("tool_choice"), tools)
        key = uuid.uuid4().hex
        payload = self.backend.prepare_api(messages, key, tools=tools, effort=effort, max_new_tokens=budget,
                                           context_capacity=self.capacity)
        return payload, key, name

    def _job(self, key: str) -> dict:
        job = self.queue.job(key)
        if job is None:
            raise ApiError("request was not retained", status=500, kind="server_error")
        if job.get("error"):
            raise ApiError(job["error"], status=503, kind="server_error")
        return job

    def wait(self, key: str, *, deadline: float) -> dict:
        while True:
            job = self._job(key)
            if job["status"] in DONE:
                return job
            if time.time() > deadline:
                raise ApiError("the resident model did not finish within the server deadline; use stream=true for long answers",
                               status=504, kind="timeout")
            time.sleep(self.poll_seconds)

    def completion(self, data) -> dict:
        payload, key, name = self.prepare(data)
        self.queue.submit(payload, key, label="api")
        job = self.wait(key, deadline=time.time() + self.wait_seconds)
        content, calls = parse(job["answer"])
        message = {"role": "assistant", "content": content or None}
        if job["thinking"]:
            message["reasoning_content"] = job["thinking"]
        if calls:
            message["tool_calls"] = [{"id": c["id"], "type": "function", "function": c["function"]} for c in calls]
        return {"id": "chatcmpl-" + key, "object": "chat.completion", "created": int(job["created"]), "model": name,
                "choices": [{"index": 0, "message": message, "logprobs": None, "finish_reason": finish_reason(job, calls)}],
                "usage": usage(job)}

    def stream(self, data):
        """Yield SSE chunks (bytes).  Tool calls are emitted once the final channel is known."""
        payload, key, name = self.prepare(data)
        self.queue.submit(payload, key, label="api")
        ident = {"id": "chatcmpl-" + key, "object": "chat.completion.chunk", "model": name, "created": int(time.time())}
        yield self.chunk(ident, {"role": "assistant", "content": ""}, None)
        deadline = time.time() + self.wait_seconds
        sent_thinking = sent_answer = 0
        while True:
            job = self._job(key)
            terminal = job["status"] in DONE
            thinking, answer = job["thinking"], job["answer"]
            if len(thinking) > sent_thinking:
                yield self.chunk(ident, {"reasoning_content": thinking[sent_thinking:]}, None)
                sent_thinking = len(thinking)
            visible = answer if terminal else answer.split(OPEN, 1)[0]  # hold text back while a tool call may be forming
            if not terminal and len(visible) > sent_answer:
                yield self.chunk(ident, {"content": visible[sent_answer:]}, None)
                sent_answer = len(visible)
            if terminal:
                break
            if time.time() > deadline:
                raise ApiError("the resident model did not finish within the server deadline", status=504, kind="timeout")
            time.sleep(self.poll_seconds)
        content, calls = parse(job["answer"])
        if len(content) > sent_answer:
            yield self.chunk(ident, {"content": content[sent_answer:]}, None)
        for call in calls:
            yield self.chunk(ident, {"tool_calls": [{"index": call["index"], "id": call["id"], "type": "function",
                                                     "function": dict(call["function"])}]}, None)
        yield self.chunk(ident, {}, finish_reason(job, calls), extra={"usage": usage(job)})
        yield b"data: [DONE]\n\n"

    @staticmethod
    def chunk(ident: dict, delta: dict, finish, *, extra=None) -> bytes:
        body = dict(ident, choices=[{"index": 0, "delta": delta, "logprobs": None, "finish_reason": finish}])
        if extra:
            body.update(extra)
        return b"data: " + json.dumps(body, ensure_ascii=False).encode() + b"\n\n"
