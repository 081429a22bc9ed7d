"""``POST /v1/chat/completions`` in front of the sequential resident queue.

The endpoint is stateless: a request is read into a ``ChatCall`` (every field validated, refusals are ``ApiError``), handed to the queue
under a fresh key, and then *followed*: ``_follow`` yields the job's snapshots until it reaches a terminal state or the server's deadline
passes.  ``completion`` keeps the last snapshot; ``stream`` turns the growth between snapshots into server-sent events.

Accepted fields: ``model`` (``glm-5.3``, or an alias that fixes the reasoning effort), ``messages``, ``tools``, ``tool_choice`` (stated
in-band, see ``chat_utils.instruct``), ``max_tokens``, ``stream``, ``reasoning_effort`` (low / high / max), ``n`` (1 only).  Sampling
parameters are ignored: decoding is greedy.  Replies keep ``reasoning_content`` apart from ``content``; ``finish_reason`` is ``stop``,
``tool_calls`` or ``length``.  A stream sends the role, reasoning deltas, content deltas (held back from the moment a ``<tool_call>``
opens, because that text is not content), the tool calls, a finish event with ``usage``, then ``[DONE]``.  Status codes: 400 bad request,
404 unknown model, 429 queue full (raised by the queue), 503 queue stopped, 504 server deadline.

Behaviour parity: reference ``glm_tpu/entrypoints/openai/serving_chat.py`` (same fields, event order and status codes).
"""

from __future__ import annotations

import json
import time
import uuid
from dataclasses import dataclass

from glm_tpu_b200.entrypoints.openai.chat_utils import check_tools, convert, instruct
from glm_tpu_b200.entrypoints.openai.protocol import ALIASES, EFFORTS, MODEL_NAME, ApiError
from glm_tpu_b200.entrypoints.openai.tool_parser import OPEN, parse
from glm_tpu_b200.entrypoints.serve.job_queue import DONE

LENGTH_CAUSES = ("context_exhausted", "output_cap")
DEADLINE_SENTENCE = "the resident model did not finish within the server deadline"


@dataclass(frozen=True)
class ChatCall:
    """A validated request."""

    model: str
    effort: str
    budget: int | None
    messages: list
    tools: list | None

    @classmethod
    def read(cls, body) -> "ChatCall":
        if not isinstance(body, dict):
            raise ApiError("expected a JSON object")
        model = body.get("model") or MODEL_NAME
        if model not in ALIASES:
            raise ApiError(f"unknown model: {model}", status=404, kind="model_not_found")
        if body.get("n", 1) not in (None, 1):
            raise ApiError("only one choice per request is supported")
        asked = body.get("reasoning_effort", "max")
        if asked not in EFFORTS:
            raise ApiError("reasoning_effort must be low, high or max")
        budget = body.get("max_tokens")
        if budget is not None and (type(budget) is not int or budget < 1):
            raise ApiError("max_tokens must be a positive integer")
        tools = check_tools(body.get("tools"))
        messages = instruct(convert(body.get("messages")), body.get("tool_choice"), tools)
        # an alias outranks the field: some clients can choose a model name but cannot send extra fields
        return cls(model, ALIASES[model] or asked, budget, messages, tools)


def _content_so_far(answer: str) -> str:
    """What of a still-growing answer may already be sent as content: everything before an opening tool-call tag, and not the
    tail that may be the beginning of one (``...<tool_c``), which is decided only when more text has arrived."""
    head, opened, _ = answer.partition(OPEN)
    if not opened:
        for n in range(len(OPEN) - 1, 0, -1):
            if head.endswith(OPEN[:n]):
                return head[:-n]
    return head


def _why_it_ended(job: dict, calls: list) -> str:
    if calls:
        return "tool_calls"
    cut_short = job["status"] != "complete" and job.get("stop_cause") in LENGTH_CAUSES
    return "length" if cut_short else "stop"


def _token_counts(job: dict) -> dict:
    asked, produced = job["prompt_tokens"], job["output_tokens"]
    return {"prompt_tokens": asked, "completion_tokens": produced, "total_tokens": asked + produced}


class OpenAIServingChat:
    def __init__(self, queue, backend, *, capacity: int, wait_seconds: float = 1800, poll_seconds: float = 0.2):
        self.queue, self.backend, self.capacity = queue, backend, capacity
        self.wait_seconds, self.poll_seconds = wait_seconds, poll_seconds

    # ------------------------------------------------------------------------------------------------------------------ admission
    def prepare(self, body):
        """``(prepared request, key, model name)``; raises ``ApiError`` for anything the endpoint does not take."""
        call = ChatCall.read(body)
        key = uuid.uuid4().hex
        prepared = self.backend.prepare_api(call.messages, key, tools=call.tools, effort=call.effort, max_new_tokens=call.budget,
                                            context_capacity=self.capacity)
        return prepared, key, call.model

    def _admit(self, body):
        prepared, key, model = self.prepare(body)
        self.queue.submit(prepared, key, label="api")
        return key, model

    # ------------------------------------------------------------------------------------------------------------------ following a job
    def _snapshot(self, key: str) -> dict:
        job = self.queue.job(key)
        if job is None:
            raise ApiError("request was not retained", status=500, kind="server_error")
        if job.get("error"):
            raise ApiError(job["error"], status=503, kind="server_error")
        return job

    def _follow(self, key: str, hint: str = ""):
        """Yield snapshots of the job; the last one is terminal.  Raises 504 once the server's deadline has passed."""
        give_up = time.time() + self.wait_seconds
        while True:
            job = self._snapshot(key)
            yield job
            if job["status"] in DONE:
                return
            if time.time() > give_up:
                raise ApiError(DEADLINE_SENTENCE + hint, status=504, kind="timeout")
            time.sleep(self.poll_seconds)

    # ------------------------------------------------------------------------------------------------------------------ one reply
    def completion(self, body) -> dict:
        key, model = self._admit(body)
        job = None
        for job in self._follow(key, hint="; use stream=true for long answers"):
            pass
        content, calls = parse(job["answer"])
        reply = {"role": "assistant", "content": content or None}
        if job["thinking"]:
            reply["reasoning_content"] = job["thinking"]
        if calls:
            reply["tool_calls"] = [{k: c[k] for k in ("id", "type", "function")} for c in calls]
        choice = {"index": 0, "message": reply, "logprobs": None, "finish_reason": _why_it_ended(job, calls)}
        return {"id": "chatcmpl-" + key, "object": "chat.completion", "created": int(job["created"]), "model": model, "choices": [choice],
                "usage": _token_counts(job)}

    # ------------------------------------------------------------------------------------------------------------------ a stream
    def stream(self, body):
        """Server-sent events (bytes)."""
        key, model = self._admit(body)
        ident = {"id": "chatcmpl-" + key, "object": "chat.completion.chunk", "model": model, "created": int(time.time())}
        yield self.chunk(ident, {"role": "assistant", "content": ""}, None)
        told = {"reasoning_content": 0, "content": 0}  # characters already sent, per channel
        job = None
        for job in self._follow(key):
            running = job["status"] not in DONE
            # while the job runs, text after an opening tool-call tag is withheld: it will become a tool call, not content;
            # the final snapshot's content is sent below, after the calls have been parsed out of it
            grown = {"reasoning_content": job["thinking"], "content": _content_so_far(job["answer"]) if running else None}
            for channel, text in grown.items():
                if text is not None and len(text) > told[channel]:
                    yield self.chunk(ident, {channel: text[told[channel]:]}, None)
                    told[channel] = len(text)
        content, calls = parse(job["answer"])
        if len(content) > told["content"]:
            yield self.chunk(ident, {"content": content[told["content"]:]}, None)
        for call in calls:
            entry = {"index": call["index"], "id": call["id"], "type": "function", "function": dict(call["function"])}
            yield self.chunk(ident, {"tool_calls": [entry]}, None)
        yield self.chunk(ident, {}, _why_it_ended(job, calls), extra={"usage": _token_counts(job)})
        yield b"data: [DONE]\n\n"

    @staticmethod
    def chunk(ident: dict, delta: dict, finish, *, extra=None) -> bytes:
        """One event: the identifying fields, a single choice with ``delta`` and ``finish_reason``, then ``extra`` (usage)."""
        event = {**ident, "choices": [{"index": 0, "delta": delta, "logprobs": None, "finish_reason": finish}], **(extra or {})}
        return b"data: " + json.dumps(event, ensure_ascii=False).encode() + b"\n\n"
