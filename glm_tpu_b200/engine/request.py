"""Prepared requests: the canonical JSON a front end hands to the engine, and its validation.

A *prepared request* binds a prompt (token ids), an output budget and the serving profile it was prepared for
(context capacity, vocabulary, EOS ids, tokenizer/template pins, model identity) into one self-hashed object:
``request_sha256`` is the SHA-256 of the canonical wire bytes of all other fields.  The engine re-derives the object
from its own inputs and refuses anything that does not match byte for byte, so a request can never be truncated,
re-budgeted or replayed against another profile silently.  Batches bind several requests (sequential queue of up to
10, or up to ``CONCURRENT_LIMIT`` concurrent chats at the 32K profile) the same way.

A ``RequestProfile`` carries the constants.  ``GLM53_PROFILE`` is the production one; fixtures derive theirs from a
``ModelGeometry``.

Parity: reference ``glm_tpu/engine/request.py:17-243`` (schema names, capacities, limits, stop causes).
"""

from __future__ import annotations

import hashlib
import json
import struct
from dataclasses import dataclass, field
from typing import Any, Iterable

from glm_tpu_b200.config import model as model_config
from glm_tpu_b200.exceptions import RequestValidationError
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

SCHEMA = "glm_b200_request_v1"
BATCH_SCHEMA = "glm_b200_batch_v1"
CONCURRENT_SCHEMA = "glm_b200_concurrent_batch_v1"

CAPACITY = 8192
CONCURRENT_CAPACITY = 32768
LONG_CAPACITY = 166912
AGENT_CAPACITY = 262144
CAPACITIES = (CAPACITY, CONCURRENT_CAPACITY, LONG_CAPACITY, AGENT_CAPACITY)
CONTEXT_ALIASES = {"8k": CAPACITY, "32k": CONCURRENT_CAPACITY, "128k": LONG_CAPACITY, "256k": AGENT_CAPACITY}
MAX_PROMPT = 131072
PROMPT_LIMITS = {CAPACITY: CAPACITY, CONCURRENT_CAPACITY: CONCURRENT_CAPACITY, LONG_CAPACITY: MAX_PROMPT, AGENT_CAPACITY: AGENT_CAPACITY}
CONCURRENT_LIMIT = 4
QUEUE_LIMIT = 10
MAX_NEW = 163840
PAYLOAD_CAP = 16 << 20
MESSAGES_CAP = 1 << 20


@dataclass(frozen=True)
class RequestProfile:
    vocab_size: int
    eos_ids: tuple[int, ...]
    capacities: tuple[int, ...] = CAPACITIES
    prompt_limits: dict = field(default_factory=lambda: dict(PROMPT_LIMITS))
    concurrent_capacity: int = CONCURRENT_CAPACITY
    concurrent_limit: int = CONCURRENT_LIMIT
    max_new: int = MAX_NEW
    model_id: str = model_config.MODEL_ID
    model_revision: str = model_config.MODEL_REVISION
    tokenizer_files: tuple = ()
    chat_template_sha256: str = ""

    @classmethod
    def for_geometry(cls, geometry, capacities: Iterable[int], concurrent_capacity: int | None = None, **kw) -> "RequestProfile":
        caps = tuple(capacities)
        return cls(vocab_size=geometry.vocab_size, eos_ids=tuple(geometry.eos_ids), capacities=caps,
                   prompt_limits={c: c for c in caps}, concurrent_capacity=concurrent_capacity or caps[-1], **kw)


GLM53_PROFILE = RequestProfile(vocab_size=154880, eos_ids=model_config.EOS_IDS)


def prompt_digest(ids: list[int]) -> str:
    """SHA-256 of the ids as little-endian int32."""
    return hashlib.sha256(struct.pack(f"<{len(ids)}i", *ids)).hexdigest()


def _check_ids(ids: Any, profile: RequestProfile) -> list[int]:
    if type(ids) is not list or not ids:
        raise RequestValidationError("prompt_ids must be a non-empty list")
    for t in ids:
        if type(t) is not int or not 0 <= t < profile.vocab_size:
            raise RequestValidationError("prompt_ids must be integers inside the vocabulary")
    return ids


def from_token_ids(ids, *, request_id: str, max_new_tokens: int, context_capacity: int = CAPACITY,
                   profile: RequestProfile = GLM53_PROFILE) -> dict:
    if type(context_capacity) is not int or context_capacity not in profile.capacities:
        raise RequestValidationError("unsupported context capacity")
    if type(request_id) is not str or not request_id or len(request_id) > 128 or not request_id.isprintable():
        raise RequestValidationError("request_id must be a short printable string")
    if type(max_new_tokens) is not int or not 1 <= max_new_tokens <= profile.max_new:
        raise RequestValidationError("max_new_tokens is out of range")
    ids = _check_ids(ids, profile)
    if len(ids) > profile.prompt_limits[context_capacity] or len(ids) + max_new_tokens > context_capacity:
        raise RequestValidationError("prompt and complete output budget exceed the selected capacity")
    body = {
        "schema": SCHEMA,
        "request_id": request_id,
        "prompt_ids": ids,
        "prompt_ids_sha256": prompt_digest(ids),
        "max_new_tokens": max_new_tokens,
        "context_capacity": context_capacity,
        "vocab_size": profile.vocab_size,
        "eos_ids": list(profile.eos_ids),
        "decode_policy": "greedy",
        "thinking": "on/max",
        "tokenizer_files": dict(profile.tokenizer_files),
        "chat_template_sha256": profile.chat_template_sha256,
        "model_id": profile.model_id,
        "model_revision": profile.model_revision,
    }
    return dict(body, request_sha256=hashlib.sha256(canonical_wire_bytes(body)).hexdigest())


CHAT_ROLES = ("system", "user", "assistant")


def check_chat(messages: Any) -> list[dict]:
    """A complete text-only conversation that the model is to continue: a bounded, non-empty list of ``{"role", "content"}`` objects
    with string content, an optional system message in first place only, and a user message last."""
    problem = None
    if type(messages) is not list or not messages:
        problem = "a non-empty list of messages"
    elif len(canonical_wire_bytes(messages)) > MESSAGES_CAP:
        problem = f"at most {MESSAGES_CAP} bytes of messages"
    elif any(type(m) is not dict or set(m) != {"role", "content"} or m["role"] not in CHAT_ROLES or type(m["content"]) is not str for m in messages):
        problem = "messages with exactly a role (system, user or assistant) and text content"
    elif any(m["role"] == "system" for m in messages[1:]):
        problem = "a system message in first place only"
    elif messages[-1]["role"] != "user":
        problem = "a user message last"
    if problem:
        raise RequestValidationError("a chat to prepare needs " + problem)
    return messages


def from_messages(messages, *, tokenizer, request_id: str, max_new_tokens: int | None = None, context_capacity: int = CAPACITY,
                  profile: RequestProfile = GLM53_PROFILE, reasoning_effort: str = "max") -> dict:
    """The prepared request for a whole conversation, rendered with ``tokenizer`` (the session's: its chat format is the pinned
    one) at maximum reasoning effort unless told otherwise.  Nothing is truncated: a conversation that does not leave room for
    one new token in ``context_capacity`` is refused.  Without ``max_new_tokens`` the answer may use whatever the capacity
    leaves, up to the profile's ceiling.

    Parity: reference ``glm_tpu/engine/request.py:180-212``."""
    ids = tokenizer.apply_chat_template(check_chat(messages), reasoning_effort=reasoning_effort)
    if type(context_capacity) is int and context_capacity in profile.capacities and len(ids) >= context_capacity:
        raise RequestValidationError(f"the conversation has {len(ids)} tokens and fills the {context_capacity}-slot context; nothing is truncated")
    if max_new_tokens is None:
        max_new_tokens = default_max_new_tokens(len(ids), context_capacity, profile) if type(context_capacity) is int else 0
    return from_token_ids(ids, request_id=request_id, max_new_tokens=max_new_tokens, context_capacity=context_capacity, profile=profile)


def default_max_new_tokens(prompt_tokens: int, context_capacity: int, profile: RequestProfile = GLM53_PROFILE) -> int:
    """The input is never truncated; the default budget is whatever the capacity leaves, capped at ``max_new``."""
    return min(profile.max_new, context_capacity - prompt_tokens)


def validate(value: Any, profile: RequestProfile = GLM53_PROFILE) -> None:
    if type(value) is not dict:
        raise RequestValidationError("a prepared request must be an object")
    try:
        expected = from_token_ids(value["prompt_ids"], request_id=value["request_id"], max_new_tokens=value["max_new_tokens"],
                                  context_capacity=value["context_capacity"], profile=profile)
    except KeyError as exc:
        raise RequestValidationError("missing request fields") from exc
    if canonical_wire_bytes(value) != canonical_wire_bytes(expected):
        raise RequestValidationError("request identity or fixed profile differs")


def batch(values: Any, *, concurrent: bool = False, profile: RequestProfile = GLM53_PROFILE) -> dict:
    if type(concurrent) is not bool:
        raise RequestValidationError("concurrent must be boolean")
    limit = profile.concurrent_limit if concurrent else QUEUE_LIMIT
    if type(values) is not list or not 1 <= len(values) <= limit:
        raise RequestValidationError(f"submit between one and {limit} requests")
    for v in values:
        validate(v, profile)
    if len({v["request_id"] for v in values}) != len(values):
        raise RequestValidationError("request IDs must be unique")
    capacities = {v["context_capacity"] for v in values}
    if len(capacities) != 1:
        raise RequestValidationError("one loaded model serves one context capacity")
    capacity = capacities.pop()
    if concurrent and capacity != profile.concurrent_capacity:
        raise RequestValidationError("concurrent conversations use the concurrent capacity profile")
    body = {"schema": CONCURRENT_SCHEMA if concurrent else BATCH_SCHEMA, "requests": values, "context_capacity": capacity}
    return dict(body, request_sha256=hashlib.sha256(canonical_wire_bytes(body)).hexdigest())


def validate_payload(value: Any, profile: RequestProfile = GLM53_PROFILE) -> None:
    if type(value) is dict and value.get("schema") in (BATCH_SCHEMA, CONCURRENT_SCHEMA):
        expected = batch(value.get("requests"), concurrent=value["schema"] == CONCURRENT_SCHEMA, profile=profile)
        if canonical_wire_bytes(value) != canonical_wire_bytes(expected):
            raise RequestValidationError("batch identity differs")
    else:
        validate(value, profile)


def read(path, profile: RequestProfile = GLM53_PROFILE, *, expected_sha256: str | None = None) -> dict:
    """A prepared request (or batch) from a file: a bounded regular file reached without links, the digest of its bytes when the
    caller pins one, then the full validation of its content against ``profile``.

    Parity: reference ``glm_tpu/engine/request.py:137-143``."""
    from pathlib import Path

    from glm_tpu_b200.utils.io_utils import read_bounded

    try:
        raw = read_bounded(Path(path), PAYLOAD_CAP)
    except (OSError, ValueError) as exc:
        raise RequestValidationError(f"the request file cannot be read: {exc}") from exc
    if expected_sha256 is not None and hashlib.sha256(raw).hexdigest() != expected_sha256:
        raise RequestValidationError("the request file is not the pinned one (digest differs)")
    try:
        value = json.loads(raw)
    except ValueError as exc:
        raise RequestValidationError("the request file is not JSON") from exc
    validate_payload(value, profile)
    return value


def requests_of(value: dict, profile: RequestProfile = GLM53_PROFILE) -> list[dict]:
    validate_payload(value, profile)
    return value["requests"] if value.get("schema") in (BATCH_SCHEMA, CONCURRENT_SCHEMA) else [value]


def is_concurrent(value: dict) -> bool:
    return value.get("schema") == CONCURRENT_SCHEMA


def stop_cause(value: dict, finish_reason: str) -> str:
    if finish_reason == "eos":
        return "eos"
    if finish_reason == "length":
        full = len(value["prompt_ids"]) + value["max_new_tokens"] == value["context_capacity"]
        return "context_exhausted" if full else "output_cap"
    raise RequestValidationError("request did not reach a terminal token condition")
