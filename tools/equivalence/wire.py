"""G9: wire formats.  Every byte string another process, a file reader or a browser parses is produced here from fixed
inputs and hashed: prepared requests (single, batch, concurrent), TokenEvent lines, resident commands and file names, worker
command lines, OpenAI chunks (SSE), tool-call parsing, the chat template rendering, canonical JSON itself.
"""

from __future__ import annotations

import hashlib
import json


def _sha(raw: bytes) -> str:
    return hashlib.sha256(raw).hexdigest()


def collect() -> dict:
    from glm_tpu_b200.engine import request as rq
    from glm_tpu_b200.engine import resident_protocol as proto
    from glm_tpu_b200.engine.outputs import TokenEvent, final_channel
    from glm_tpu_b200.entrypoints.openai import tool_parser
    from glm_tpu_b200.entrypoints.openai.serving_chat import OpenAIServingChat
    from glm_tpu_b200.tokenizer import ByteTokenizer, chat_template
    from glm_tpu_b200.utils.json_utils import canonical_hash_bytes, canonical_wire_bytes
    from tools.equivalence.fixture import fixture_geometry

    g = fixture_geometry()
    profile = rq.RequestProfile.for_geometry(g, (96,), concurrent_capacity=96)
    out: dict = {}
    sample = {"b": [1, 2.5, None, True], "a": "é\n\"q\"", "nested": {"z": 0, "y": [[]]}}
    out["canonical_wire_bytes"] = _sha(canonical_wire_bytes(sample))
    out["canonical_hash_bytes"] = _sha(canonical_hash_bytes(sample))
    one = rq.from_token_ids([1, 2, 3, 4], request_id="request-01", max_new_tokens=5, context_capacity=96, profile=profile)
    two = rq.from_token_ids([9, 8, 7], request_id="request-02", max_new_tokens=3, context_capacity=96, profile=profile)
    out["prepared_request"] = _sha(canonical_wire_bytes(one))
    out["prepared_request_keys"] = sorted(one)
    out["batch_sequential"] = _sha(canonical_wire_bytes(rq.batch([one, two], profile=profile)))
    out["batch_concurrent"] = _sha(canonical_wire_bytes(rq.batch([one, two], concurrent=True, profile=profile)))
    events = [TokenEvent("request-01", 0, 65, None), TokenEvent("request-01", 1, 253, "stop"), TokenEvent("request-02", 0, 7, "length", batch_round=3)]
    out["token_event_lines"] = _sha(b"".join(canonical_wire_bytes(e.wire()) + b"\n" for e in events))
    out["resident_command"] = _sha(proto.encode_command(3, one))
    out["resident_names"] = [proto.inbox_name(7), proto.runner_file(2), proto.worker_started_file(5), str(proto.result_dir("/r", 0)),
                             str(proto.result_dir("/r", 12)), proto.TOKENS_FILE, proto.ANSWER_FILE, proto.SUMMARY_FILE, proto.STDOUT_RUN,
                             proto.STDOUT_RESIDENT_RESULT, proto.WORKER_MODULE, proto.WORKER_ENV_FLAG]
    out["final_channel"] = list(final_channel("<think>plan</think>The answer is 4.<|user|>ignored"))
    messages = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "2+2?"},
                {"role": "assistant", "content": "4", "reasoning_content": "add"}, {"role": "user", "content": "and 3+3?"}]
    tools = [{"type": "function", "function": {"name": "calc", "description": "adds", "parameters": {"type": "object", "properties": {"x": {"type": "number"}}}}}]
    out["chat_template_plain"] = _sha(chat_template.render(messages, reasoning_effort="max").encode())
    out["chat_template_tools"] = _sha(chat_template.render(messages, tools=tools, reasoning_effort="high").encode())
    round_trip = [{"role": "user", "content": [{"type": "text", "text": "look: "}, {"type": "image_url", "image_url": {"url": "x"}}, {"type": "text", "text": "Köln?"}]},
                  {"role": "assistant", "content": "", "reasoning_content": "need it",
                   "tool_calls": [{"type": "function", "function": {"name": "calc", "arguments": {"x": 2.5, "label": "größe", "deep": {"a": [1, None]}}}}]},
                  {"role": "tool", "content": [{"type": "text", "text": "7"}, {"type": "text", "text": " degrees"}]}, {"role": "tool", "content": "second"},
                  {"role": "assistant", "content": " It is 7. \n"}, {"role": "user", "content": "thanks"}]
    out["chat_template_parts_and_tool_round"] = _sha(chat_template.render(round_trip, tools=tools, reasoning_effort="low").encode())
    out["chat_template_cleared_reasoning"] = _sha(chat_template.render(round_trip, clear_thinking=True, add_generation_prompt=False).encode())
    tok = ByteTokenizer(g.vocab_size + 1024, g.eos_ids)
    out["chat_template_token_ids"] = _sha(json.dumps(tok.apply_chat_template(messages[:2], reasoning_effort="max")).encode())
    text, calls = tool_parser.parse("I will call it.<tool_call>calc<arg_key>x</arg_key><arg_value>3</arg_value></tool_call>")
    out["tool_call_parse"] = [text, [{k: v for k, v in call.items() if k != "id"} for call in calls]]  # the id is random by design
    out["tool_call_id_shape"] = [len(calls[0]["id"]), calls[0]["id"][:5]]
    ident = {"id": "chatcmpl-0001", "created": 1700000000, "model": "glm-5.3"}
    out["sse_chunks"] = _sha(OpenAIServingChat.chunk(ident, {"role": "assistant"}, None) + OpenAIServingChat.chunk(ident, {"content": "4"}, None)
                             + OpenAIServingChat.chunk(ident, {}, "stop", extra={"usage": {"prompt_tokens": 4, "completion_tokens": 1, "total_tokens": 5}}))
    return out
