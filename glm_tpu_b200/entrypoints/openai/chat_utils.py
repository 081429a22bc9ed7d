"""From an OpenAI chat request to the messages the GLM chat format renders.

Three entry points, used in this order by ``serving_chat``:

* ``check_tools(tools)``: only function tools, each with a name and (optionally) a JSON-schema object;
* ``convert(messages)``: one converter per role (``_CONVERTERS``) turns a validated OpenAI message into the template's message; content may
  be a string or a list of text parts, assistant turns may carry ``reasoning_content`` and ``tool_calls`` whose arguments arrive as a
  JSON string and leave as a mapping, tool turns must name the call they answer;
* ``instruct(messages, tool_choice, tools)``: the chat format has no ``tool_choice`` field, so a constraint is stated in-band, appended
  to the system turn (or put in a new one).

Every refusal is an ``ApiError`` with the sentence the client reads.  Behaviour parity: reference
``glm_tpu/entrypoints/openai/chat_utils.py`` (same accepted shapes, same refusal sentences).
"""

from __future__ import annotations

import json

from glm_tpu_b200.entrypoints.openai.protocol import MESSAGES_CAP, TOOLS_CAP, ApiError

CHOICE_NOTES = {
    "none": "Do not call any function for this turn. Answer directly in plain text.",
    "required": "You must answer this turn by calling one of the provided functions.",
}
NAMED_CHOICE_NOTE = "You must answer this turn by calling the function named {name}."


def _require(ok: bool, sentence: str) -> None:
    if not ok:
        raise ApiError(sentence)


def _is(value, kind) -> bool:
    return type(value) is kind  # exact types: a bool is not an int, a subclass is not the JSON type


def _wire_size(value) -> int:
    return len(json.dumps(value).encode())


# ------------------------------------------------------------------------------------------------------------------ content and arguments
def _flatten(content) -> str:
    """OpenAI content (null, a string, or text parts) as one string."""
    if content is None or _is(content, str):
        return content or ""
    _require(_is(content, list), "message content must be a string or a list of text parts")
    pieces = []
    for part in content:
        _require(_is(part, dict) and part.get("type") == "text" and _is(part.get("text"), str), "only text content parts are supported")
        pieces.append(part["text"])
    return "".join(pieces)


def _argument_mapping(raw) -> dict:
    """Tool-call arguments as the mapping the chat format wants (OpenAI sends a JSON string)."""
    if _is(raw, dict):
        return raw
    _require(_is(raw, str), "tool call arguments must be a JSON object string")
    if raw.strip() == "":
        return {}
    try:
        decoded = json.loads(raw)
    except ValueError as exc:
        raise ApiError("tool call arguments are not valid JSON") from exc
    _require(_is(decoded, dict), "tool call arguments must decode to an object")
    return decoded


def _tool_call(call) -> dict:
    function = call.get("function") if _is(call, dict) else None
    _require(_is(function, dict) and _is(function.get("name"), str), "each tool call needs function.name")
    return {"id": call.get("id") or "", "type": "function",
            "function": {"name": function["name"], "arguments": _argument_mapping(function.get("arguments", "{}"))}}


# ------------------------------------------------------------------------------------------------------------------ one converter per role
def _spoken(message: dict, text: str) -> dict:
    """system and user turns: they must say something."""
    _require(text.strip() != "", message["role"] + " messages need text content")
    return {"role": message["role"], "content": text}


def _assistant(message: dict, text: str) -> dict:
    turn = {"role": "assistant", "content": text}
    if _is(message.get("reasoning_content"), str):
        turn["reasoning_content"] = message["reasoning_content"]
    calls = message.get("tool_calls")
    if calls is not None:
        _require(_is(calls, list) and len(calls) > 0, "tool_calls must be a non-empty array")
        turn["tool_calls"] = [_tool_call(call) for call in calls]
    _require(text != "" or "tool_calls" in turn, "assistant messages need content or tool_calls")
    return turn


def _tool_result(message: dict, text: str) -> dict:
    answered = message.get("tool_call_id")
    _require(_is(answered, str) and answered != "", "tool messages need tool_call_id")
    return {"role": "tool", "content": text, "tool_call_id": answered}


_CONVERTERS = {"system": _spoken, "user": _spoken, "assistant": _assistant, "tool": _tool_result}


def convert(messages) -> list[dict]:
    _require(_is(messages, list) and len(messages) > 0, "messages must be a non-empty array")
    _require(_wire_size(messages) <= MESSAGES_CAP, "messages exceed the supported size")
    turns = []
    for message in messages:
        converter = _CONVERTERS.get(message.get("role")) if _is(message, dict) else None
        _require(converter is not None, "each message needs a role of system, user, assistant or tool")
        turns.append(converter(message, _flatten(message.get("content"))))
    return turns


# ------------------------------------------------------------------------------------------------------------------ tools
def check_tools(tools):
    if tools is None:
        return None
    _require(_is(tools, list) and len(tools) > 0, "tools must be a non-empty array when present")
    _require(_wire_size(tools) <= TOOLS_CAP, "tool definitions exceed the supported size")
    for tool in tools:
        _require(_is(tool, dict) and tool.get("type") in (None, "function"), "only function tools are supported")
        function = tool.get("function", tool)  # both the wrapped and the bare form are in use
        _require(_is(function, dict) and _is(function.get("name"), str), "each tool needs function.name")
        schema = function.get("parameters")
        _require(schema is None or _is(schema, dict), "tool parameters must be a JSON schema object")
    return tools


def _choice_note(tool_choice) -> str:
    if _is(tool_choice, str) and tool_choice in CHOICE_NOTES:
        return CHOICE_NOTES[tool_choice]
    selector = tool_choice.get("function") if _is(tool_choice, dict) else None
    _require(_is(selector, dict), "tool_choice must be auto, none, required or a function selector")
    _require(_is(selector.get("name"), str), "tool_choice.function.name must be a string")
    return NAMED_CHOICE_NOTE.format(name=selector["name"])


def instruct(messages: list[dict], tool_choice, tools) -> list[dict]:
    if not tools or tool_choice is None or tool_choice == "auto":
        return messages
    note = _choice_note(tool_choice)
    head, rest = messages[0], list(messages[1:])
    if head["role"] != "system":
        return [{"role": "system", "content": note}, head, *rest]
    return [{**head, "content": head["content"].rstrip() + "\n\n" + note}, *rest]
