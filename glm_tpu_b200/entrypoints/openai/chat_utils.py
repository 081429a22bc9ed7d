"""OpenAI chat messages and tools mapped onto what the GLM chat format renders.

``convert`` validates an OpenAI message array (roles system / user / assistant / tool; string or text-part content;
assistant ``tool_calls`` with JSON-string arguments; tool messages with ``tool_call_id``) and returns the template's
shape.  ``check_tools`` accepts function tools only.  ``instruct`` states a ``tool_choice`` constraint in-band, as a
system instruction, because the chat format has no such field.

Parity: reference ``glm_tpu/entrypoints/openai/chat_utils.py:11-128``.
"""

from __future__ import annotations

import json

from glm_tpu_b200.entrypoints.openai.protocol import MESSAGES_CAP, TOOLS_CAP, ApiError

ROLES = ("system", "user", "assistant", "tool")


def text_of(content) -> str:
    if content is None:
        return ""
    if type(content) is str:
        return content
    if type(content) is list:
        parts = []
        for part in content:
            if type(part) is not dict or part.get("type") != "text" or type(part.get("text")) is not str:
                raise ApiError("only text content parts are supported")
            parts.append(part["text"])
        return "".join(parts)
    raise ApiError("message content must be a string or a list of text parts")


def arguments_of(value) -> dict:
    if type(value) is dict:
        return value
    if type(value) is not str:
        raise ApiError("tool call arguments must be a JSON object string")
    if not value.strip():
        return {}
    try:
        parsed = json.loads(value)
    except ValueError as exc:
        raise ApiError("tool call arguments are not valid JSON") from exc
    if type(parsed) is not dict:
        raise ApiError("tool call arguments must decode to an object")
    return parsed


def convert(messages) -> list[dict]:
    if type(messages) is not list or not messages:
        raise ApiError("messages must be a non-empty array")
    if len(json.dumps(messages).encode()) > MESSAGES_CAP:
        raise ApiError("messages exceed the supported size")
    out = []
    for message in messages:
        if type(message) is not dict or message.get("role") not in ROLES:
            raise ApiError("each message needs a role of system, user, assistant or tool")
        role = message["role"]
        rendered = {"role": role, "content": text_of(message.get("content"))}
        if role == "assistant":
            if type(message.get("reasoning_content")) is str:
                rendered["reasoning_content"] = message["reasoning_content"]
            calls = message.get("tool_calls")
            if calls is not None:
                if type(calls) is not list or not calls:
                    raise ApiError("tool_calls must be a non-empty array")
                rendered["tool_calls"] = []
                for call in calls:
                    fn = call.get("function") if type(call) is dict else None
                    if type(fn) is not dict or type(fn.get("name")) is not str:
                        raise ApiError("each tool call needs function.name")
                    rendered["tool_calls"].append({"id": call.get("id") or "", "type": "function",
                                                   "function": {"name": fn["name"], "arguments": arguments_of(fn.get("arguments", "{}"))}})
            if not rendered["content"] and "tool_calls" not in rendered:
                raise ApiError("assistant messages need content or tool_calls")
        elif role == "tool":
            if type(message.get("tool_call_id")) is not str or not message["tool_call_id"]:
                raise ApiError("tool messages need tool_call_id")
            rendered["tool_call_id"] = message["tool_call_id"]
        elif not rendered["content"].strip():
            raise ApiError(role + " messages need text content")
        out.append(rendered)
    return out


def check_tools(tools):
    if tools is None:
        return None
    if type(tools) is not list or not tools:
        raise ApiError("tools must be a non-empty array when present")
    if len(json.dumps(tools).encode()) > TOOLS_CAP:
        raise ApiError("tool definitions exceed the supported size")
    for tool in tools:
        if type(tool) is not dict or tool.get("type") not in (None, "function"):
            raise ApiError("only function tools are supported")
        fn = tool.get("function", tool)
        if type(fn) is not dict or type(fn.get("name")) is not str:
            raise ApiError("each tool needs function.name")
        if fn.get("parameters") is not None and type(fn["parameters"]) is not dict:
            raise ApiError("tool parameters must be a JSON schema object")
    return tools


def instruct(messages: list[dict], tool_choice, tools) -> list[dict]:
    if tool_choice in (None, "auto") or not tools:
        return messages
    if tool_choice == "none":
        note = "Do not call any function for this turn. Answer directly in plain text."
    elif tool_choice == "required":
        note = "You must answer this turn by calling one of the provided functions."
    elif type(tool_choice) is dict and type(tool_choice.get("function")) is dict:
        name = tool_choice["function"].get("name")
        if type(name) is not str:
            raise ApiError("tool_choice.function.name must be a string")
        note = "You must answer this turn by calling the function named " + name + "."
    else:
        raise ApiError("tool_choice must be auto, none, required or a function selector")
    messages = list(messages)
    if messages[0]["role"] == "system":
        messages[0] = dict(messages[0], content=messages[0]["content"].rstrip() + "\n\n" + note)
    else:
        messages.insert(0, {"role": "system", "content": note})
    return messages
