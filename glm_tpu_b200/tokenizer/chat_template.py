"""The GLM-5.3 chat format rendered in Python.

Produces the same prompt text as the model's published template for the message shapes the engine accepts:
``[gMASK]<sop>``, a ``Reasoning Effort`` system line (low / high / max), an optional ``# Tools`` system block with one
JSON signature per line inside ``<tools>``, then the turns -- ``<|system|>``, ``<|user|>``, ``<|assistant|>`` with its
``<think>...</think>`` block and ``<tool_call>name<arg_key>k</arg_key><arg_value>v</arg_value></tool_call>`` calls,
``<|observation|>`` with one ``<tool_response>`` per tool result -- and the generation prompt ``<|assistant|><think>``.

Message content may be a string or a list of parts; only text parts are rendered (other media get the model's
"unable to process" reminder).  When a checkpoint directory ships ``chat_template.jinja`` and jinja2 is available, the
tokenizer wrapper prefers that file; this module is the dependency-free default and the reference for the tests.

Parity: reference ``glm_tpu/models/glm_moe_dsa/hf_config/chat_template.jinja`` (format), ``engine/request.py:180-212``.
"""

from __future__ import annotations

import json
from typing import Any, Iterable

MEDIA = ("image", "image_url", "video", "video_url", "audio", "audio_url", "input_audio")
TOOLS_HEADER = (
    "<|system|>\n# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
    "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n"
)
TOOLS_FOOTER = (
    "</tools>\n\nFor each function call, output the function name and arguments within the following XML format:\n"
    "<tool_call>{function-name}<arg_key>{arg-key-1}</arg_key><arg_value>{arg-value-1}</arg_value>"
    "<arg_key>{arg-key-2}</arg_key><arg_value>{arg-value-2}</arg_value>...</tool_call>"
)


def _json(value: Any) -> str:
    return json.dumps(value, ensure_ascii=False)


def visible_text(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if isinstance(content, dict):
        return str(content)
    out = []
    for item in content:
        if isinstance(item, str):
            out.append(item)
        elif isinstance(item, dict) and item.get("type") == "text":
            out.append(item.get("text", ""))
        elif isinstance(item, dict) and item.get("type") in MEDIA:
            kind = item["type"].replace("_url", "").replace("input_", "")
            out.append(f"<reminder>You are unable to process this {kind} because you don't have multi-modal input ability. "
                       "Try different methods.</reminder>")
    return "".join(out)


def _tool_json(tool: dict) -> str:
    if "function" in tool:
        tool = tool["function"]
    parts = [f'"{k}": {_json(v)}' for k, v in tool.items() if k not in ("defer_loading", "strict")]
    return "{" + ", ".join(parts) + "}"


def _assistant(m: dict, show_reasoning: bool) -> str:
    content = visible_text(m.get("content"))
    reasoning = m.get("reasoning_content") if isinstance(m.get("reasoning_content"), str) else None
    if reasoning is None and "</think>" in content:
        reasoning = content.split("</think>")[0].split("<think>")[-1]
        content = content.split("</think>")[-1]
    out = "<|assistant|>"
    out += f"<think>{reasoning}</think>" if (show_reasoning and reasoning is not None) else "<think></think>"
    if content.strip():
        out += content.strip()
    for tc in m.get("tool_calls") or []:
        fn = tc.get("function", tc)
        args = fn.get("arguments") or {}
        if isinstance(args, str):
            args = json.loads(args) if args.strip() else {}
        out += "<tool_call>" + fn["name"]
        for k, v in args.items():
            out += f"<arg_key>{k}</arg_key><arg_value>{v if isinstance(v, str) else _json(v)}</arg_value>"
        out += "</tool_call>"
    return out


def render(messages: Iterable[dict], *, tools: list | None = None, reasoning_effort: str | None = None,
           add_generation_prompt: bool = True, clear_thinking: bool = False) -> str:
    messages = list(messages)
    effort = reasoning_effort if reasoning_effort in ("low", "high") else "max"
    out = "[gMASK]<sop>" + f"<|system|>Reasoning Effort: {effort.capitalize()}"
    if tools:
        out += TOOLS_HEADER
        for tool in tools:
            body = tool.get("function", tool)
            if not body.get("defer_loading"):
                out += _tool_json(tool) + "\n"
        out += TOOLS_FOOTER
    last_user = max((i for i, m in enumerate(messages) if m.get("role") == "user"), default=-1)
    for i, m in enumerate(messages):
        role = m.get("role")
        if role == "user":
            out += "<|user|>" + visible_text(m.get("content"))
        elif role == "system":
            out += "<|system|>" + visible_text(m.get("content"))
        elif role == "assistant":
            out += _assistant(m, show_reasoning=(not clear_thinking) or i > last_user)
        elif role == "tool":
            if i == 0 or messages[i - 1].get("role") != "tool":
                out += "<|observation|>"
            out += "<tool_response>" + visible_text(m.get("content")) + "</tool_response>"
        else:
            raise ValueError(f"unsupported message role {role!r}")
    if add_generation_prompt:
        out += "<|assistant|><think>"
    return out
