"""Parse GLM ``<tool_call>name<arg_key>k</arg_key><arg_value>v</arg_value>...</tool_call>`` blocks out of an answer.

Parity: reference ``glm_tpu/entrypoints/openai/tool_parser.py:11-39``.
"""

from __future__ import annotations

import json
import re
import uuid

CALL = re.compile(r"<tool_call>(.*?)</tool_call>", re.S)
ARGUMENT = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)
OPEN = "<tool_call>"


def parse(answer: str):
    """``(visible content, OpenAI tool calls)``; argument values are JSON when they parse, else strings."""
    calls = []
    for block in CALL.findall(answer):
        name = block.split("<arg_key>", 1)[0].strip()
        if not name:
            continue
        arguments = {}
        for key, raw in ARGUMENT.findall(block):
            value = raw.strip()
            try:
                arguments[key.strip()] = json.loads(value)
            except ValueError:
                arguments[key.strip()] = value
        calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function", "index": len(calls),
                      "function": {"name": name, "arguments": json.dumps(arguments, ensure_ascii=False)}})
    return CALL.sub("", answer).strip(), calls
