"""Tool calls in generated text.

GLM writes a call as ``<tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call>`` inside its answer.  ``parse`` walks the
answer once with a cursor: text outside call blocks is the visible content, each block becomes one OpenAI ``tool_calls`` entry.  An
argument value that is valid JSON keeps its JSON type (numbers, booleans, objects); anything else is passed on as a string.  A block
without a name is dropped; an unterminated ``<tool_call>`` is not a call and stays in the content.

Behaviour parity: reference ``glm_tpu/entrypoints/openai/tool_parser.py`` (same output shape: ``id``, ``type``, ``index``, ``function``).
"""

from __future__ import annotations

import json
import uuid

OPEN, CLOSE = "<tool_call>", "</tool_call>"
KEY_OPEN, KEY_CLOSE = "<arg_key>", "</arg_key>"
VALUE_OPEN, VALUE_CLOSE = "<arg_value>", "</arg_value>"


def _between(text: str, start: int, opening: str, closing: str):
    """``(inner, index after closing)`` of the next ``opening ... closing`` at or after ``start``; ``None`` when there is none."""
    a = text.find(opening, start)
    if a < 0:
        return None
    b = text.find(closing, a + len(opening))
    if b < 0:
        return None
    return text[a + len(opening):b], b + len(closing)


def _typed(raw: str):
    raw = raw.strip()
    try:
        return json.loads(raw)
    except ValueError:
        return raw


def _call(block: str, index: int):
    name = block.partition(KEY_OPEN)[0].strip()
    if not name:
        return None
    arguments, cursor = {}, 0
    while True:
        key = _between(block, cursor, KEY_OPEN, KEY_CLOSE)
        if key is None:
            break
        value = _between(block, key[1], VALUE_OPEN, VALUE_CLOSE)
        if value is None or block[key[1]:block.find(VALUE_OPEN, key[1])].strip():
            break  # a key without its value directly after it ends the argument list
        arguments[key[0].strip()] = _typed(value[0])
        cursor = value[1]
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function", "index": index,
            "function": {"name": name, "arguments": json.dumps(arguments, ensure_ascii=False)}}


def parse(answer: str):
    """``(visible content, tool calls)``."""
    visible, calls, cursor = [], [], 0
    while True:
        start = answer.find(OPEN, cursor)
        found = _between(answer, cursor, OPEN, CLOSE) if start >= 0 else None
        if found is None:
            visible.append(answer[cursor:])
            break
        visible.append(answer[cursor:start])
        call = _call(found[0], len(calls))
        if call is not None:
            calls.append(call)
        cursor = found[1]
    return "".join(visible).strip(), calls
