"""Tool calls both ways: what the chat format writes for an assistant turn with calls is what the parser reads back from generated
text, and the parser's behaviour on the shapes a model actually produces (newlines, several calls, text around them, blocks that
never close).

Reference counterparts: ``tests/entrypoints/openai/test_serving_chat.py`` (tool-call conversion both ways)."""

import json

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from glm_tpu_b200.entrypoints.openai import chat_utils, tool_parser
from glm_tpu_b200.exceptions import ApiError
from glm_tpu_b200.tokenizer import chat_template


def is_json(text: str) -> bool:
    try:
        json.loads(text.strip())
        return True
    except ValueError:
        return False


MARKUP = ("<", ">")
plain_text = st.text(alphabet=st.characters(blacklist_categories=("Cs",), blacklist_characters="<>"), min_size=1, max_size=20)
# a string value comes back as a string only if it is not itself JSON (a model that writes 12 means the number) and survives strip()
string_values = plain_text.filter(lambda s: s == s.strip() and s != "" and not is_json(s))
json_values = st.recursive(st.none() | st.booleans() | st.integers(-10**6, 10**6) | st.floats(allow_nan=False, allow_infinity=False, width=32),
                           lambda inner: st.lists(inner, max_size=3) | st.dictionaries(st.text("abc", min_size=1, max_size=3), inner, max_size=3), max_leaves=6)
keys = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_0123456789", min_size=1, max_size=12)
names = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_.-0123456789", min_size=1, max_size=20).filter(lambda s: s == s.strip())


@settings(max_examples=150, deadline=None)
@given(name=names, arguments=st.dictionaries(keys, string_values | json_values, max_size=5), before=st.sampled_from(["", "I will look.", "Zeile\nzwei "]))
def test_what_the_format_writes_the_parser_reads(name, arguments, before):
    turn = {"role": "assistant", "content": before, "tool_calls": [{"function": {"name": name, "arguments": arguments}}]}
    text = chat_template.render([{"role": "user", "content": "q"}, turn], add_generation_prompt=False)
    generated = text.split("</think>", 1)[1]  # what a model would have produced after its reasoning
    content, calls = tool_parser.parse(generated)
    assert content == before.strip()
    assert len(calls) == 1 and calls[0]["function"]["name"] == name and calls[0]["index"] == 0 and calls[0]["type"] == "function"
    assert json.loads(calls[0]["function"]["arguments"]) == arguments
    # and once more through the request side: an OpenAI client sends the call back as history
    history = chat_utils.convert([{"role": "user", "content": "q"},
                                  {"role": "assistant", "content": content or None, "tool_calls": [{"id": calls[0]["id"], "type": "function",
                                                                                                    "function": calls[0]["function"]}]},
                                  {"role": "tool", "tool_call_id": calls[0]["id"], "content": "result"}])
    assert history[1]["tool_calls"][0]["function"] == {"name": name, "arguments": arguments}
    assert chat_template.render(history[:2], add_generation_prompt=False) == text


def test_shapes_a_model_produces():
    content, calls = tool_parser.parse("Let me check.\n<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Köln</arg_value>\n"
                                       "<arg_key>days</arg_key>\n<arg_value>2</arg_value>\n</tool_call>\n")
    assert content == "Let me check." and json.loads(calls[0]["function"]["arguments"]) == {"city": "Köln", "days": 2}
    assert "Köln" in calls[0]["function"]["arguments"]  # not \\u-escaped

    content, calls = tool_parser.parse("<tool_call>a<arg_key>x</arg_key><arg_value>1</arg_value></tool_call> and "
                                       "<tool_call>b</tool_call> done")
    assert content == "and  done" and [c["function"]["name"] for c in calls] == ["a", "b"] and [c["index"] for c in calls] == [0, 1]
    assert json.loads(calls[1]["function"]["arguments"]) == {} and calls[0]["id"] != calls[1]["id"]
    assert all(c["id"].startswith("call_") and len(c["id"]) == 29 for c in calls)

    typed = tool_parser.parse('<tool_call>f<arg_key>a</arg_key><arg_value>{"k": [1, true, null]}</arg_value><arg_key>b</arg_key><arg_value> 3.5 </arg_value>'
                              "<arg_key>c</arg_key><arg_value>not json {</arg_value><arg_key>d</arg_key><arg_value>\"quoted\"</arg_value></tool_call>")[1][0]
    assert json.loads(typed["function"]["arguments"]) == {"a": {"k": [1, True, None]}, "b": 3.5, "c": "not json {", "d": "quoted"}


def test_blocks_that_are_not_calls():
    assert tool_parser.parse("just text") == ("just text", [])
    assert tool_parser.parse("") == ("", [])
    assert tool_parser.parse("before <tool_call>never closed<arg_key>a</arg_key>") == ("before <tool_call>never closed<arg_key>a</arg_key>", [])
    assert tool_parser.parse("a <tool_call></tool_call> b") == ("a  b", [])  # a block without a name is dropped
    assert tool_parser.parse("a <tool_call>  <arg_key>k</arg_key><arg_value>v</arg_value></tool_call> b") == ("a  b", [])
    content, calls = tool_parser.parse("<tool_call>f<arg_key>a</arg_key><arg_key>b</arg_key><arg_value>1</arg_value></tool_call>")
    assert content == "" and json.loads(calls[0]["function"]["arguments"]) == {}  # a key without its value ends the list
    content, calls = tool_parser.parse("<tool_call>f<arg_key>a</arg_key><arg_value>1</arg_value><arg_key>b</arg_key></tool_call>")
    assert json.loads(calls[0]["function"]["arguments"]) == {"a": 1}
    content, calls = tool_parser.parse("x</tool_call>y<tool_call>f</tool_call>")
    assert content == "x</tool_call>y" and len(calls) == 1  # a stray closing tag is text
    content, calls = tool_parser.parse("<tool_call>f</tool_call><tool_call>open")
    assert content == "<tool_call>open" and len(calls) == 1


def test_history_shapes_that_are_refused():
    user = {"role": "user", "content": "q"}
    for bad, sentence in (
        ([user, {"role": "assistant", "content": None, "tool_calls": []}], "non-empty array"),
        ([user, {"role": "assistant", "content": None, "tool_calls": [{"function": {"arguments": "{}"}}]}], "function.name"),
        ([user, {"role": "assistant", "content": None, "tool_calls": [{"function": {"name": "f", "arguments": "[1]"}}]}], "decode to an object"),
        ([user, {"role": "assistant", "content": None, "tool_calls": [{"function": {"name": "f", "arguments": "{oops"}}]}], "not valid JSON"),
        ([user, {"role": "assistant", "content": None, "tool_calls": [{"function": {"name": "f", "arguments": 5}}]}], "JSON object string"),
        ([user, {"role": "assistant", "content": None, "tool_calls": "f"}], "non-empty array"),
        ([user, {"role": "assistant", "content": None}], "content or tool_calls"),
        ([user, {"role": "tool", "content": "r"}], "tool_call_id"),
        ([user, {"role": "tool", "content": "r", "tool_call_id": ""}], "tool_call_id"),
        ([{"role": "user", "content": [{"type": "image_url", "image_url": {}}]}], "only text content parts"),
        ([{"role": "user", "content": 5}], "string or a list"),
        ([{"role": "user", "content": " \n"}], "need text content"),
        ([{"role": "developer", "content": "x"}], "role of system, user, assistant or tool"),
        (["user"], "role of system"),
        ([], "non-empty array"),
        ({"role": "user"}, "non-empty array"),
    ):
        with pytest.raises(ApiError, match=sentence):
            chat_utils.convert(bad)
    ok = chat_utils.convert([user, {"role": "assistant", "content": None, "tool_calls": [{"id": "c1", "function": {"name": "f", "arguments": ""}}]},
                             {"role": "tool", "tool_call_id": "c1", "content": None}])
    assert ok[1]["tool_calls"][0]["function"]["arguments"] == {} and ok[2] == {"role": "tool", "content": "", "tool_call_id": "c1"}


def test_tool_definitions_and_choices():
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}, {"name": "bare"}]
    assert chat_utils.check_tools(tools) is tools and chat_utils.check_tools(None) is None
    for bad, sentence in (([], "non-empty array"), ("f", "non-empty array"), ([{"type": "retrieval"}], "only function tools"),
                          ([{"type": "function", "function": {"description": "no name"}}], "function.name"),
                          ([{"type": "function", "function": {"name": "f", "parameters": []}}], "JSON schema object"), ([5], "only function tools")):
        with pytest.raises(ApiError, match=sentence):
            chat_utils.check_tools(bad)
    plain = [{"role": "user", "content": "hi"}]
    assert chat_utils.instruct(plain, "auto", tools) is plain and chat_utils.instruct(plain, None, tools) is plain
    assert chat_utils.instruct(plain, "required", None) is plain  # nothing to call: nothing to demand
    forced = chat_utils.instruct(plain, "required", tools)
    assert forced[0] == {"role": "system", "content": chat_utils.CHOICE_NOTES["required"]} and forced[1:] == plain
    named = chat_utils.instruct([{"role": "system", "content": "be brief \n"}, *plain], {"type": "function", "function": {"name": "f"}}, tools)
    assert named[0]["content"] == "be brief\n\nYou must answer this turn by calling the function named f." and named[1:] == plain
    assert "Do not call any function" in chat_utils.instruct(plain, "none", tools)[0]["content"]
    for bad in ("whatever", 5, {"type": "function"}, {"function": {"name": 5}}):
        with pytest.raises(ApiError, match="tool_choice"):
            chat_utils.instruct(plain, bad, tools)
