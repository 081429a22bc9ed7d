"""The chat format, conversation by conversation, against digests of what the model's published ``chat_template.jinja`` renders for
the same messages (computed once with jinja2 from the template file of the GLM-5.3 repository; ``trim_blocks`` and
``lstrip_blocks`` on, ``tojson`` without ASCII escaping).  A change to ``tokenizer/chat_template.py`` that alters one byte of one of
these prompts changes the tokens the model sees, so it has to show up here.

Reference counterpart: the pinned ``glm_tpu/models/glm_moe_dsa/hf_config/chat_template.jinja`` and ``tests/engine/test_request.py``."""

import hashlib

import pytest

from glm_tpu_b200.tokenizer import chat_template

TOOLS = [
    {"type": "function", "function": {"name": "get_weather", "description": "Weather für a city",
                                      "parameters": {"type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}},
                                                     "required": ["city"]}}},
    {"type": "function", "function": {"name": "hidden", "description": "x", "parameters": {}, "defer_loading": True}},
    {"name": "bare", "description": "no wrapper", "parameters": {"type": "object"}, "strict": True},
]
WEATHER_CALL = {"type": "function", "function": {"name": "get_weather", "arguments": {"city": "Köln", "days": 2}}}
CASES = {
    "user": (dict(messages=[{"role": "user", "content": "Hi"}]), "52dda9a6f66c9bf241b9c7b3839c46a7f82a886bb3f3bc3f03e300d5409c453e"),
    "system_user": (dict(messages=[{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"}]),
                    "03146e8dfd8434008c51526917d413d240f628387d17f9a06868f8e9299677e5"),
    "low": (dict(messages=[{"role": "user", "content": "Hi"}], reasoning_effort="low"),
            "e5066f3ce8efe86e111c2cc37d753c67b6d17d6308e297a820e6d05643ea227c"),
    "high": (dict(messages=[{"role": "user", "content": "Hi"}], reasoning_effort="high"),
             "da98d84ee17dbb0151b1cac2ed3fe45709311161aaea615d36eb943159bc1ff5"),
    "max": (dict(messages=[{"role": "user", "content": "Hi"}], reasoning_effort="max"),
            "52dda9a6f66c9bf241b9c7b3839c46a7f82a886bb3f3bc3f03e300d5409c453e"),
    "multi": (dict(messages=[{"role": "user", "content": "1+1"}, {"role": "assistant", "content": "2", "reasoning_content": "adding"},
                             {"role": "user", "content": "and 2+2?"}]),
              "924064de514f98b8055d931fbb39fa5792da582b196ad6ab81b7b2759a16e0b4"),
    "multi_inline_think": (dict(messages=[{"role": "user", "content": "1+1"}, {"role": "assistant", "content": "<think>adding</think>\n2\n"},
                                          {"role": "user", "content": "more"}]),
                           "f951b413a4b881e87350fd31b7e464300b476657f1ef92ba079ed00dac251051"),
    "assistant_last": (dict(messages=[{"role": "user", "content": "1+1"}, {"role": "assistant", "content": "2", "reasoning_content": "adding"}]),
                       "3d7a95cc394d59ba8dfc8c952dcd4307b38af7ac2977dd287d4ffc3c530b831b"),
    "no_generation_prompt": (dict(messages=[{"role": "user", "content": "Hi"}], add_generation_prompt=False),
                             "b1c3effec667179e7c121f982f0981189a3ca1c4deadb56cc2caeb4f2237b7ca"),
    "tools": (dict(messages=[{"role": "user", "content": "Weather in Köln?"}], tools=TOOLS),
              "7cc7d14c19c3aaebdee5367ac6d2b9d8b8cbf939f94903956b5f598be74656f3"),
    "tool_round": (dict(messages=[{"role": "user", "content": "Weather?"},
                                  {"role": "assistant", "content": "", "reasoning_content": "need tool", "tool_calls": [WEATHER_CALL]},
                                  {"role": "tool", "content": "{\"temp\": 7}"}, {"role": "tool", "content": "second"},
                                  {"role": "assistant", "content": "It is 7 degrees."}, {"role": "user", "content": "thanks"}], tools=TOOLS),
                   "cbe260efd0e029d077aec6437ba088884217684ba19f1e33f7853278f9c90e86"),
    "content_parts": (dict(messages=[{"role": "user", "content": [{"type": "text", "text": "look: "}, {"type": "image_url", "image_url": {"url": "x"}},
                                                                   {"type": "text", "text": " done"}]}]),
                      "26c844b0e62ade89bea83e74b2d0b8af5eac807b471ea0f988090e93d11bcc0a"),
    "clear_thinking": (dict(messages=[{"role": "user", "content": "1+1"}, {"role": "assistant", "content": "2", "reasoning_content": "adding"},
                                      {"role": "user", "content": "x"}, {"role": "assistant", "content": "y", "reasoning_content": "later"}],
                            clear_thinking=True),
                       "bd8764cc9fb7293cc21d5b91f0e4065fcd4cf5187cc88c2058a0304e95c05c63"),
    "system_in_the_middle": (dict(messages=[{"role": "user", "content": "a"}, {"role": "system", "content": "s"}, {"role": "user", "content": "b"}]),
                             "b61d543eb288f3ed8a876c5c366f8b24ffb9d49b09d9757d4dc89e9be2fb956b"),
    "assistant_without_content": (dict(messages=[{"role": "user", "content": "a"},
                                                 {"role": "assistant", "content": None, "tool_calls": [{"function": {"name": "bare", "arguments": {}}}]},
                                                 {"role": "tool", "content": "r"}], tools=TOOLS),
                                  "daf15fdf7cc779420fce7c0af0ffb67dffe0bfdd73bba689daaaa8d483c6fa6b"),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_prompt_matches_the_published_template(name):
    kw, digest = CASES[name]
    kw = dict(kw)
    text = chat_template.render(kw.pop("messages"), **kw)
    assert hashlib.sha256(text.encode("utf-8")).hexdigest() == digest, text

U = {"role": "user", "content": "q"}
EDGE_CASES = {
    "empty_reasoning": (dict(messages=[U, {"role": "assistant", "content": "a", "reasoning_content": ""}, U]),
                        "f3e032c0e088a8033b251b1a9697def3787fad0011c51bf3d6ef1703c0a543aa"),
    "assistant_content_is_stripped": (dict(messages=[U, {"role": "assistant", "content": "  a \n"}, U]),
                                      "f3e032c0e088a8033b251b1a9697def3787fad0011c51bf3d6ef1703c0a543aa"),
    "assistant_only_whitespace": (dict(messages=[U, {"role": "assistant", "content": "  \n"}, U]),
                                  "a420b645c6ca1271df15ccde23cde1520a7ab185418d6d22e16599c227a25dc8"),
    "unknown_effort_is_max": (dict(messages=[U], reasoning_effort="medium"), "6783283c6dfca3913a7ecd8f8b28ba0a13a71f65706a8c994c28628f078297cd"),
    "no_effort_is_max": (dict(messages=[U], reasoning_effort=None), "6783283c6dfca3913a7ecd8f8b28ba0a13a71f65706a8c994c28628f078297cd"),
    "empty_tool_list": (dict(messages=[U], tools=[]), "6783283c6dfca3913a7ecd8f8b28ba0a13a71f65706a8c994c28628f078297cd"),
    "argument_types": (dict(messages=[U, {"role": "assistant", "content": "", "tool_calls": [
        {"function": {"name": "f", "arguments": {"b": True, "n": None, "x": 1.5, "s": "ü", "l": ["ä", 1]}}}]}]),
                       "b5c0ffc703b1fa20ea6b2850540bd2c479d2f1358c3736901783518f75b08972"),
    "tool_result_first": (dict(messages=[{"role": "tool", "content": "r"}, U]), "1710330dac8cff92e5260162eaa65db42900e7933390b40b7764e25a3848cab7"),
    "tool_result_in_parts": (dict(messages=[U, {"role": "tool", "content": [{"type": "text", "text": "a"}, {"type": "text", "text": "b"}]}]),
                             "0560f0a11da28ee2bee5b967637c577563ea44fb587730627bd13fa927efb3db"),
    "tool_result_with_media": (dict(messages=[U, {"role": "tool", "content": [{"type": "image", "image": "x"}]}]),
                               "3ee503ea1c9c60440abb8a0e9252d729b89503b165dd72fd2ccc6a11873ab6fd"),
    "user_without_content": (dict(messages=[{"role": "user", "content": None}]), "e69c157c0ca86608e0090d6ff3263d1ca330eb16c54753f302086daffea6d03c"),
    "video_and_audio_parts": (dict(messages=[{"role": "user", "content": [{"type": "video_url"}, {"type": "input_audio"}, {"type": "audio"}]}]),
                              "28cbf839a1d6b7ad9efa73d6327a886db4251a2a455c724c39b96e1cebfd73fa"),
    "two_calls_in_one_turn": (dict(messages=[U, {"role": "assistant", "content": "x", "tool_calls": [
        {"function": {"name": "f", "arguments": {"a": 1}}}, {"function": {"name": "g", "arguments": {}}}]}]),
                              "33f6021b7ac6c2e242eeb1cd9175432b8712d74cb0873423d49f9de044c8579d"),
    "call_without_function_wrapper": (dict(messages=[U, {"role": "assistant", "content": "x", "tool_calls": [{"name": "f", "arguments": {"a": "1"}}]}]),
                                      "8e5fe79aac7269404d2f712db036074b704548202892660065195706260a62af"),
    "given_reasoning_wins_over_inline": (dict(messages=[U, {"role": "assistant", "content": "<think>old</think>visible", "reasoning_content": "given"}, U]),
                                         "9f497953626eac7a61438549c94616fbb15bec3acc6b03fa283188ced490659c"),
    "reasoning_kept_in_every_turn": (dict(messages=[U, {"role": "assistant", "content": "a", "reasoning_content": "r1"}, U,
                                                    {"role": "assistant", "content": "b", "reasoning_content": "r2"}, U], clear_thinking=False),
                                     "9f8046aa25d18930897ecd4607dfb8f10c9b0229f3b8bf5a3d73748a4c95a780"),
    "cleared_reasoning_survives_after_the_last_user_turn": (dict(messages=[
        U, {"role": "assistant", "content": "", "reasoning_content": "r1", "tool_calls": [{"function": {"name": "f", "arguments": {}}}]},
        {"role": "tool", "content": "t"}, {"role": "assistant", "content": "b", "reasoning_content": "r2"}], clear_thinking=True),
                                                            "94bca739d4828724dcac5833373b88730f27946149c59c5a7321812335248731"),
    "system_in_parts": (dict(messages=[{"role": "system", "content": [{"type": "text", "text": "S"}]}, U]),
                        "1760381dd3fbd79c05259963c36febd0168492ee2e175a5718aeece062d46689"),
    "nested_unicode_in_a_signature": (dict(messages=[U], tools=[{"type": "function", "function": {
        "name": "f", "description": "d", "parameters": {"type": "object", "properties": {"a": {"enum": ["ä", "b"]}}}}}]),
                                      "512e98c0b0d3b1a04771300306cd82f1669704bdc7f484777098bf0eec996fec"),
}


@pytest.mark.parametrize("name", sorted(EDGE_CASES))
def test_edge_cases_match_the_published_template(name):
    kw, digest = EDGE_CASES[name]
    kw = dict(kw)
    text = chat_template.render(kw.pop("messages"), **kw)
    assert hashlib.sha256(text.encode("utf-8")).hexdigest() == digest, text


def test_what_the_digests_stand_for():
    """Spot checks in clear text, so that a reader sees the format without computing a digest."""
    kw, _ = CASES["tool_round"]
    text = chat_template.render(kw["messages"], tools=kw["tools"])
    assert text.startswith("[gMASK]<sop><|system|>Reasoning Effort: Max<|system|>\n# Tools\n")
    assert '"name": "get_weather"' in text and '"hidden"' not in text and '"strict"' not in text  # deferred tools and the strict flag are left out
    assert "Weather für a city" in text  # no ASCII escaping
    assert "<|assistant|><think>need tool</think><tool_call>get_weather<arg_key>city</arg_key><arg_value>Köln</arg_value><arg_key>days</arg_key><arg_value>2</arg_value></tool_call>" in text
    assert '<|observation|><tool_response>{"temp": 7}</tool_response><tool_response>second</tool_response><|assistant|>' in text
    assert text.endswith("<|user|>thanks<|assistant|><think>")
    assert CASES["user"][1] == CASES["max"][1]  # maximum effort is the default


def test_arguments_sent_as_a_json_string_render_like_the_object():
    """OpenAI clients send ``arguments`` as a JSON string; the published template only takes an object.  Here both give the same prompt."""
    as_object = {"role": "assistant", "content": "calling", "tool_calls": [{"function": {"name": "get_weather", "arguments": {"city": "Bonn", "opts": {"a": [1, 2]}}}}]}
    as_string = {"role": "assistant", "content": "calling", "tool_calls": [{"function": {"name": "get_weather", "arguments": "{\"city\": \"Bonn\", \"opts\": {\"a\": [1, 2]}}"}}]}
    user = {"role": "user", "content": "Weather?"}
    assert chat_template.render([user, as_string], tools=TOOLS) == chat_template.render([user, as_object], tools=TOOLS)
    assert '<arg_key>opts</arg_key><arg_value>{"a": [1, 2]}</arg_value>' in chat_template.render([user, as_object])
    empty = {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "bare", "arguments": ""}}]}
    assert "<tool_call>bare</tool_call>" in chat_template.render([user, empty])


def test_an_unknown_role_is_refused():
    with pytest.raises(ValueError, match="unsupported message role"):
        chat_template.render([{"role": "developer", "content": "x"}])
