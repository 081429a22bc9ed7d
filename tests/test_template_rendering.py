"""A checkpoint's own ``chat_template.jinja`` is rendered the way the model's tooling renders it.  The part that matters most is
``tojson``: tool signatures reach the model as plain ``json.dumps`` text (given key order, no ASCII or HTML escaping), which is also
what the built-in Python statement of the chat format writes.

Reference counterpart: the pinned template under ``glm_tpu/models/glm_moe_dsa/hf_config`` rendered through the tokenizer library."""

import json

import pytest

jinja2 = pytest.importorskip("jinja2")

from glm_tpu_b200.tokenizer import chat_template, render_jinja  # noqa: E402

TOOL = {"type": "function", "function": {"name": "cmp", "description": "is a < b & 'q' für?",
                                         "parameters": {"type": "object", "properties": {"z": {"type": "string"}, "a": {"type": "integer"}}, "required": ["z"]}}}


def test_tojson_is_plain_json():
    out = render_jinja("{{ tool | tojson(ensure_ascii=False) }}|{{ tool | tojson }}|{{ tool | tojson(ensure_ascii=True) }}", tool=TOOL)
    plain, default, ascii_only = out.split("|")
    assert plain == default == json.dumps(TOOL, ensure_ascii=False)  # keys in their given order ("z" before "a"), '<', '&', "'" and 'ü' as they are
    assert "\\u003c" not in plain and "&amp;" not in plain and '"z": {"type": "string"}, "a"' in plain
    assert ascii_only == json.dumps(TOOL, ensure_ascii=True) and "f\\u00fcr" in ascii_only
    assert render_jinja("{{ v | tojson(indent=2) }}", v={"b": 1, "a": [1, 2]}) == json.dumps({"b": 1, "a": [1, 2]}, indent=2)
    assert render_jinja("{{ v | tojson(sort_keys=True) }}", v={"b": 1, "a": 2}) == '{"a": 2, "b": 1}'
    # jinja2's own filter would have produced other bytes for the same value
    stock = jinja2.Environment().from_string("{{ tool | tojson }}").render(tool=TOOL)
    assert stock != plain and "\\u003c" in stock


def test_the_tools_block_of_a_template_equals_the_built_in_one():
    """The signature lines as the published template writes them (``tojson(ensure_ascii=False)`` per item of the signature)."""
    template = ("{% for tool in tools %}{% set f = tool.function if tool.function is defined else tool %}"
                "{\"name\": {{ f.name | tojson(ensure_ascii=False) }}, \"description\": {{ f.description | tojson(ensure_ascii=False) }}, "
                "\"parameters\": {{ f.parameters | tojson(ensure_ascii=False) }}}\n{% endfor %}")
    rendered = render_jinja(template, tools=[TOOL])
    built_in = chat_template.render([{"role": "user", "content": "q"}], tools=[TOOL])
    line = built_in.split("<tools>\n", 1)[1].split("</tools>", 1)[0]
    assert rendered == line == '{"name": "cmp", "description": "is a < b & \'q\' für?", "parameters": ' + json.dumps(TOOL["function"]["parameters"]) + "}\n"


def test_helpers_and_whitespace_control():
    with pytest.raises(jinja2.exceptions.TemplateError, match="no user message"):
        render_jinja("{% if not messages %}{{ raise_exception('no user message') }}{% endif %}", messages=[])
    year = render_jinja("{{ strftime_now('%Y') }}")
    assert len(year) == 4 and year.isdigit()
    text = render_jinja("{% for m in messages %}\n    {% if m == 'stop' %}{% break %}{% endif %}\n<{{ m }}>\n{% endfor %}\nend", messages=["a", "b", "stop", "c"])
    assert text == "<a>\n<b>\nend"  # block lines leave no blank lines or indentation behind (trim_blocks, lstrip_blocks); loop controls work
    assert render_jinja("{{ missing }}|{{ effort or 'max' }}", effort=None) == "|max"


def test_templates_run_in_a_sandbox():
    for hostile in ("{{ ''.__class__.__mro__ }}", "{{ messages.__class__.__base__.__subclasses__() }}", "{{ cycler.__init__.__globals__ }}"):
        with pytest.raises(jinja2.exceptions.SecurityError):
            render_jinja(hostile, messages=[])
    with pytest.raises(jinja2.exceptions.SecurityError):
        render_jinja("{% set _ = messages.append(1) %}", messages=[])  # a template may read the conversation, not change it
