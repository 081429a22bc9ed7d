"""Tokenizer access for the front ends.

``load_tokenizer(path)`` returns an object with ``encode(text) -> list[int]``, ``decode(ids) -> str``,
``apply_chat_template(messages, tools=..., reasoning_effort=...) -> list[int]`` and ``files`` (name -> SHA-256 of the
tokenizer files it read, pinned into every prepared request):

* a checkpoint directory with ``tokenizer.json``: the Hugging Face fast tokenizer (``tokenizers`` library);
* no tokenizer files (fixtures, synthetic benchmarks): ``ByteTokenizer``, a reversible byte-level vocabulary with the
  chat format's special tokens, so every front end can be exercised offline.

Parity: reference ``glm_tpu/engine/request.py:180-212`` (``AutoTokenizer.apply_chat_template`` with pinned files),
``glm_tpu/config/model.py:269-282`` (``verified_template``).
"""

from __future__ import annotations

import hashlib
from pathlib import Path

from glm_tpu_b200.tokenizer import chat_template

SPECIAL_TOKENS = ("<|endoftext|>", "[MASK]", "[gMASK]", "[sMASK]", "<sop>", "<eop>", "<|system|>", "<|user|>", "<|assistant|>",
                  "<|observation|>", "<think>", "</think>", "<tool_call>", "</tool_call>", "<tool_response>", "</tool_response>",
                  "<arg_key>", "</arg_key>", "<arg_value>", "</arg_value>")


def _sha(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


class ByteTokenizer:
    """ids 0..255 are bytes; ids 256.. are the special tokens; the top of the vocabulary holds the EOS ids."""

    def __init__(self, vocab_size: int = 1024, eos_ids: tuple = ()):
        if vocab_size < 256 + len(SPECIAL_TOKENS):
            raise ValueError("vocabulary too small for the byte tokenizer")
        self.vocab_size = vocab_size
        self.special = {tok: 256 + i for i, tok in enumerate(SPECIAL_TOKENS)}
        self.special_rev = {v: k for k, v in self.special.items()}
        self.eos_ids = tuple(eos_ids)
        self.files: dict = {}
        self.template_sha256 = hashlib.sha256(Path(chat_template.__file__).read_bytes()).hexdigest()

    def encode(self, text: str) -> list[int]:
        ids, i = [], 0
        while i < len(text):
            for tok, tid in self.special.items():
                if text.startswith(tok, i):
                    ids.append(tid)
                    i += len(tok)
                    break
            else:
                ids.extend(text[i].encode("utf-8"))
                i += 1
        return ids

    def decode(self, ids) -> str:
        out, buf = [], bytearray()
        for t in ids:
            if 0 <= t < 256:
                buf.append(t)
                continue
            if buf:
                out.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            if t in self.special_rev:
                out.append(self.special_rev[t])
            elif t in self.eos_ids:
                out.append("<|endoftext|>")
            else:
                out.append(f"<0x{t:X}>")
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def apply_chat_template(self, messages, *, tools=None, reasoning_effort=None, add_generation_prompt=True) -> list[int]:
        return self.encode(chat_template.render(messages, tools=tools, reasoning_effort=reasoning_effort,
                                                add_generation_prompt=add_generation_prompt))


def render_jinja(template: str, **variables) -> str | None:
    """``template`` (a checkpoint's ``chat_template.jinja``) rendered the way the model's own tooling renders it: sandboxed,
    ``trim_blocks`` / ``lstrip_blocks`` on, loop controls, and the three helpers such templates rely on.  ``tojson`` is plain
    ``json.dumps`` -- keys in their given order, text as it is (``ensure_ascii=False``), no HTML escaping -- and NOT jinja2's own filter,
    which sorts keys and writes ``<`` as ``\\u003c``: with that one a tool signature would reach the model in other bytes than
    the ones it was trained on.  ``None`` when jinja2 is not installed."""
    try:
        from jinja2.exceptions import TemplateError
        from jinja2.sandbox import ImmutableSandboxedEnvironment
    except ImportError:
        return None
    import datetime
    import json

    def tojson(value, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
        return json.dumps(value, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

    def raise_exception(message):
        raise TemplateError(message)

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
    env.filters["tojson"] = tojson
    env.globals["raise_exception"] = raise_exception
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    return env.from_string(template).render(**variables)


class HfTokenizer:
    def __init__(self, path: Path):
        from tokenizers import Tokenizer

        self.path = Path(path)
        self._tok = Tokenizer.from_file(str(self.path / "tokenizer.json"))
        self.vocab_size = self._tok.get_vocab_size()
        self.files = {name: _sha(self.path / name) for name in ("tokenizer.json", "tokenizer_config.json") if (self.path / name).exists()}
        jinja = self.path / "chat_template.jinja"
        self._jinja = jinja.read_text(encoding="utf-8") if jinja.exists() else None
        self.template_sha256 = _sha(jinja) if jinja.exists() else hashlib.sha256(Path(chat_template.__file__).read_bytes()).hexdigest()

    def encode(self, text: str) -> list[int]:
        return self._tok.encode(text, add_special_tokens=False).ids

    def decode(self, ids) -> str:
        return self._tok.decode(list(ids), skip_special_tokens=False)

    def apply_chat_template(self, messages, *, tools=None, reasoning_effort=None, add_generation_prompt=True) -> list[int]:
        text = None
        if self._jinja is not None:
            text = render_jinja(self._jinja, messages=messages, tools=tools, reasoning_effort=reasoning_effort,
                                add_generation_prompt=add_generation_prompt)
        if text is None:
            text = chat_template.render(messages, tools=tools, reasoning_effort=reasoning_effort,
                                        add_generation_prompt=add_generation_prompt)
        return self.encode(text)


def load_tokenizer(path=None, *, vocab_size: int = 1024, eos_ids: tuple = ()):
    if path is not None and (Path(path) / "tokenizer.json").exists():
        return HfTokenizer(Path(path))
    return ByteTokenizer(vocab_size, eos_ids)
