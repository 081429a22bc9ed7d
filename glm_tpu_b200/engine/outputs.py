"""What the engine emits: one ``TokenEvent`` per generated token (a wire format: one JSON object per line in
``tokens.jsonl``) and the split of the generated text into reasoning and final answer.

Parity: reference ``glm_tpu/engine/outputs.py:10-23``.
"""

from __future__ import annotations

import re
from dataclasses import asdict, dataclass

_STOP_MARKERS = re.compile(r"<\|(?:user|endoftext|observation)\|>")


@dataclass(frozen=True)
class TokenEvent:
    request_id: str
    index: int
    token_id: int
    finish_reason: str | None
    batch_round: int | None = None  # only in concurrent mode

    def wire(self) -> dict:
        out = asdict(self)
        if self.batch_round is None:
            del out["batch_round"]
        return out


def final_channel(text: str) -> tuple[str, str]:
    """``(thinking, answer)``: everything before ``</think>`` is reasoning; the answer stops at the next turn marker."""
    if "</think>" not in text:
        return text.removeprefix("<think>").strip(), ""
    thinking, answer = text.split("</think>", 1)
    answer = _STOP_MARKERS.split(answer, maxsplit=1)[0]
    return thinking.removeprefix("<think>").strip(), answer.strip()
