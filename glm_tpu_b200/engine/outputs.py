"""What the engine emits.

``TokenEvent`` is the record of one generated token; its ``wire()`` form is one line of ``tokens.jsonl`` (``batch_round`` appears only
when several chats decode together).  ``final_channel`` splits generated text into the model's reasoning and its answer: GLM opens its
output with a ``<think>`` section, the answer follows ``</think>`` and ends at the first marker that would start another turn.

Behaviour parity: reference ``glm_tpu/engine/outputs.py`` (same event fields, same split).
"""

from __future__ import annotations

from dataclasses import dataclass

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
TURN_MARKERS = ("<|user|>", "<|endoftext|>", "<|observation|>")


@dataclass(frozen=True)
class TokenEvent:
    request_id: str
    index: int
    token_id: int
    finish_reason: str | None
    batch_round: int | None = None

    def wire(self) -> dict:
        record = {"request_id": self.request_id, "index": self.index, "token_id": self.token_id, "finish_reason": self.finish_reason}
        if self.batch_round is not None:
            record["batch_round"] = self.batch_round
        return record


def _without_opening_tag(reasoning: str) -> str:
    return (reasoning[len(THINK_OPEN):] if reasoning.startswith(THINK_OPEN) else reasoning).strip()


def final_channel(text: str) -> tuple[str, str]:
    """``(reasoning, answer)``.  Text whose reasoning section has not been closed yet is all reasoning."""
    reasoning, closed, rest = text.partition(THINK_CLOSE)
    if not closed:
        return _without_opening_tag(text), ""
    cut = min((at for at in (rest.find(marker) for marker in TURN_MARKERS) if at >= 0), default=len(rest))
    return _without_opening_tag(reasoning), rest[:cut].strip()
