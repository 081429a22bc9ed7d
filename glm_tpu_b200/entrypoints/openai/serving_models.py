"""``GET /v1/models``.

One model is loaded; it is listed once per name it answers to (its id, plus the aliases that fix the reasoning effort for clients that
can only choose a model name).  Each entry tells a client what the LOADED session can take, not what the architecture could: the context
window of the session, the largest prompt and the largest answer that fit it, and the deadline after which the server gives up on a
request, so that clients compact their history and set their expectations against real limits.

Behaviour parity: reference ``glm_tpu/entrypoints/openai/serving_models.py`` (same entry fields).
"""

from __future__ import annotations

from dataclasses import dataclass

from glm_tpu_b200.entrypoints.openai.protocol import ALIASES, EFFORTS

CAPABILITIES = {"tools": True, "streaming": True, "parallel_requests": False, "sampling": False}


@dataclass(frozen=True)
class SessionLimits:
    window: int          # context slots of the loaded session
    longest_prompt: int  # prompt ceiling of its profile
    longest_answer: int  # output ceiling of the engine
    deadline: float      # seconds the server waits for one request

    def entry(self, name: str, forced_effort: str | None) -> dict:
        room = self.window - 1  # at least one slot is the other side's
        supports = {"tools": CAPABILITIES["tools"], "streaming": CAPABILITIES["streaming"], "reasoning_effort": list(EFFORTS),
                    "parallel_requests": CAPABILITIES["parallel_requests"], "sampling": CAPABILITIES["sampling"]}
        return {"id": name, "object": "model", "owned_by": "local", "created": 0, "context_window": self.window,
                "max_input_tokens": min(self.longest_prompt, room), "max_output_tokens": min(self.longest_answer, room),
                "request_deadline_seconds": self.deadline, "reasoning_effort": forced_effort or "max", "supports": supports}


class OpenAIServingModels:
    def __init__(self, *, capacity: int, wait_seconds: float, prompt_limit: int | None = None, max_new: int = 163840):
        self.limits = SessionLimits(capacity, capacity if prompt_limit is None else prompt_limit, max_new, wait_seconds)

    def models(self) -> dict:
        return {"object": "list", "data": [self.limits.entry(name, forced) for name, forced in ALIASES.items()]}
