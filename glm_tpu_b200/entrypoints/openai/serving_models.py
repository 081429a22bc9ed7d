"""``GET /v1/models``: the one loaded model under its id and its reasoning-effort aliases, with the session's real
window, prompt and output ceilings and the server's request deadline, so that clients size requests correctly.

Parity: reference ``glm_tpu/entrypoints/openai/serving_models.py:12-49``.
"""

from __future__ import annotations

from glm_tpu_b200.entrypoints.openai.protocol import ALIASES, EFFORTS


class OpenAIServingModels:
    def __init__(self, *, capacity: int, wait_seconds: float, prompt_limit: int | None = None, max_new: int = 163840):
        self.capacity, self.wait_seconds = capacity, wait_seconds
        self.prompt_limit = prompt_limit if prompt_limit is not None else capacity
        self.max_new = max_new

    def models(self) -> dict:
        return {
            "object": "list",
            "data": [
                {
                    "id": name, "object": "model", "owned_by": "local", "created": 0,
                    "context_window": self.capacity,
                    "max_input_tokens": min(self.prompt_limit, self.capacity - 1),
                    "max_output_tokens": min(self.max_new, self.capacity - 1),
                    "request_deadline_seconds": self.wait_seconds,
                    "reasoning_effort": forced or "max",
                    "supports": {"tools": True, "streaming": True, "reasoning_effort": list(EFFORTS), "parallel_requests": False,
                                 "sampling": False},
                }
                for name, forced in ALIASES.items()
            ],
        }
