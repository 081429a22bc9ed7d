"""Constants of the OpenAI-compatible surface and the error type it answers with.

Parity: reference ``glm_tpu/entrypoints/openai/protocol.py:8-14``.
"""

from glm_tpu_b200.engine.request import MESSAGES_CAP
from glm_tpu_b200.exceptions import ApiError

__all__ = ["ApiError", "MODEL_NAME", "ALIASES", "EFFORTS", "MESSAGES_CAP", "TOOLS_CAP", "BODY_CAP"]

MODEL_NAME = "glm-5.3"
EFFORTS = ("low", "high", "max")
# model id -> reasoning effort it forces (None: the request's own ``reasoning_effort``, default max)
ALIASES = {MODEL_NAME: None, MODEL_NAME + "-low": "low", MODEL_NAME + "-high": "high"}
TOOLS_CAP = 256 << 10
BODY_CAP = 4 << 20
