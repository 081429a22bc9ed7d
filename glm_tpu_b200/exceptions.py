"""Error types shared by every layer.

``ConfigValidationError`` and its subclasses are fail-closed refusals of an invalid immutable
input (geometry, device inventory, layout plan, checkpoint).  ``EngineFailure`` poisons an
engine.  ``ApiError`` is the refusal of an OpenAI-compatible request with its HTTP status.

Parity: reference ``glm_tpu/exceptions.py:6-33``.
"""

from __future__ import annotations


class ConfigValidationError(ValueError):
    pass


class GeometryValidationError(ConfigValidationError):
    pass


class TopologyValidationError(ConfigValidationError):
    pass


class PlanValidationError(ConfigValidationError):
    pass


class CheckpointValidationError(ConfigValidationError):
    pass


class RequestValidationError(ValueError):
    pass


class EngineFailure(RuntimeError):
    """A step failed its health vote; the engine that raised it refuses all later requests."""


class DeviceStatusError(RuntimeError):
    """A kernel reported a non-zero status word (a bounded wait ran out, or an index was clamped)."""

    def __init__(self, message: str, status: int = 0):
        super().__init__(message)
        self.status = status


class ApiError(ValueError):
    def __init__(self, message: str, *, status: int = 400, kind: str = "invalid_request_error"):
        super().__init__(message)
        self.status = status
        self.kind = kind

    def body(self) -> dict:
        return {"error": {"message": str(self), "type": self.kind, "param": None, "code": None}}
