"""Error types shared by every layer, grouped by who has to act on them.

* The operator: ``ConfigValidationError`` and its four kinds are raised while immutable inputs are read (model geometry, GPU inventory,
  layout or memory plan, checkpoint); they always mean "fix the input and start again", nothing was launched.
* The caller: ``RequestValidationError`` (a prepared request that does not satisfy the schema or the limits) and ``ApiError`` (the same for
  an OpenAI-style request, carrying the HTTP status and the error type of its JSON body).
* Nobody, any more: ``EngineFailure`` (a step lost its health vote; the engine that raised it answers no further request) and
  ``DeviceStatusError`` (a kernel left a non-zero status word: a bounded wait ran out, an index had to be clamped, a value was not finite).

Parity: reference ``glm_tpu/exceptions.py`` (same names for the validation errors and ``ApiError``).
"""

from __future__ import annotations


# ---------------------------------------------------------------------------------------------------------------------- caller
class RequestValidationError(ValueError):
    """A prepared request is malformed, too large, or pinned to other assets than the ones loaded."""


class ApiError(ValueError):
    """Refusal of an OpenAI-compatible request.  ``status`` is the HTTP status, ``kind`` the ``type`` of the error object."""

    def __init__(self, message: str, *, status: int = 400, kind: str = "invalid_request_error"):
        super().__init__(message)
        self.status, self.kind = status, kind

    def body(self) -> dict:
        return {"error": {"message": self.args[0], "type": self.kind, "param": None, "code": None}}


# ---------------------------------------------------------------------------------------------------------------------- operator
class ConfigValidationError(ValueError):
    """An immutable input is invalid; raised before anything runs."""


class GeometryValidationError(ConfigValidationError):
    """The model geometry is incomplete or contradicts itself."""


class TopologyValidationError(ConfigValidationError):
    """The GPU inventory is not the box the binding was made for."""


class PlanValidationError(ConfigValidationError):
    """A layout, memory or exchange plan breaks one of its stated invariants."""


class CheckpointValidationError(ConfigValidationError):
    """Checkpoint metadata, ownership or byte accounting does not reconcile."""


# ---------------------------------------------------------------------------------------------------------------------- terminal
class EngineFailure(RuntimeError):
    """A step failed its all-rank health vote; the engine is poisoned."""


class DeviceStatusError(RuntimeError):
    """A kernel reported through the status word.  ``status`` holds the bits."""

    def __init__(self, message: str, status: int = 0):
        super().__init__(message)
        self.status = status
