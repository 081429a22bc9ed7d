"""Registry of the ``GLM_B200_*`` environment variables, read lazily as module attributes.

``glm_tpu_b200.envs.GLM_B200_RUN_ROOT`` evaluates the variable when it is accessed, so tests can
set the environment after import.  Precedence everywhere: CLI flag > environment > site file > default.

Parity: reference ``glm_tpu/envs.py:77-139`` (``GLM_TPU_*`` registry).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable


@dataclass(frozen=True)
class EnvVar:
    getter: Callable[[], Any]
    help: str
    secret: bool = False


def _abs_path(name: str):
    value = os.environ.get(name, "")
    if not value:
        return None
    if not os.path.isabs(value):
        raise ValueError(f"{name} must be an absolute path")
    return Path(value)


def _config_root() -> Path:
    explicit = _abs_path("GLM_B200_CONFIG_ROOT")
    if explicit is not None:
        return explicit
    xdg = os.environ.get("XDG_CONFIG_HOME", "")
    base = xdg if os.path.isabs(xdg) else os.path.join(os.path.expanduser("~"), ".config")
    return Path(base) / "glm-b200"


def _positive(name: str, default: float) -> float:
    value = os.environ.get(name, "")
    if not value:
        return default
    number = float(value)
    if not number > 0:
        raise ValueError(f"{name} must be a positive number")
    return number


def _flag(name: str, default: bool = False) -> bool:
    value = os.environ.get(name, "")
    if not value:
        return default
    if value not in ("0", "1"):
        raise ValueError(f"{name} must be 0 or 1")
    return value == "1"


def _choice(name: str, allowed: tuple[str, ...]) -> str:
    value = os.environ.get(name, "")
    if not value:
        return allowed[0]
    if value not in allowed:
        raise ValueError(f"{name} must be one of {', '.join(allowed)}")
    return value


environment_variables: dict[str, EnvVar] = {
    "GLM_B200_CONFIG_ROOT": EnvVar(_config_root, "Directory of site.toml (default $XDG_CONFIG_HOME/glm-b200 or ~/.config/glm-b200)."),
    "GLM_B200_SITE_CONFIG": EnvVar(
        lambda: _abs_path("GLM_B200_SITE_CONFIG") or _config_root() / "site.toml", "Explicit site file, absolute."
    ),
    "GLM_B200_RUN_ROOT": EnvVar(lambda: _abs_path("GLM_B200_RUN_ROOT"), "Override of the site's paths.run_root."),
    "GLM_B200_MODEL_PATH": EnvVar(lambda: _abs_path("GLM_B200_MODEL_PATH"), "Override of paths.model_path (checkpoint and tokenizer)."),
    "GLM_B200_COMM": EnvVar(
        lambda: os.environ.get("GLM_B200_COMM") or "fused",
        "Cross-GPU path: 'fused' (in-kernel peer-memory collectives) or 'nccl' (baseline).",
    ),
    "GLM_B200_CUDA_GRAPHS": EnvVar(lambda: _flag("GLM_B200_CUDA_GRAPHS", True), "Replay the decode step from a CUDA graph (1) or launch eagerly (0)."),
    "GLM_B200_WAIT_LIMIT": EnvVar(
        lambda: int(_positive("GLM_B200_WAIT_LIMIT", 20_000_000)), "Iteration limit of every device-side wait on a peer flag."
    ),
    # kernel-path switches for A/B runs: read where the path is chosen (ops/native.py, models/glm_moe_dsa/model.py), listed here
    # so that the environment report shows them and refuses a value that would silently select the default
    "GLM_B200_PDL": EnvVar(lambda: _flag("GLM_B200_PDL", True), "Programmatic dependent launch between consecutive kernels (1) or plain stream order (0)."),
    "GLM_B200_OVERLAP": EnvVar(lambda: _flag("GLM_B200_OVERLAP", True), "Independent branches of a layer on a second stream (1) or one stream (0)."),
    "GLM_B200_FOLD_Q_POST": EnvVar(lambda: _flag("GLM_B200_FOLD_Q_POST", True), "Decode: query RoPE folded into q-absorb and the indexer (1) or a kernel of its own (0)."),
    "GLM_B200_NVTX": EnvVar(lambda: _flag("GLM_B200_NVTX", False), "NVTX ranges per layer and block."),
    "GLM_B200_INDEXER": EnvVar(lambda: _choice("GLM_B200_INDEXER", ("tcgen05", "cuda")), "DSA indexer on tcgen05 or the CUDA-core kernel."),
    "GLM_B200_INDEXER_ROWS": EnvVar(lambda: _flag("GLM_B200_INDEXER_ROWS", True), "Prefill chunks: many-rows tcgen05 indexer (1) or the one-row kernel per row (0)."),
    "GLM_B200_ROUTE_SORT": EnvVar(lambda: _choice("GLM_B200_ROUTE_SORT", ("kernel", "torch")), "Prefill expert sort: one launch or library operations."),
    "GLM_B200_PREFILL_ATTENTION": EnvVar(lambda: _choice("GLM_B200_PREFILL_ATTENTION", ("rows", "split")), "Prefill attention: one kernel per row block, or split partials + merge."),
    "GLM_B200_PREFILL_GEMM_AR": EnvVar(lambda: _choice("GLM_B200_PREFILL_GEMM_AR", ("fused", "nccl")), "Prefill o_proj / down projections: all-reduce inside the GEMM, or GEMM then NCCL."),
    "GLM_B200_API_KEY_FILE": EnvVar(lambda: _abs_path("GLM_B200_API_KEY_FILE"), "Bearer key file (0600) for /v1.", secret=True),
    "GLM_B200_TEST_TIMEOUT_SCALE": EnvVar(lambda: _positive("GLM_B200_TEST_TIMEOUT_SCALE", 1.0), "Tests: multiplier for subprocess timeouts."),
}


def __getattr__(name: str) -> Any:
    if name in environment_variables:
        return environment_variables[name].getter()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return list(environment_variables)


def is_set(name: str) -> bool:
    if name not in environment_variables:
        raise KeyError(name)
    return name in os.environ


def describe() -> dict[str, str]:
    out = {}
    for name, var in environment_variables.items():
        if var.secret:
            out[name] = "<set>" if name in os.environ else "<unset>"
        else:
            try:
                out[name] = str(var.getter()) if name in os.environ else "<unset>"
            except ValueError as exc:  # an environment report lists a bad value, it does not die of it
                out[name] = f"<invalid: {exc}>"
    return out
