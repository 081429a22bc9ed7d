"""Registry of the ``GLM_B200_*`` environment variables, read lazily as module attributes.

``glm_tpu_b200.envs.GLM_B200_RUN_ROOT`` evaluates the variable when it is accessed, so tests can set the environment
after import.  Precedence everywhere: CLI flag > environment > site file > default.

Every variable is one row of ``TABLE``: a *kind* that names its parser in ``PARSERS`` (``path``, ``flag``, ``choice``,
``number``, ``count``), a default (a value, or a function for defaults that depend on other variables) and a help line.
There is one code path from a row to a value (``value_of``): look the text up, hand it to the kind's parser, fall back to
the default when it is unset or empty.  A text the parser refuses raises ``ValueError`` naming the variable, so a typo
never silently selects the default.

Parity: reference ``glm_tpu/envs.py:77-139`` (``GLM_TPU_*`` registry).
"""

from __future__ import annotations

import os
from pathlib import Path
from typing import Any, Callable, NamedTuple


class Row(NamedTuple):
    kind: str
    default: Any  # a value, or a zero-argument function evaluated when the variable is unset
    help: str
    choices: tuple = ()
    secret: bool = False


def _parse_path(text: str, row: Row) -> Path:
    if not os.path.isabs(text):
        raise ValueError("must be an absolute path")
    return Path(text)


def _parse_flag(text: str, row: Row) -> bool:
    if text not in ("0", "1"):
        raise ValueError("must be 0 or 1")
    return text == "1"


def _parse_choice(text: str, row: Row) -> str:
    if text not in row.choices:
        raise ValueError("must be one of " + ", ".join(row.choices))
    return text


def _parse_number(text: str, row: Row) -> float:
    number = float(text)
    if not number > 0:
        raise ValueError("must be a positive number")
    return number


PARSERS: dict[str, Callable[[str, Row], Any]] = {
    "path": _parse_path,
    "flag": _parse_flag,
    "choice": _parse_choice,
    "number": _parse_number,
    "count": lambda text, row: int(_parse_number(text, row)),
}


def _default_config_root() -> Path:
    xdg = os.environ.get("XDG_CONFIG_HOME", "")
    return Path(xdg if os.path.isabs(xdg) else Path.home() / ".config") / "glm-b200"


TABLE: dict[str, Row] = {
    "GLM_B200_CONFIG_ROOT": Row("path", _default_config_root, "Directory of site.toml (default $XDG_CONFIG_HOME/glm-b200 or ~/.config/glm-b200)."),
    "GLM_B200_SITE_CONFIG": Row("path", lambda: value_of("GLM_B200_CONFIG_ROOT") / "site.toml", "Explicit site file, absolute."),
    "GLM_B200_RUN_ROOT": Row("path", None, "Override of the site's paths.run_root."),
    "GLM_B200_MODEL_PATH": Row("path", None, "Override of paths.model_path (checkpoint and tokenizer)."),
    "GLM_B200_API_KEY_FILE": Row("path", None, "Bearer key file (0600) for /v1.", secret=True),
    "GLM_B200_COMM": Row("choice", "fused", "Cross-GPU path: in-kernel peer-memory collectives, or the NCCL baseline.", ("fused", "nccl")),
    "GLM_B200_CUDA_GRAPHS": Row("flag", True, "Replay the decode step from a CUDA graph (1) or launch eagerly (0)."),
    "GLM_B200_WAIT_LIMIT": Row("count", 2_000_000, "Iteration limit of every device-side wait on a peer flag."),
    # kernel-path switches for A/B runs: read where the path is chosen (ops/native.py, config/parallel.py, runner/gpu_runner.py,
    # models/glm_moe_dsa/), listed here so that the environment report shows them and refuses a value that would silently select
    # the default
    "GLM_B200_DECODE": Row("choice", "kernels", "Decode step: one kernel per operation, one per fused phase, or the persistent cooperative kernel.",
                           ("kernels", "phases", "mega")),
    "GLM_B200_EXPERT_SPLIT": Row("choice", "", "Routed experts per GPU: whole experts or a column slice of every expert (unset: sliced where the FP8 blocks allow).",
                                 ("", "whole", "sliced")),
    "GLM_B200_VOTE": Row("choice", "shm", "Host votes of the ranks of one box: through a memory-mapped file, or over the gloo process group.", ("shm", "gloo")),
    "GLM_B200_AR": Row("choice", "pairs", "In-kernel all-reduce: (value, sequence number) pairs, or values + fence + flag.", ("pairs", "flags")),
    "GLM_B200_MEGA_KSPLIT": Row("choice", "", "Fused decode phases: the stand-alone kernels' K decomposition (compat) or an even one (balanced).",
                                ("", "compat", "balanced")),
    "GLM_B200_MEGA_PREFETCH": Row("count", 24 << 20, "Persistent decode kernel: bytes of the next phases' weights asked into L2 ahead of time."),
    "GLM_B200_PDL": Row("flag", True, "Programmatic dependent launch between consecutive kernels (1) or plain stream order (0)."),
    "GLM_B200_OVERLAP": Row("flag", True, "Independent branches of a layer on a second stream (1) or one stream (0)."),
    "GLM_B200_FOLD_Q_POST": Row("flag", True, "Decode: query RoPE folded into q-absorb and the indexer (1) or a kernel of its own (0)."),
    "GLM_B200_MERGE_VPROJ": Row("flag", True, "Decode, local keys: chunk merge and value projection in one launch (1) or two (0)."),
    "GLM_B200_FEW_ROUTES": Row("count", 12, "Prefill chunks below this mean number of routes per expert run the routed experts on the GEMV kernels (8-route tiles)."),
    "GLM_B200_NVTX": Row("flag", False, "NVTX ranges per layer and block."),
    "GLM_B200_INDEXER": Row("choice", "tcgen05", "DSA indexer on tcgen05 or the CUDA-core kernel.", ("tcgen05", "cuda")),
    "GLM_B200_INDEXER_ROWS": Row("flag", True, "Prefill chunks: many-rows tcgen05 indexer (1) or the one-row kernel per row (0)."),
    "GLM_B200_PREFILL_ATTENTION": Row("choice", "rows", "Prefill attention: one kernel per row block, or split partials + merge.", ("rows", "split")),
    "GLM_B200_PREFILL_GEMM_AR": Row("choice", "fused", "Prefill o_proj / down projections: all-reduce inside the GEMM, or GEMM then NCCL.", ("fused", "nccl")),
    "GLM_B200_TEST_TIMEOUT_SCALE": Row("number", 1.0, "Tests: multiplier for subprocess timeouts."),
    "GLM_B200_TEST_WORLDS": Row("choice", "", "Tests: run the multi-GPU model test at this rank count only.", ("", "2", "4", "8")),
}


def value_of(name: str) -> Any:
    row = TABLE[name]
    text = os.environ.get(name, "")
    if text == "":
        return row.default() if callable(row.default) else row.default
    try:
        return PARSERS[row.kind](text, row)
    except ValueError as exc:
        raise ValueError(f"{name} {exc}") from None


def __getattr__(name: str) -> Any:
    if name in TABLE:
        return value_of(name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return sorted(TABLE)


def is_set(name: str) -> bool:
    TABLE[name]  # an unknown name is a KeyError, not "unset"
    return bool(os.environ.get(name))


def describe() -> dict[str, str]:
    """What the environment report shows: the parsed value of every variable that is set (secrets only as set/unset)."""

    def shown(name: str, row: Row) -> str:
        if not is_set(name):
            return "<unset>"
        if row.secret:
            return "<set>"
        try:
            return str(value_of(name))
        except ValueError as exc:  # a report lists a bad value, it does not die of it
            return f"<invalid: {exc}>"

    return {name: shown(name, row) for name, row in TABLE.items()}
