"""Admission checks done before a program runs: memory projection and the collective plan.

``project_memory`` adds up what one GPU will hold (resident weights, caches for every lane, staging, workspaces)
and refuses a configuration that does not fit the device with a safety margin, before anything large is
allocated.  ``check_collective_plan`` validates the list of cross-GPU exchanges a program performs against the
rules the in-kernel protocol depends on (alternating all-reduce channels, every signal separated by an
all-reduce, payloads within the staging regions).

Parity: reference ``glm_tpu/runner/admission.py:6-89`` (``check_hlo_collectives`` on compiled HLO and
``project_memory``); here the plan is the engine's own launch list rather than parsed compiler output.
"""

from __future__ import annotations

from glm_tpu_b200.exceptions import PlanValidationError

HBM_BYTES = 183_359 * (1 << 20)  # what nvidia-smi reports for a B200
SAFETY_FRACTION = 0.94


def project_memory(geometry, layout, cache, weight_bytes: int, staging_bytes: int, hbm_bytes: int = HBM_BYTES) -> dict:
    g = geometry
    cache_bytes = cache.cache_bytes_per_gpu()
    rows = cache.lanes
    top_k_chunks = -(-g.index_top_k // 32)
    workspace = rows * (
        g.attention_heads * top_k_chunks * (g.kv_lora_rank + 2) * 4  # attention partials
        + cache.context_capacity * 4  # indexer scores
        + 16 * g.hidden_size * 4
        + g.routed_top_k * (g.hidden_size + g.moe_intermediate_size) * 2
        + layout.vocab_local * 2
    )
    total = weight_bytes + cache_bytes + staging_bytes + workspace
    out = {
        "weights": int(weight_bytes),
        "caches": int(cache_bytes),
        "staging": int(staging_bytes),
        "workspace": int(workspace),
        "total": int(total),
        "limit": int(hbm_bytes * SAFETY_FRACTION),
        "admitted": total <= hbm_bytes * SAFETY_FRACTION,
    }
    return out


def project_live(projection: dict, free_bytes: int, total_bytes: int, *, already_resident: int, reserve_bytes: int = 512 << 20) -> dict:
    """The projection against what the driver reports right now: what is still to be allocated (the projected total minus
    what is already resident, e.g. the weights) plus a reserve must fit into the free memory of the device."""
    to_allocate = max(0, projection["total"] - already_resident)
    out = dict(projection, device_free=int(free_bytes), device_total=int(total_bytes), to_allocate=int(to_allocate), reserve=int(reserve_bytes))
    out["admitted"] = bool(projection["admitted"]) and to_allocate + reserve_bytes <= free_bytes
    if not out["admitted"]:
        out["limit"] = min(projection["limit"], already_resident + max(0, free_bytes - reserve_bytes))
    return out


def require_admitted(projection: dict) -> None:
    if not projection["admitted"]:
        need, limit = projection["total"] / 2**30, projection["limit"] / 2**30
        raise PlanValidationError(f"memory admission refused: needs {need:.2f} GiB, limit {limit:.2f} GiB")


def check_collective_plan(plan: list[dict], *, world: int, ar_slice_floats: int = 256, ar_max_ctas: int = 1024) -> None:
    """``plan`` is the ordered list of exchanges of one program: ``{"kind": "allreduce", "channel": c, "ctas": n,
    "floats_per_cta": f}`` or ``{"kind": "signal", "signal": s}``."""
    if world == 1:
        return
    last_channel = None
    seen_since_ar: set[int] = set()
    for op in plan:
        if op["kind"] == "allreduce":
            if op["channel"] == last_channel:
                raise PlanValidationError("two consecutive all-reduces use the same channel")
            if op["ctas"] > ar_max_ctas or op["floats_per_cta"] > ar_slice_floats:
                raise PlanValidationError("all-reduce exceeds the per-CTA flag table or slice size")
            last_channel = op["channel"]
            seen_since_ar.clear()
        elif op["kind"] == "signal":
            if op["signal"] in seen_since_ar:
                raise PlanValidationError(f"signal {op['signal']} is raised twice without an all-reduce in between")
            seen_since_ar.add(op["signal"])
        else:
            raise PlanValidationError(f"unknown exchange kind {op['kind']!r}")
