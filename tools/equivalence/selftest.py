"""G14: mutation self-test.  Each mutant changes one rule of the numerical contract or of a wire format; the corresponding gate
must notice.  A mutant that leaves every digest unchanged means the fixture (or the gate) is blind to that rule.
"""

from __future__ import annotations

import contextlib

import torch


@contextlib.contextmanager
def _patched(obj, name, value):
    old = getattr(obj, name)
    setattr(obj, name, value)
    try:
        yield
    finally:
        setattr(obj, name, old)


def oracle_mutants():
    """(name, context manager) pairs that break one contract rule each."""
    from glm_tpu_b200.oracle import contract as c

    def rms_weight_before_round(x, weight, eps):  # rule: round to bf16, THEN multiply by the weight
        xf = x.float()
        inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return c.bf16_round(xf * inv * weight.float())

    def top_k_skips_best(scores, context_length, top_k):  # rule: the top_k BEST positions are kept
        n = int(context_length)
        if n <= top_k:
            return torch.arange(n, dtype=torch.int64)
        order = torch.argsort(-c.orderable_key(scores[:n]), stable=True)
        return torch.sort(order[1 : top_k + 1]).values

    def dequant_no_round(bits, scale, block):  # rule: the decoded weight is rounded to bf16
        out = c_dequant(bits, scale, block)
        return out.float() * (1.0 + 2.0**-9)

    c_dequant = c.dequantize_fp8
    yield "rms_norm: weight applied before the bf16 rounding", _patched(c, "rms_norm", rms_weight_before_round)
    yield "top-k: the best position dropped", _patched(c, "top_k_positions", top_k_skips_best)
    yield "fp8 decode: scale perturbed by 2^-9", _patched(c, "dequantize_fp8", dequant_no_round)
    yield "routed scaling factor 2.5 -> 2.0", _geometry_patch(routed_scaling_factor=2.0)
    yield "rope theta halved", _geometry_patch(rope_theta=4000000.0)
    yield "rms eps x10", _geometry_patch(rms_norm_eps=1e-4)


def _geometry_patch(**changes):
    import dataclasses

    from tools.equivalence import fixture as fx

    original = fx.fixture_geometry
    return _patched(fx, "fixture_geometry", lambda: dataclasses.replace(original(), **changes))


def wire_mutants():
    from glm_tpu_b200.engine import resident_protocol as proto
    from glm_tpu_b200.utils import json_utils

    compact = json_utils.canonical_wire_bytes

    def spaced(value):
        return compact(value).replace(b",", b", ")

    yield "canonical JSON with spaces after commas", _patched(json_utils, "canonical_wire_bytes", spaced)
    yield "tokens file renamed", _patched(proto, "TOKENS_FILE", "tokens.ndjson")


def run() -> dict:
    """{mutant: caught?}.  Geometry mutants are skipped for digests that do not depend on the geometry."""
    import importlib

    from tools.equivalence import digests, wire

    base_oracle = digests.oracle_digests()
    results = {}
    for name, patch in oracle_mutants():
        with patch:
            results[name] = digests.oracle_digests() != base_oracle
    base_wire = wire.collect()
    for name, patch in wire_mutants():
        with patch:
            importlib.reload(importlib.import_module("glm_tpu_b200.engine.request")) if "JSON" in name else None
            results[name] = wire.collect() != base_wire
    importlib.reload(importlib.import_module("glm_tpu_b200.engine.request"))
    return results
