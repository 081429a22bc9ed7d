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
    yield from more_oracle_mutants()


def more_oracle_mutants():
    """One mutant per further rule of the contract: roundings, orders of operations, tie rules, which tensor a term enters."""
    from glm_tpu_b200.oracle import contract as c

    F32 = torch.float32
    orig = {name: getattr(c, name) for name in (
        "linear", "add_rms_norm", "layer_norm_affine", "rope_interleaved_table", "rope_interleaved_fp32", "top_k_positions",
        "absorbed_attention_row", "swiglu_act", "router", "greedy", "dequantize_fp8", "rope_table", "indexer_scores", "sparse_moe")}

    def linear_no_round(x, weight, out_bf16=True):  # rule: a projection's output is rounded to bf16
        return orig["linear"](x, weight, out_bf16=False)

    def add_norm_on_rounded_sum(update, residual, weight, eps):  # rule: the norm consumes the UNROUNDED sum
        s = residual.to(F32) if update is None else update.to(F32) + residual.to(F32)
        return c.rms_norm(c.bf16_round(s), weight, eps), c.bf16_round(s)

    def add_norm_residual_unrounded(update, residual, weight, eps):  # rule: the carried residual is bf16
        s = residual.to(F32) if update is None else update.to(F32) + residual.to(F32)
        return c.rms_norm(s, weight, eps), s * (1.0 + 2.0**-10)

    def layer_norm_no_bias(x, weight, bias, eps):  # rule: the index key norm has a bias
        return orig["layer_norm_affine"](x, weight, torch.zeros_like(bias), eps)

    def layer_norm_biased_variance(x, weight, bias, eps):  # rule: eps sits inside the square root, variance over all features
        return orig["layer_norm_affine"](x, weight, bias, eps * 1e4)

    def rope_half_split(x, positions, table):  # rule: pairs are (2j, 2j+1), not (j, j + d/2)
        half = x.shape[-1] // 2
        rows = table[positions.long()].to(F32)
        shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
        cos, sin = rows[:, :half].reshape(shape), rows[:, half:].reshape(shape)
        x = x.to(F32)
        a, b = x[..., :half], x[..., half:]
        return c.bf16_round(torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1))

    def rope_wrong_sign(x, positions, table):  # rule: rotation by +angle
        flipped = table.clone()
        half = table.shape[-1] // 2
        flipped[:, half:] = -flipped[:, half:]
        return orig["rope_interleaved_table"](x, positions, flipped)

    def rope_table_unrounded_angle(capacity, dim, theta):  # rule: the table is built in fp32 with this frequency formula
        return orig["rope_table"](capacity, dim, theta * (1.0 + 2.0**-8))

    def indexer_rope_all_features(x, positions, theta, rope_dim):  # rule: only the first rope_dim features rotate
        return orig["rope_interleaved_fp32"](x, positions, theta, min(rope_dim * 2, x.shape[-1]))

    def top_k_ties_to_highest(scores, context_length, top_k):  # rule: ties go to the LOWEST position
        n = int(context_length)
        if n <= top_k:
            return torch.arange(n, dtype=torch.int64)
        key = c.orderable_key(scores[:n])
        order = torch.argsort(-key.flip(0), stable=True)
        return torch.sort((n - 1 - order)[:top_k]).values

    def top_k_one_short(scores, context_length, top_k):  # rule: exactly min(top_k, context) positions
        return orig["top_k_positions"](scores, context_length, max(top_k - 1, 1))

    def attention_p_not_rounded(q_c, q_rope, kv_rows, selected, scale):  # rule: P is rounded to bf16 before P.V, l sums unrounded P
        lora = q_c.shape[-1]
        if selected.numel() == 0:
            return torch.zeros_like(q_c)
        rows = kv_rows[selected.long()].to(F32)
        s = (q_c.to(F32) @ rows[:, :lora].T + q_rope.to(F32) @ rows[:, lora:].T) * scale
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        return c.bf16_round((p @ rows[:, :lora]) / p.sum(dim=-1, keepdim=True))

    def attention_l_from_rounded_p(q_c, q_rope, kv_rows, selected, scale):  # rule: the denominator sums the UNROUNDED probabilities
        lora = q_c.shape[-1]
        if selected.numel() == 0:
            return torch.zeros_like(q_c)
        rows = kv_rows[selected.long()].to(F32)
        s = (q_c.to(F32) @ rows[:, :lora].T + q_rope.to(F32) @ rows[:, lora:].T) * scale
        p = c.bf16_round(torch.exp(s - s.max(dim=-1, keepdim=True).values))
        return c.bf16_round((p @ rows[:, :lora]) / p.sum(dim=-1, keepdim=True))

    def attention_scale_on_nope_only(q_c, q_rope, kv_rows, selected, scale):  # rule: the scale multiplies latent AND rope dots
        return orig["absorbed_attention_row"](q_c, q_rope / max(scale, 1e-9), kv_rows, selected, scale)

    def attention_ignores_last_key(q_c, q_rope, kv_rows, selected, scale):  # rule: every selected row is attended
        return orig["absorbed_attention_row"](q_c, q_rope, kv_rows, selected[:-1] if selected.numel() > 1 else selected, scale)

    def swiglu_rounds_gate_activation(gate, up):  # rule: ONE rounding after the product
        return c.bf16_round(c.bf16_round(gate * torch.sigmoid(gate)) * up)

    def swiglu_swapped(gate, up):  # rule: the activation applies to the gate projection
        return orig["swiglu_act"](up, gate)

    def router_bias_in_weights(x, weight, bias, top_k, imposed=None):  # rule: the bias enters the choice only
        ids, _, choice = orig["router"](x, weight, bias, top_k, imposed)
        picked = torch.gather(choice, 1, ids)
        return ids, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20), choice

    def router_no_normalisation(x, weight, bias, top_k, imposed=None):  # rule: weights are normalised over the chosen experts
        ids, weights, choice = orig["router"](x, weight, bias, top_k, imposed)
        return ids, torch.gather(torch.sigmoid(x.to(F32) @ weight.to(F32).T), 1, ids), choice

    def router_softmax_scores(x, weight, bias, top_k, imposed=None):  # rule: sigmoid scores, not softmax
        logits = x.to(F32) @ weight.to(F32).T
        scores = torch.softmax(logits, dim=-1)
        choice = scores + bias.to(F32)[None, :]
        ids = torch.argsort(-c.orderable_key(choice), dim=-1, stable=True)[:, :top_k] if imposed is None else imposed.long()
        picked = torch.gather(scores, 1, ids)
        return ids, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20), choice

    def router_one_expert_less(x, weight, bias, top_k, imposed=None):  # rule: top_k experts
        ids, weights, choice = orig["router"](x, weight, bias, top_k, imposed)
        weights = weights.clone()
        weights[:, -1] = 0.0
        return ids, weights, choice

    def greedy_ties_to_highest(logits):  # rule: ties to the lowest id
        top = logits.max(dim=-1, keepdim=True).values
        ids = torch.arange(logits.shape[-1])[None, :].expand_as(logits)
        return torch.where(logits == top, ids, -1).max(dim=-1).values

    def greedy_second_best(logits):  # rule: the maximum
        return torch.topk(logits, 2, dim=-1).indices[:, 1]

    def dequant_transposed_blocks(bits, scale, block):  # rule: scale_inv[n // bn, k // bk]
        if scale.shape[-1] == scale.shape[-2] and scale.shape[-1] > 1:
            return orig["dequantize_fp8"](bits, scale.transpose(-1, -2).contiguous(), block)
        return orig["dequantize_fp8"](bits, scale * (1.0 + 2.0**-7), block)

    def dequant_unrounded(bits, scale, block):  # rule: bf16(f32(e4m3) * scale)
        return orig["dequantize_fp8"](bits, scale, block).float() * (1.0 - 2.0**-9)

    def indexer_without_relu(x, q_resid, w, layer, positions):  # rule: relu on the per-head dots before the weighted sum
        relu = torch.relu
        try:
            torch.relu = lambda t: t
            return orig["indexer_scores"](x, q_resid, w, layer, positions)
        finally:
            torch.relu = relu

    def indexer_keys_unrounded(x, q_resid, w, layer, positions):  # rule: the cached index keys are exactly bf16(rope(norm(.)))
        key, scores = orig["indexer_scores"](x, q_resid, w, layer, positions)
        return key * (1.0 + 2.0**-6), scores

    def moe_shared_dropped(x, w, layer, trace, imposed=None):  # rule: routed * factor + shared
        out = orig["sparse_moe"](x, w, layer, trace, imposed)
        return c.bf16_round(out * (1.0 - 2.0**-6))

    table = [
        ("linear: output not rounded to bf16", "linear", linear_no_round),
        ("add+norm: the norm consumes the rounded sum", "add_rms_norm", add_norm_on_rounded_sum),
        ("add+norm: the carried residual is not bf16", "add_rms_norm", add_norm_residual_unrounded),
        ("index key norm: bias dropped", "layer_norm_affine", layer_norm_no_bias),
        ("index key norm: eps 1e-2", "layer_norm_affine", layer_norm_biased_variance),
        ("rope: half-split pairing instead of interleaved", "rope_interleaved_table", rope_half_split),
        ("rope: rotation by the negative angle", "rope_interleaved_table", rope_wrong_sign),
        ("rope table: frequency base perturbed by 2^-8", "rope_table", rope_table_unrounded_angle),
        ("indexer rope: twice as many features rotate", "rope_interleaved_fp32", indexer_rope_all_features),
        ("top-k: ties to the highest position", "top_k_positions", top_k_ties_to_highest),
        ("top-k: one position short", "top_k_positions", top_k_one_short),
        ("attention: P not rounded to bf16", "absorbed_attention_row", attention_p_not_rounded),
        ("attention: denominator from the rounded P", "absorbed_attention_row", attention_l_from_rounded_p),
        ("attention: rope dots unscaled", "absorbed_attention_row", attention_scale_on_nope_only),
        ("attention: the last selected key ignored", "absorbed_attention_row", attention_ignores_last_key),
        ("swiglu: the activated gate rounded before the product", "swiglu_act", swiglu_rounds_gate_activation),
        ("swiglu: gate and up swapped", "swiglu_act", swiglu_swapped),
        ("router: bias enters the weights", "router", router_bias_in_weights),
        ("router: weights not normalised", "router", router_no_normalisation),
        ("router: softmax instead of sigmoid", "router", router_softmax_scores),
        ("router: the last chosen expert weighs nothing", "router", router_one_expert_less),
        ("sampler: ties to the highest id", "greedy", greedy_ties_to_highest),
        ("sampler: second best token", "greedy", greedy_second_best),
        ("fp8 decode: block scales transposed or perturbed", "dequantize_fp8", dequant_transposed_blocks),
        ("fp8 decode: result scaled by 1 - 2^-9", "dequantize_fp8", dequant_unrounded),
        ("indexer: no relu on the head dots", "indexer_scores", indexer_without_relu),
        ("indexer: cached keys perturbed by 2^-6", "indexer_scores", indexer_keys_unrounded),
        ("moe: block output scaled by 1 - 2^-6", "sparse_moe", moe_shared_dropped),
    ]
    for name, attr, fn in table:
        yield name, _patched(c, attr, fn)
    yield "index top-k 16 -> 8", _geometry_patch(index_top_k=8)
    yield "routed top-k one less", _geometry_patch(routed_top_k=max(1, _fixture_value("routed_top_k") - 1))


def _fixture_value(name: str):
    from tools.equivalence import fixture as fx

    return getattr(fx.fixture_geometry(), name)


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
    yield "inbox names with six digits", _patched(proto, "SEQUENCE_DIGITS", 6)
    yield "another marker in front of the run directory on stdout", _patched(proto, "STDOUT_RUN", "RUNDIR ")

    import struct

    from glm_tpu_b200.engine import outputs
    from glm_tpu_b200.engine import request as rq
    from glm_tpu_b200.entrypoints.openai import tool_parser
    from glm_tpu_b200.tokenizer import chat_template

    yield "prompt digest over big-endian ids", _patched(rq, "prompt_digest", lambda ids: __import__("hashlib").sha256(struct.pack(f">{len(ids)}i", *ids)).hexdigest())
    yield "request schema renamed", _patched(rq, "SCHEMA", "glm_b200_request_v2")
    yield "concurrent batches under the sequential schema name", _patched(rq, "CONCURRENT_SCHEMA", rq.BATCH_SCHEMA)
    plain_wire = outputs.TokenEvent.wire
    yield "token events without their index", _patched(outputs.TokenEvent, "wire", lambda self: {k: v for k, v in plain_wire(self).items() if k != "index"})
    yield "an answer is not cut at the next turn marker", _patched(outputs, "TURN_MARKERS", ())
    yield "tool-call arguments always as strings", _patched(tool_parser, "_typed", lambda raw: raw.strip())
    yield "tool-call blocks closed by another tag", _patched(tool_parser, "CLOSE", "</call>")
    yield "chat format: tool instructions without their last sentence", _patched(chat_template, "TOOLS_FOOTER", chat_template.TOOLS_FOOTER.split("\n\n")[0])
    plain_assistant = chat_template._assistant
    yield "chat format: earlier answers keep their surrounding whitespace", _patched(
        chat_template, "_assistant", lambda m, show_reasoning: plain_assistant(dict(m, content=" " + (m.get("content") or "") + " "), show_reasoning).replace(
            "</think>" + (m.get("content") or "").strip(), "</think> " + (m.get("content") or "") + " "))
    plain_visible = chat_template.visible_text
    yield "chat format: text parts joined by a newline", _patched(chat_template, "visible_text", lambda c: plain_visible(c) if isinstance(c, (str, type(None))) else "\n".join(
        plain_visible([p]) for p in c))


def default_mutants():
    """Changed defaults that no functional test would notice: each must change the production-defaults gate."""
    import dataclasses

    from glm_tpu_b200 import envs
    from glm_tpu_b200.config import site
    from glm_tpu_b200.engine import request as rq
    from glm_tpu_b200.entrypoints.openai import protocol as api
    from glm_tpu_b200.entrypoints.serve import http_handler, job_queue

    yield "eleven jobs may wait", _patched(job_queue, "PENDING", 11)
    yield "answers may be twice as long", _patched(rq, "MAX_NEW", 2 * rq.MAX_NEW)
    yield "the 128k profile admits its whole window as prompt", _patched(rq, "PROMPT_LIMITS", {**rq.PROMPT_LIMITS, rq.LONG_CAPACITY: rq.LONG_CAPACITY})
    yield "request bodies of 40 MB", _patched(api, "BODY_CAP", 40 << 20)
    yield "replies without the no-sniff header", _patched(http_handler, "SECURITY_HEADERS", tuple(h for h in http_handler.SECURITY_HEADERS if h[0] != "X-Content-Type-Options"))
    yield "a model alias for a medium effort", _patched(api, "ALIASES", dict(api.ALIASES, **{"glm-5.3-medium": "high"}))
    table = dict(envs.TABLE)
    table["GLM_B200_COMM"] = table["GLM_B200_COMM"]._replace(default="nccl")
    yield "the library collectives by default", _patched(envs, "TABLE", table)
    table = dict(envs.TABLE)
    table["GLM_B200_API_KEY_FILE"] = table["GLM_B200_API_KEY_FILE"]._replace(secret=False)
    yield "the key file's name no longer treated as a secret", _patched(envs, "TABLE", table)
    plain = site.SiteConfig
    yield "a site without a file launches strictly", _patched(site, "SiteConfig", dataclasses.make_dataclass(
        "SiteConfig", [("policy", str, dataclasses.field(default="strict"))], bases=(plain,), frozen=True))


def run() -> dict:
    """{mutant: caught?}.  Geometry mutants are skipped for digests that do not depend on the geometry."""
    import importlib

    from tools.equivalence import digests, wire

    base_oracle = digests.oracle_digests()
    results = {}
    for name, patch in oracle_mutants():
        with patch:
            results[name] = digests.oracle_digests() != base_oracle
    from tools.equivalence import defaults

    base_defaults = defaults.collect()
    for name, patch in default_mutants():
        with patch:
            results[name] = defaults.collect() != base_defaults
    assert defaults.collect() == base_defaults, "a mutant outlived its patch"
    base_wire = wire.collect()
    request_module = importlib.import_module("glm_tpu_b200.engine.request")
    for name, patch in wire_mutants():
        rebinds = "JSON" in name  # engine.request took the function by name when it was imported: it has to be imported again to see the mutant
        with patch:
            if rebinds:
                importlib.reload(request_module)
            try:
                results[name] = wire.collect() != base_wire
            except Exception:  # noqa: BLE001 - a mutant that makes the collection itself fail is caught as well
                results[name] = True
        if rebinds:
            importlib.reload(request_module)  # and once more without the mutant, before the next one is judged
    assert wire.collect() == base_wire, "a mutant outlived its patch"
    return results
