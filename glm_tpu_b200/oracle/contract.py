"""CPU restatement of the model with every rounding boundary of the engine ("contract reference").

Each function restates one operation in plain PyTorch: bf16 operands are widened to fp32, every
contraction accumulates in fp32 and every activation that crosses an operation boundary is rounded to
bf16, exactly where the CUDA kernels round.  ``forward`` runs a whole sequence at once: row ``p``'s
selection, routes and attention depend only on rows ``<= p``, so row ``p`` is what an incremental engine
computes for position ``p`` under any prefill partition or decode step.

Semantics follow the reference's unsharded restatements (``tests/reference/independent.py:104-356``,
``tests/reference/model.py:293-362``) and the rounding rules of its layers (``glm_tpu/layers/norm.py:55-122``,
``layers/rope.py:41-56,145-199``, ``layers/fp8.py:113-126``, ``layers/moe/router.py:40-55``,
``layers/moe/routed_experts.py:279-304``, ``layers/sampler.py:46-99``, ``kernels/sparse_mla/kernel.py:148-183``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping

import numpy as np
import torch

from glm_tpu_b200.config.model import ModelGeometry

BF16 = torch.bfloat16
F32 = torch.float32
_FP8_ABLE = ("q_a_proj", "kv_a_proj_with_mqa", "q_b_proj", "kv_b_proj", "o_proj", "wq_b", "wk", "gate_proj", "up_proj", "down_proj")


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """Round an fp32 tensor to bf16 (nearest even) and widen it back."""
    return x.to(F32).to(BF16).to(F32)


# --------------------------------------------------------------------------- FP8
def dequantize_fp8(bits: torch.Tensor, scale_inv: torch.Tensor, block: tuple[int, int] = (128, 128)) -> torch.Tensor:
    """``bf16(f32(e4m3fn(bits)) * scale_inv[n // bn, k // bk])`` for ``bits [..., N, K]`` (uint8)."""
    values = bits.contiguous().view(torch.float8_e4m3fn).to(F32)
    bn, bk = block
    scale = scale_inv.to(F32).repeat_interleave(bn, dim=-2).repeat_interleave(bk, dim=-1)
    scale = scale[..., : values.shape[-2], : values.shape[-1]]
    return (values * scale).to(BF16)


def linear(x: torch.Tensor, weight: torch.Tensor, out_bf16: bool = True) -> torch.Tensor:
    """``x @ weight.T`` with bf16 operands widened to fp32 and fp32 accumulation."""
    y = x.to(F32) @ weight.to(F32).T
    return bf16_round(y) if out_bf16 else y


# --------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 mean square; ``bf16(x * rsqrt(ms + eps))`` then ``bf16(. * weight)``."""
    x = x.to(F32)
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return bf16_round(bf16_round(x * inv) * weight.to(F32))


def add_rms_norm(update, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """``s = f32(update) + f32(residual)``; the norm consumes the unrounded sum; the carried residual is ``bf16(s)``."""
    s = residual.to(F32) if update is None else update.to(F32) + residual.to(F32)
    return rms_norm(s, weight, eps), bf16_round(s)


def layer_norm_affine(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F32)
    mean = x.mean(dim=-1, keepdim=True)
    var = (x - mean).pow(2).mean(dim=-1, keepdim=True)
    return (x - mean) * torch.rsqrt(var + eps) * weight.to(F32) + bias.to(F32)


# --------------------------------------------------------------------------- RoPE
def rope_table(capacity: int, dim: int, theta: float) -> torch.Tensor:
    """``[capacity, dim]`` bf16 table ``cos | sin`` built with NumPy fp32 (frequency, angle, cos/sin all fp32)."""
    j = np.arange(0, dim, 2, dtype=np.float32)
    inv_freq = (np.float32(1.0) / np.power(np.float32(theta), j / np.float32(dim))).astype(np.float32)
    angle = np.arange(capacity, dtype=np.float32)[:, None] * inv_freq[None, :]
    table = np.concatenate([np.cos(angle), np.sin(angle)], axis=1).astype(np.float32)
    return torch.from_numpy(table).to(BF16)


def rope_interleaved_table(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Rotate pairs ``(2j, 2j+1)`` of ``x[rows, ..., dim]`` with the bf16 table; fp32 products, one bf16 round."""
    half = x.shape[-1] // 2
    rows = table[positions.long()].to(F32)
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
    cos, sin = rows[:, :half].reshape(shape), rows[:, half:].reshape(shape)
    x = x.to(F32)
    even, odd = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = even * cos - odd * sin
    out[..., 1::2] = odd * cos + even * sin
    return bf16_round(out)


def rope_interleaved_fp32(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: int) -> torch.Tensor:
    """Indexer RoPE: fp32 ``cos/sin(position * theta**(-2j/rope_dim))`` on the first ``rope_dim`` features; stays fp32."""
    j = torch.arange(0, rope_dim, 2, dtype=F32)
    inv_freq = torch.pow(torch.tensor(theta, dtype=F32), -j / rope_dim)
    angle = positions.to(F32)[:, None] * inv_freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (rope_dim // 2,)
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    x = x.to(F32).clone()
    even, odd = x[..., 0:rope_dim:2].clone(), x[..., 1:rope_dim:2].clone()
    x[..., 0:rope_dim:2] = even * cos - odd * sin
    x[..., 1:rope_dim:2] = odd * cos + even * sin
    return x


# --------------------------------------------------------------------------- top-k
def orderable_key(scores: torch.Tensor) -> torch.Tensor:
    """Map fp32 to int64 keys whose integer order is the total fp32 order (``-0 < +0``)."""
    bits = scores.to(F32).contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    negative = bits >> 31 == 1
    return torch.where(negative, 0xFFFFFFFF - bits, bits + 0x80000000)


def top_k_positions(scores: torch.Tensor, context_length: int, top_k: int) -> torch.Tensor:
    """Ascending list of the ``min(top_k, context_length)`` best positions of ``scores[:context_length]``."""
    n = int(context_length)
    if n <= top_k:
        return torch.arange(n, dtype=torch.int64)
    key = orderable_key(scores[:n])
    order = torch.argsort(-key, stable=True)  # descending key; stable => lowest position first among ties
    return torch.sort(order[:top_k]).values


# --------------------------------------------------------------------------- weights view
@dataclass
class OracleWeights:
    """bf16-resident view of a runtime-layout checkpoint (FP8 pairs decoded with the contract formula)."""

    geometry: ModelGeometry
    tensors: dict[str, torch.Tensor]

    @classmethod
    def from_checkpoint(cls, geometry: ModelGeometry, arrays: Mapping[str, torch.Tensor]) -> "OracleWeights":
        out: dict[str, torch.Tensor] = {}
        for name, value in arrays.items():
            if name.endswith(".scale_inv"):
                continue
            if name.endswith(".weight_bits"):
                prefix = name[: -len(".weight_bits")]
                out[prefix] = dequantize_fp8(value.cpu(), arrays[prefix + ".scale_inv"].cpu(), geometry.fp8_block_shape)
            elif name.endswith(".weight") and name.split(".")[-2] in _FP8_ABLE:
                out[name[: -len(".weight")]] = value.cpu()  # a projection stored in bf16
            else:
                out[name] = value.cpu()
        return cls(geometry, out)

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.tensors[name]


@dataclass
class Trace:
    logits: torch.Tensor  # [rows, vocab] bf16-rounded fp32
    tokens: torch.Tensor  # [rows] greedy argmax (lowest id on ties)
    residual: torch.Tensor
    selected: list = field(default_factory=list)  # per layer: list over rows of ascending position tensors
    index_scores: dict = field(default_factory=dict)  # full layer -> [rows, rows] fp32 (-inf above diagonal)
    expert_ids: dict = field(default_factory=dict)  # sparse layer -> [rows, k]
    route_weights: dict = field(default_factory=dict)
    router_choice: dict = field(default_factory=dict)
    layer_outputs: list = field(default_factory=list)  # hidden update of each block pair (attn, mlp)
    kv_rows: list = field(default_factory=list)  # per layer [rows, kv_row_width]
    index_keys: dict = field(default_factory=dict)


# --------------------------------------------------------------------------- blocks
def attention_inputs(x, w: OracleWeights, layer: int, positions, table):
    g = w.geometry
    a = f"model.layers.{layer}.self_attn"
    q_resid = rms_norm(linear(x, w[a + ".q_a_proj"]), w[a + ".q_a_layernorm.weight"], g.rms_norm_eps)
    q = linear(q_resid, w[a + ".q_b_proj"]).reshape(x.shape[0], g.attention_heads, g.qk_head_dim)
    q_nope = q[..., : g.qk_nope_head_dim]
    q_rope = rope_interleaved_table(q[..., g.qk_nope_head_dim :], positions, table)
    compressed = linear(x, w[a + ".kv_a_proj_with_mqa"])
    latent = rms_norm(compressed[:, : g.kv_lora_rank], w[a + ".kv_a_layernorm.weight"], g.rms_norm_eps)
    k_rope = rope_interleaved_table(compressed[:, g.kv_lora_rank :], positions, table)
    return q_resid, q_nope, q_rope, latent, k_rope


def indexer_scores(x, q_resid, w: OracleWeights, layer: int, positions):
    """``(keys bf16 [rows, d], scores fp32 [rows, rows])``; scores above the diagonal are -inf."""
    g = w.geometry
    p = f"model.layers.{layer}.self_attn.indexer"
    rows = x.shape[0]
    key = layer_norm_affine(linear(x, w[p + ".wk"], out_bf16=False), w[p + ".k_norm.weight"], w[p + ".k_norm.bias"], 1e-6)
    key = bf16_round(rope_interleaved_fp32(key, positions, g.rope_theta, g.qk_rope_head_dim))
    query = linear(q_resid, w[p + ".wq_b"], out_bf16=False).reshape(rows, g.index_heads, g.index_head_dim)
    query = rope_interleaved_fp32(query, positions, g.rope_theta, g.qk_rope_head_dim)
    head_w = linear(x, w[p + ".weights_proj.weight"], out_bf16=False) * (g.index_heads**-0.5)
    dots = torch.einsum("shd,td->sht", query, key) * (g.index_head_dim**-0.5)
    scores = torch.einsum("sh,sht->st", head_w, torch.relu(dots))
    causal = torch.arange(rows)[None, :] <= torch.arange(rows)[:, None]
    return key, torch.where(causal, scores, torch.tensor(float("-inf")))


def absorbed_attention_row(q_c, q_rope, kv_rows, selected, scale):
    """One query row, all heads: softmax over ``selected`` cached rows with the bf16-P contract.

    ``q_c [H, lora]``, ``q_rope [H, r]``, ``kv_rows [ctx, lora + r]``; returns ``bf16 [H, lora]``.
    """
    lora = q_c.shape[-1]
    if selected.numel() == 0:
        return torch.zeros_like(q_c)
    rows = kv_rows[selected.long()].to(F32)
    s = (q_c.to(F32) @ rows[:, :lora].T + q_rope.to(F32) @ rows[:, lora:].T) * scale
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    o = bf16_round(p) @ rows[:, :lora]
    return bf16_round(o / l)


def attention_block(x, w: OracleWeights, layer: int, positions, table, selected_rows, trace: Trace):
    g = w.geometry
    a = f"model.layers.{layer}.self_attn"
    q_resid, q_nope, q_rope, latent, k_rope = attention_inputs(x, w, layer, positions, table)
    kv_rows = torch.cat([latent, k_rope], dim=-1)
    trace.kv_rows.append(kv_rows)
    rows = x.shape[0]
    if g.indexer_types[layer] == "full":
        keys, scores = indexer_scores(x, q_resid, w, layer, positions)
        trace.index_keys[layer] = keys
        trace.index_scores[layer] = scores
        if selected_rows is None:
            selected_rows = [top_k_positions(scores[r], r + 1, g.index_top_k) for r in range(rows)]
    kv_b = w[a + ".kv_b_proj"].to(F32).reshape(g.attention_heads, g.kv_b_rows_per_head, g.kv_lora_rank)
    w_k, w_v = kv_b[:, : g.qk_nope_head_dim], kv_b[:, g.qk_nope_head_dim :]
    q_c = bf16_round(torch.einsum("shd,hdc->shc", q_nope, w_k))
    scale = g.qk_head_dim**-0.5
    o_lat = torch.stack([absorbed_attention_row(q_c[r], q_rope[r], kv_rows, selected_rows[r], scale) for r in range(rows)])
    v = bf16_round(torch.einsum("shc,hvc->shv", o_lat, w_v)).reshape(rows, g.attention_heads * g.v_head_dim)
    return linear(v, w[a + ".o_proj"]), selected_rows


def swiglu_act(gate, up):
    return bf16_round(gate * torch.sigmoid(gate) * up)


def dense_mlp(x, w: OracleWeights, prefix: str):
    act = swiglu_act(linear(x, w[prefix + ".gate_proj"]), linear(x, w[prefix + ".up_proj"]))
    return linear(act, w[prefix + ".down_proj"])


def router(x, weight, bias, top_k: int, imposed=None):
    """``(expert ids [rows, k] in descending-choice order, fp32 weights [rows, k], choice [rows, E])``."""
    logits = x.to(F32) @ weight.to(F32).T
    scores = torch.sigmoid(logits)
    choice = scores + bias.to(F32)[None, :]
    if imposed is None:
        ids = torch.argsort(-orderable_key(choice), dim=-1, stable=True)[:, :top_k]
    else:
        ids = imposed.long()
    picked = torch.gather(scores, 1, ids)
    weights = picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)
    return ids, weights, choice


def sparse_moe(x, w: OracleWeights, layer: int, trace: Trace, imposed=None):
    g = w.geometry
    p = f"model.layers.{layer}.mlp"
    ids, weights, choice = router(x, w[p + ".gate.weight"], w[p + ".gate.e_score_correction_bias"], g.routed_top_k, imposed)
    trace.expert_ids[layer], trace.route_weights[layer], trace.router_choice[layer] = ids, weights, choice
    gate_w, up_w, down_w = w[p + ".experts.gate_proj"], w[p + ".experts.up_proj"], w[p + ".experts.down_proj"]
    routed = torch.zeros(x.shape[0], g.hidden_size, dtype=F32)
    for r in range(x.shape[0]):
        for k in range(g.routed_top_k):
            e = int(ids[r, k])
            act = swiglu_act(linear(x[r : r + 1], gate_w[e]), linear(x[r : r + 1], up_w[e]))
            down = linear(act, down_w[e])
            routed[r] += bf16_round(down[0] * bf16_round(weights[r, k]))
    shared = dense_mlp(x, w, p + ".shared_experts")
    scaled = bf16_round(bf16_round(routed) * g.routed_scaling_factor)
    return bf16_round(scaled + shared)


def greedy(logits: torch.Tensor) -> torch.Tensor:
    """Argmax of bf16-rounded logits, ties to the lowest id."""
    top = logits.max(dim=-1, keepdim=True).values
    ids = torch.arange(logits.shape[-1])[None, :].expand_as(logits)
    return torch.where(logits == top, ids, logits.shape[-1]).min(dim=-1).values


def forward(
    w: OracleWeights,
    tokens,
    *,
    capacity: int | None = None,
    selected: Mapping[int, list] | None = None,
    expert_ids: Mapping[int, torch.Tensor] | None = None,
) -> Trace:
    """Run ``tokens`` (positions ``0..rows-1``).  ``selected``/``expert_ids`` impose another system's discrete decisions."""
    g = w.geometry
    tokens = torch.as_tensor(tokens, dtype=torch.int64).reshape(-1)
    rows = tokens.shape[0]
    positions = torch.arange(rows)
    table = rope_table(capacity or rows, g.qk_rope_head_dim, g.rope_theta)
    selected, expert_ids = dict(selected or {}), dict(expert_ids or {})
    trace = Trace(torch.empty(0), torch.empty(0), torch.empty(0))

    residual = w["model.embed_tokens.weight"][tokens].to(F32)
    update = None
    current = None
    for i in range(g.num_layers):
        p = f"model.layers.{i}"
        x, residual = add_rms_norm(update, residual, w[p + ".input_layernorm.weight"], g.rms_norm_eps)
        imposed = selected.get(i) if g.indexer_types[i] == "full" else current
        attn, current = attention_block(x, w, i, positions, table, imposed, trace)
        trace.selected.append(current)
        x, residual = add_rms_norm(attn, residual, w[p + ".post_attention_layernorm.weight"], g.rms_norm_eps)
        if g.mlp_layer_types[i] == "dense":
            update = dense_mlp(x, w, p + ".mlp")
        else:
            update = sparse_moe(x, w, i, trace, expert_ids.get(i))
        trace.layer_outputs.append((attn, update))
    x, residual = add_rms_norm(update, residual, w["model.norm.weight"], g.rms_norm_eps)
    trace.residual = residual
    trace.logits = linear(x, w["lm_head.weight"])
    trace.tokens = greedy(trace.logits)
    return trace
