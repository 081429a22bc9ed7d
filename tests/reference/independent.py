"""An independent FP64 NumPy restatement of the GLM-MoE-DSA forward pass.

It shares no code with ``glm_tpu_b200/oracle/contract.py``: its own e4m3 parser and bf16 rounding for the *weights* (which are
data: the checkpoint defines them as ``bf16(e4m3 * scale)``), and exact float64 arithmetic for everything else: no intermediate
rounding, attention in the plain (non-absorbed) form with explicit per-head keys and values, a dense masked softmax.  Discrete
decisions (DSA selections, routed experts) are *imposed* from the system under test, because a near-tie legitimately flips them;
``selection_regret`` and ``routing_regret`` then check that the imposed decisions are optimal up to a small margin under this
restatement's own scores.

Parity: reference ``tests/reference/independent.py:1-357`` (FP64 restatement with imposed decisions + regret checks).
"""

from __future__ import annotations

import numpy as np


# ---------------------------------------------------------------------------------------------- weights (data)
def e4m3_to_f64(bits: np.ndarray) -> np.ndarray:
    b = bits.astype(np.int64)
    sign = np.where(b & 0x80, -1.0, 1.0)
    exp, man = (b >> 3) & 0xF, b & 0x7
    normal = (1.0 + man / 8.0) * np.exp2(exp - 7.0)
    sub = (man / 8.0) * 2.0**-6
    return sign * np.where(exp == 0, sub, normal)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to 8 significant bits, via the fp32 bit pattern."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def table(ckpt: dict, prefix: str, block=(128, 128)) -> np.ndarray:
    if prefix + ".weight" in ckpt:
        return ckpt[prefix + ".weight"].float().numpy().astype(np.float64)
    bits = ckpt[prefix + ".weight_bits"].numpy()
    scale = ckpt[prefix + ".scale_inv"].float().numpy().astype(np.float32)
    scale = np.repeat(np.repeat(scale, block[0], axis=-2), block[1], axis=-1)[..., : bits.shape[-2], : bits.shape[-1]]
    return round_bf16(e4m3_to_f64(bits).astype(np.float32) * scale)  # the product itself is an fp32 product by definition


def vec(ckpt: dict, name: str) -> np.ndarray:
    return ckpt[name].float().numpy().astype(np.float64)


# ---------------------------------------------------------------------------------------------- math
def rms(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def rotate_pairs(x, pos, theta, dim):
    """Interleaved RoPE on the first ``dim`` features of the last axis; ``x [rows, ..., width]``."""
    j = np.arange(0, dim, 2, dtype=np.float64)
    ang = pos.astype(np.float64)[:, None] * theta ** (-j / dim)
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dim // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = x.copy()
    ev, od = x[..., 0:dim:2], x[..., 1:dim:2]
    out[..., 0:dim:2] = ev * c - od * s
    out[..., 1:dim:2] = od * c + ev * s
    return out


def silu(x):
    return x / (1.0 + np.exp(-x))


def forward(g, ckpt: dict, tokens, selected: dict, expert_ids: dict) -> dict:
    """``selected``: layer -> list over rows of position arrays (every layer, shared layers included);
    ``expert_ids``: sparse layer -> [rows, k].  Returns logits, index scores and router choice scores in float64."""
    tokens = np.asarray(tokens, dtype=np.int64)
    rows = tokens.shape[0]
    pos = np.arange(rows)
    h = vec(ckpt, "model.embed_tokens.weight")[tokens]
    out = {"index_scores": {}, "router_choice": {}}
    H, nope, rd, vd, L = g.attention_heads, g.qk_nope_head_dim, g.qk_rope_head_dim, g.v_head_dim, g.kv_lora_rank
    for i in range(g.num_layers):
        p, a = f"model.layers.{i}", f"model.layers.{i}.self_attn"
        x = rms(h, vec(ckpt, p + ".input_layernorm.weight"), g.rms_norm_eps)
        qr = rms(x @ table(ckpt, a + ".q_a_proj").T, vec(ckpt, a + ".q_a_layernorm.weight"), g.rms_norm_eps)
        q = (qr @ table(ckpt, a + ".q_b_proj").T).reshape(rows, H, nope + rd)
        q = np.concatenate([q[..., :nope], rotate_pairs(q[..., nope:], pos, g.rope_theta, rd)], axis=-1)
        comp = x @ table(ckpt, a + ".kv_a_proj_with_mqa").T
        latent = rms(comp[:, :L], vec(ckpt, a + ".kv_a_layernorm.weight"), g.rms_norm_eps)
        k_rope = rotate_pairs(comp[:, L:], pos, g.rope_theta, rd)
        kv_b = table(ckpt, a + ".kv_b_proj").reshape(H, nope + vd, L)
        k = np.concatenate([np.einsum("tc,hdc->thd", latent, kv_b[:, :nope]), np.broadcast_to(k_rope[:, None, :], (rows, H, rd))], axis=-1)
        v = np.einsum("tc,hvc->thv", latent, kv_b[:, nope:])
        if g.indexer_types[i] == "full":
            ix = a + ".indexer"
            key = x @ table(ckpt, ix + ".wk").T
            key = (key - key.mean(-1, keepdims=True)) / np.sqrt(key.var(-1, keepdims=True) + 1e-6) * vec(ckpt, ix + ".k_norm.weight") + vec(ckpt, ix + ".k_norm.bias")
            key = rotate_pairs(key, pos, g.rope_theta, rd)
            qi = rotate_pairs((qr @ table(ckpt, ix + ".wq_b").T).reshape(rows, g.index_heads, g.index_head_dim), pos, g.rope_theta, rd)
            hw = x @ vec(ckpt, ix + ".weights_proj.weight").T * g.index_heads**-0.5
            dots = np.einsum("shd,td->sht", qi, key) * g.index_head_dim**-0.5
            out["index_scores"][i] = np.einsum("sh,sht->st", hw, np.maximum(dots, 0.0))
        mask = np.full((rows, rows), -np.inf)
        for r in range(rows):
            mask[r, np.asarray(selected[i][r], dtype=np.int64)] = 0.0
        s = np.einsum("shd,thd->hst", q, k) * (nope + rd) ** -0.5 + mask[None]
        s = s - s.max(-1, keepdims=True)
        pr = np.exp(s)
        pr /= pr.sum(-1, keepdims=True)
        attn = np.einsum("hst,thv->shv", pr, v).reshape(rows, H * vd) @ table(ckpt, a + ".o_proj").T
        h = h + attn
        x = rms(h, vec(ckpt, p + ".post_attention_layernorm.weight"), g.rms_norm_eps)
        m = p + ".mlp"
        if g.mlp_layer_types[i] == "dense":
            upd = (silu(x @ table(ckpt, m + ".gate_proj").T) * (x @ table(ckpt, m + ".up_proj").T)) @ table(ckpt, m + ".down_proj").T
        else:
            sc = 1.0 / (1.0 + np.exp(-(x @ vec(ckpt, m + ".gate.weight").T)))
            out["router_choice"][i] = sc + vec(ckpt, m + ".gate.e_score_correction_bias")[None]
            ids = np.asarray(expert_ids[i], dtype=np.int64)
            wsel = np.take_along_axis(sc, ids, axis=1)
            wsel = wsel / wsel.sum(-1, keepdims=True)
            wg, wu, wd = table(ckpt, m + ".experts.gate_proj"), table(ckpt, m + ".experts.up_proj"), table(ckpt, m + ".experts.down_proj")
            routed = np.zeros_like(x)
            for r in range(rows):
                for j, e in enumerate(ids[r]):
                    routed[r] += wsel[r, j] * ((silu(x[r] @ wg[e].T) * (x[r] @ wu[e].T)) @ wd[e].T)
            sh = m + ".shared_experts"
            shared = (silu(x @ table(ckpt, sh + ".gate_proj").T) * (x @ table(ckpt, sh + ".up_proj").T)) @ table(ckpt, sh + ".down_proj").T
            upd = routed * g.routed_scaling_factor + shared
        h = h + upd
    x = rms(h, vec(ckpt, "model.norm.weight"), g.rms_norm_eps)
    out["logits"] = x @ vec(ckpt, "lm_head.weight").T
    return out


# ---------------------------------------------------------------------------------------------- regret
def selection_regret(scores_row: np.ndarray, chosen, ctx: int, top_k: int) -> float:
    """How much better the best unchosen position scores than the worst chosen one (<= 0: the choice is optimal)."""
    chosen = np.asarray(chosen, dtype=np.int64)
    if ctx <= top_k:
        return 0.0 if len(chosen) == ctx else np.inf
    inside = np.zeros(ctx, dtype=bool)
    inside[chosen] = True
    return float(scores_row[:ctx][~inside].max() - scores_row[:ctx][inside].min())


def routing_regret(choice_row: np.ndarray, chosen) -> float:
    chosen = np.asarray(chosen, dtype=np.int64)
    inside = np.zeros(choice_row.shape[0], dtype=bool)
    inside[chosen] = True
    return float(choice_row[~inside].max() - choice_row[inside].min())
