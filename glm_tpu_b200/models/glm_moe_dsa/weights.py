"""Weight names, the runtime checkpoint layout, and the per-GPU resident weights.

**Runtime layout** (one flat ``name -> tensor`` mapping, the layout the loader produces and the oracle reads):
FP8 tables are a pair ``<prefix>.weight_bits`` (uint8 e4m3fn) + ``<prefix>.scale_inv`` (fp32, one per 128x128
block); bf16 tables are ``<prefix>.weight``.  Routed experts are *stacked* per layer:
``model.layers.{i}.mlp.experts.{gate,up,down}_proj.weight_bits`` is ``[E, N, K]`` with scales ``[E, N/128, K/128]``
(built from the per-expert Hugging Face tensors ``...experts.{e}.{proj}.weight`` / ``.weight_scale_inv``).

**Resident weights** (``DeviceWeights``): what one GPU keeps.  Non-routed FP8 tables are decoded once at load
to bf16 with ``bf16(f32(e4m3) * scale_inv)`` and cut by the parallel layout (heads, MLP columns, vocabulary
rows); small tables every GPU needs are replicated and several projections that consume the same activation are
concatenated so that one streaming kernel serves them.  Routed experts stay FP8: each GPU keeps its
``experts_local`` experts whole, or (``ParallelLayout.expert_split == "sliced"``) its slice of the intermediate columns of
every expert, cut on FP8 block boundaries so that the block scales are cut with the bits.

Parity: reference ``glm_tpu/models/glm_moe_dsa/weights.py:37-216`` (trees, specs, bf16 residency),
``:338-445`` (exact tensor names), ``glm_tpu/model_loader/placement.py:75-196`` (source shapes).
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Mapping

import torch

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.config.parallel import ParallelLayout

FP8_PROJECTIONS = (
    "q_a_proj", "kv_a_proj_with_mqa", "q_b_proj", "kv_b_proj", "o_proj", "wq_b", "wk", "gate_proj", "up_proj", "down_proj",
)


def projection_shapes(g: ModelGeometry, layer: int) -> dict[str, tuple[int, ...]]:
    """Shape of every 2-D/3-D weight table of ``layer`` keyed by its name prefix (without the role suffix)."""
    p = f"model.layers.{layer}"
    a = p + ".self_attn"
    shapes: dict[str, tuple[int, ...]] = {
        a + ".q_a_proj": (g.q_lora_rank, g.hidden_size),
        a + ".kv_a_proj_with_mqa": (g.kv_row_width, g.hidden_size),
        a + ".q_b_proj": (g.attention_heads * g.qk_head_dim, g.q_lora_rank),
        a + ".kv_b_proj": (g.attention_heads * g.kv_b_rows_per_head, g.kv_lora_rank),
        a + ".o_proj": (g.hidden_size, g.attention_heads * g.v_head_dim),
    }
    if g.indexer_types[layer] == "full":
        shapes[a + ".indexer.wq_b"] = (g.index_heads * g.index_head_dim, g.q_lora_rank)
        shapes[a + ".indexer.wk"] = (g.index_head_dim, g.hidden_size)
    if g.mlp_layer_types[layer] == "dense":
        shapes[p + ".mlp.gate_proj"] = (g.dense_intermediate_size, g.hidden_size)
        shapes[p + ".mlp.up_proj"] = (g.dense_intermediate_size, g.hidden_size)
        shapes[p + ".mlp.down_proj"] = (g.hidden_size, g.dense_intermediate_size)
    else:
        e, i, s = g.num_routed_experts, g.moe_intermediate_size, g.moe_intermediate_size * g.num_shared_experts
        shapes[p + ".mlp.experts.gate_proj"] = (e, i, g.hidden_size)
        shapes[p + ".mlp.experts.up_proj"] = (e, i, g.hidden_size)
        shapes[p + ".mlp.experts.down_proj"] = (e, g.hidden_size, i)
        shapes[p + ".mlp.shared_experts.gate_proj"] = (s, g.hidden_size)
        shapes[p + ".mlp.shared_experts.up_proj"] = (s, g.hidden_size)
        shapes[p + ".mlp.shared_experts.down_proj"] = (g.hidden_size, s)
    return shapes


def plain_shapes(g: ModelGeometry, layer: int) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
    """Tensors that are never FP8: norms, router, indexer small tables."""
    p = f"model.layers.{layer}"
    a = p + ".self_attn"
    out = {
        p + ".input_layernorm.weight": ((g.hidden_size,), torch.bfloat16),
        p + ".post_attention_layernorm.weight": ((g.hidden_size,), torch.bfloat16),
        a + ".q_a_layernorm.weight": ((g.q_lora_rank,), torch.bfloat16),
        a + ".kv_a_layernorm.weight": ((g.kv_lora_rank,), torch.bfloat16),
    }
    if g.indexer_types[layer] == "full":
        out[a + ".indexer.k_norm.weight"] = ((g.index_head_dim,), torch.bfloat16)
        out[a + ".indexer.k_norm.bias"] = ((g.index_head_dim,), torch.bfloat16)
        out[a + ".indexer.weights_proj.weight"] = ((g.index_heads, g.hidden_size), torch.bfloat16)
    if g.mlp_layer_types[layer] == "sparse":
        out[p + ".mlp.gate.weight"] = ((g.num_routed_experts, g.hidden_size), torch.bfloat16)
        out[p + ".mlp.gate.e_score_correction_bias"] = ((g.num_routed_experts,), torch.float32)
    return out


def runtime_tensor_names(g: ModelGeometry, fp8: bool = True) -> list[str]:
    """Every tensor name of the runtime layout, in a fixed order (the name bijection the loader checks)."""
    names = ["model.embed_tokens.weight"]
    for i in range(g.num_layers):
        for prefix in projection_shapes(g, i):
            names += [prefix + ".weight_bits", prefix + ".scale_inv"] if fp8 else [prefix + ".weight"]
        names += list(plain_shapes(g, i))
    names += ["model.norm.weight", "lm_head.weight"]
    return names


def scale_shape(shape: tuple[int, ...], block: tuple[int, int]) -> tuple[int, ...]:
    return (*shape[:-2], -(-shape[-2] // block[0]), -(-shape[-1] // block[1]))


def quantize_fp8(w: torch.Tensor, block: tuple[int, int], generator: torch.Generator | None = None):
    """Block-quantize ``w [..., N, K]`` to e4m3 with scales ``U(0.5, 2) * amax / 448`` per block (fixture rule)."""
    bn, bk = block
    *lead, n, k = w.shape
    nb, kb = -(-n // bn), -(-k // bk)
    padded = torch.zeros(*lead, nb * bn, kb * bk, dtype=torch.float32)
    padded[..., :n, :k] = w.float()
    blocks = padded.reshape(*lead, nb, bn, kb, bk)
    amax = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-12)
    jitter = torch.rand(amax.shape, generator=generator) * 1.5 + 0.5 if generator is not None else torch.ones_like(amax)
    scale = (jitter * amax / 448.0).float()
    q = (blocks / scale[..., :, None, :, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    bits = q.reshape(*lead, nb * bn, kb * bk)[..., :n, :k].contiguous().view(torch.uint8)
    return bits, scale


def random_checkpoint(g: ModelGeometry, seed: int = 0, fp8: str = "all") -> dict[str, torch.Tensor]:
    """A random runtime-layout checkpoint on the CPU (fixtures).  ``fp8``: 'all' FP8-able tables, or 'routed' only.

    Weights are ``N(0, 0.02)``; norm weights ``N(1, 0.1)``; router bias ``N(0, 0.02)``; FP8 scales follow the
    fixture rule of ``quantize_fp8``.
    """
    gen = torch.Generator().manual_seed(seed)
    out: dict[str, torch.Tensor] = {}

    def normal(shape, std=0.02, mean=0.0):
        return torch.randn(shape, generator=gen) * std + mean

    out["model.embed_tokens.weight"] = normal((g.vocab_size, g.hidden_size)).to(torch.bfloat16)
    for i in range(g.num_layers):
        for prefix, shape in projection_shapes(g, i).items():
            w = normal(shape)
            if fp8 == "all" or (fp8 == "routed" and ".experts." in prefix):
                out[prefix + ".weight_bits"], out[prefix + ".scale_inv"] = quantize_fp8(w, g.fp8_block_shape, gen)
            else:
                out[prefix + ".weight"] = w.to(torch.bfloat16)
        for name, (shape, dtype) in plain_shapes(g, i).items():
            if name.endswith("layernorm.weight") or name.endswith("k_norm.weight"):
                out[name] = normal(shape, 0.1, 1.0).to(dtype)
            elif name.endswith("k_norm.bias"):
                out[name] = normal(shape, 0.05).to(dtype)
            elif name.endswith("e_score_correction_bias"):
                out[name] = normal(shape, 0.02).to(dtype)
            else:
                out[name] = normal(shape).to(dtype)
    out["model.norm.weight"] = normal((g.hidden_size,), 0.1, 1.0).to(torch.bfloat16)
    out["lm_head.weight"] = normal((g.vocab_size, g.hidden_size)).to(torch.bfloat16)
    return out


# ----------------------------------------------------------------------------------------------------
@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    w_qkv_a: torch.Tensor  # [Q + L + rd (+ D + IH), H] bf16, replicated: q_a | kv_a | indexer wk | indexer weights_proj
    q_a_norm: torch.Tensor
    kv_a_norm: torch.Tensor
    w_q_b: torch.Tensor  # [heads_local * qk (+ IH * D), Q] bf16: this GPU's heads | indexer wq_b
    kv_b: torch.Tensor  # [heads_local, nope + v, L] bf16
    w_o: torch.Tensor  # [H, heads_local * v] bf16 (K-slice of o_proj)
    k_norm_w: torch.Tensor | None = None  # fp32 [D]
    k_norm_b: torch.Tensor | None = None
    # dense MLP (column slice)
    dense_gate: torch.Tensor | None = None  # [I_local, H]
    dense_up: torch.Tensor | None = None
    dense_down: torch.Tensor | None = None  # [H, I_local]
    # MoE
    router_w: torch.Tensor | None = None  # [E, H] bf16
    router_bias: torch.Tensor | None = None  # [E] fp32
    exp_gate_bits: torch.Tensor | None = None  # [E_local, I, H] uint8 (whole experts) or [E, I / world, H] (sliced)
    exp_gate_scale: torch.Tensor | None = None
    exp_up_bits: torch.Tensor | None = None
    exp_up_scale: torch.Tensor | None = None
    exp_down_bits: torch.Tensor | None = None  # [E_local, H, I] or [E, H, I / world]
    exp_down_scale: torch.Tensor | None = None
    shared_gate: torch.Tensor | None = None  # [Is_local, H]
    shared_up: torch.Tensor | None = None
    shared_down: torch.Tensor | None = None  # [H, Is_local]


@dataclass
class DeviceWeights:
    geometry: ModelGeometry
    layout: ParallelLayout
    embed: torch.Tensor  # [V, H] bf16 replicated
    layers: list[LayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor  # [V_local, H]
    bytes_resident: int = 0
    notes: dict = field(default_factory=dict)

    def count_bytes(self) -> int:
        total = self.embed.numel() * 2 + self.final_norm.numel() * 2 + self.lm_head.numel() * 2
        for lw in self.layers:
            for value in vars(lw).values():
                if isinstance(value, torch.Tensor):
                    total += value.numel() * value.element_size()
        self.bytes_resident = total
        return total


def _decode(arrays: Mapping[str, torch.Tensor], prefix: str, g: ModelGeometry, device, use_kernel: bool) -> torch.Tensor:
    """The bf16 table of ``prefix`` (decoding its FP8 pair on ``device`` if that is how it is stored)."""
    if prefix + ".weight" in arrays:
        return arrays[prefix + ".weight"].to(device=device, dtype=torch.bfloat16)
    bits = arrays[prefix + ".weight_bits"].to(device)
    scale = arrays[prefix + ".scale_inv"].to(device=device, dtype=torch.float32)
    if use_kernel and bits.is_cuda:
        from glm_tpu_b200.ops import native

        out = torch.empty(bits.shape, dtype=torch.bfloat16, device=device)
        native.fp8_to_bf16(bits.contiguous(), scale.contiguous(), out, g.fp8_block_shape)
        return out
    from glm_tpu_b200.oracle.contract import dequantize_fp8

    return dequantize_fp8(bits.cpu(), scale.cpu(), g.fp8_block_shape).to(device)


def shard_checkpoint(arrays: Mapping[str, torch.Tensor], layout: ParallelLayout, device, use_kernel: bool = True) -> DeviceWeights:
    """Cut a runtime-layout checkpoint into one GPU's resident weights (see the module docstring)."""
    g = layout.geometry
    r, hl = layout.rank, layout.heads_local
    dev = torch.device(device)
    # A packed checkpoint hands over the routed experts already cut for (rank, world); it says so with this marker.
    presliced = "__experts_presliced__" in arrays
    if presliced and arrays["__experts_presliced__"].tolist() != [layout.rank, layout.world]:
        raise ValueError("the expert tensors were cut for another rank or world size")

    def to_dev(name, dtype=None):
        t = arrays[name].to(dev)
        return t.to(dtype) if dtype is not None else t

    layers: list[LayerWeights] = []
    for i in range(g.num_layers):
        p = f"model.layers.{i}"
        a = p + ".self_attn"
        full = g.indexer_types[i] == "full"
        qkv = [_decode(arrays, a + ".q_a_proj", g, dev, use_kernel), _decode(arrays, a + ".kv_a_proj_with_mqa", g, dev, use_kernel)]
        q_b = _decode(arrays, a + ".q_b_proj", g, dev, use_kernel)
        q_b_parts = [q_b[r * hl * g.qk_head_dim : (r + 1) * hl * g.qk_head_dim]]
        if full:
            qkv += [_decode(arrays, a + ".indexer.wk", g, dev, use_kernel), to_dev(a + ".indexer.weights_proj.weight", torch.bfloat16)]
            q_b_parts.append(_decode(arrays, a + ".indexer.wq_b", g, dev, use_kernel))
        kv_b = _decode(arrays, a + ".kv_b_proj", g, dev, use_kernel).reshape(g.attention_heads, g.kv_b_rows_per_head, g.kv_lora_rank)
        o = _decode(arrays, a + ".o_proj", g, dev, use_kernel)
        lw = LayerWeights(
            input_norm=to_dev(p + ".input_layernorm.weight"),
            post_norm=to_dev(p + ".post_attention_layernorm.weight"),
            w_qkv_a=torch.cat(qkv, dim=0).contiguous(),
            q_a_norm=to_dev(a + ".q_a_layernorm.weight"),
            kv_a_norm=to_dev(a + ".kv_a_layernorm.weight"),
            w_q_b=torch.cat(q_b_parts, dim=0).contiguous(),
            kv_b=kv_b[r * hl : (r + 1) * hl].contiguous(),
            w_o=o[:, r * hl * g.v_head_dim : (r + 1) * hl * g.v_head_dim].contiguous(),
        )
        if full:
            lw.k_norm_w = to_dev(a + ".indexer.k_norm.weight", torch.float32)
            lw.k_norm_b = to_dev(a + ".indexer.k_norm.bias", torch.float32)
        if g.mlp_layer_types[i] == "dense":
            c = layout.dense_cols_local
            lw.dense_gate = _decode(arrays, p + ".mlp.gate_proj", g, dev, use_kernel)[r * c : (r + 1) * c].contiguous()
            lw.dense_up = _decode(arrays, p + ".mlp.up_proj", g, dev, use_kernel)[r * c : (r + 1) * c].contiguous()
            lw.dense_down = _decode(arrays, p + ".mlp.down_proj", g, dev, use_kernel)[:, r * c : (r + 1) * c].contiguous()
        else:
            c = layout.shared_cols_local
            lw.router_w = to_dev(p + ".mlp.gate.weight", torch.bfloat16)
            lw.router_bias = to_dev(p + ".mlp.gate.e_score_correction_bias", torch.float32)
            for proj, attr in (("gate_proj", "exp_gate"), ("up_proj", "exp_up"), ("down_proj", "exp_down")):
                prefix = f"{p}.mlp.experts.{proj}"
                if prefix + ".weight_bits" not in arrays:
                    raise ValueError(f"{prefix} must be stored as FP8 (weight_bits + scale_inv)")
                bits, scale = arrays[prefix + ".weight_bits"], arrays[prefix + ".scale_inv"]
                if not presliced:
                    bits, scale = cut_routed(bits, scale, proj, layout)
                want = routed_shape(layout, proj)
                if tuple(bits.shape) != want:
                    raise ValueError(f"{prefix}: shape {tuple(bits.shape)} where this GPU holds {want}")
                setattr(lw, attr + "_bits", bits.to(dev).contiguous())
                setattr(lw, attr + "_scale", scale.to(dev, torch.float32).contiguous())
            lw.shared_gate = _decode(arrays, p + ".mlp.shared_experts.gate_proj", g, dev, use_kernel)[r * c : (r + 1) * c].contiguous()
            lw.shared_up = _decode(arrays, p + ".mlp.shared_experts.up_proj", g, dev, use_kernel)[r * c : (r + 1) * c].contiguous()
            lw.shared_down = _decode(arrays, p + ".mlp.shared_experts.down_proj", g, dev, use_kernel)[:, r * c : (r + 1) * c].contiguous()
        layers.append(lw)
    vl = layout.vocab_local
    weights = DeviceWeights(
        geometry=g,
        layout=layout,
        embed=to_dev("model.embed_tokens.weight"),
        layers=layers,
        final_norm=to_dev("model.norm.weight"),
        lm_head=to_dev("lm_head.weight")[r * vl : (r + 1) * vl].contiguous(),
    )
    weights.count_bytes()
    return weights


def routed_shape(layout: ParallelLayout, proj: str) -> tuple[int, int, int]:
    """Shape of the resident FP8 table of one routed projection ('gate_proj', 'up_proj' or 'down_proj') on one GPU."""
    g = layout.geometry
    e, c, h = layout.experts_resident, layout.moe_cols_local, g.hidden_size
    return (e, h, c) if proj == "down_proj" else (e, c, h)


def cut_routed(bits: torch.Tensor, scale: torch.Tensor, proj: str, layout: ParallelLayout):
    """One GPU's part of a stacked routed table ``[E, N, K]`` and of its block scales."""
    r = layout.rank
    if not layout.sliced:
        el = layout.experts_local
        return bits[r * el : (r + 1) * el], scale[r * el : (r + 1) * el]
    c = layout.moe_cols_local
    bn, bk = layout.geometry.fp8_block_shape
    if proj == "down_proj":  # [E, H, I]: a slice of K
        return bits[:, :, r * c : (r + 1) * c], scale[:, :, r * c // bk : (r + 1) * c // bk]
    return bits[:, r * c : (r + 1) * c], scale[:, r * c // bn : (r + 1) * c // bn]


def _seed_of(name: str, seed: int) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


def random_device_weights(layout: ParallelLayout, device, seed: int = 0) -> DeviceWeights:
    """Random-init resident weights generated directly in device memory (benchmarks at full size).

    Replicated tables use a seed derived from the tensor name only, so every rank generates identical bits;
    sharded tables mix the rank into the seed.  Routed experts are random e4m3 codes with ~N(0, 112^2) decoded
    values and block scales ``U(0.5, 2) * 0.02 / 112`` so the decoded weights have a standard deviation near 0.02.
    """
    from glm_tpu_b200.ops import native

    g = layout.geometry
    dev = torch.device(device)
    r = layout.rank

    def bf16(name, shape, mean=0.0, std=0.02, sharded=False):
        t = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        native.fill_random_bf16(t, _seed_of(name + (f"@{r}" if sharded else ""), seed), mean, std)
        return t

    def fp8(name, shape):
        bits = torch.empty(shape, dtype=torch.uint8, device=dev)
        native.fill_random_fp8(bits, _seed_of(f"{name}@{r}", seed))
        scale = torch.empty(scale_shape(shape, g.fp8_block_shape), dtype=torch.float32, device=dev)
        native.fill_uniform_f32(scale, _seed_of(f"{name}.scale@{r}", seed), 0.5 * 0.02 / 112.0, 2.0 * 0.02 / 112.0)
        return bits, scale

    def f32(name, shape, mean=0.0, std=0.02):
        return bf16(name, shape, mean, std).float()

    H, Q, L, rd = g.hidden_size, g.q_lora_rank, g.kv_lora_rank, g.qk_rope_head_dim
    hl = layout.heads_local
    layers = []
    for i in range(g.num_layers):
        p = f"L{i}"
        full = g.indexer_types[i] == "full"
        n_qkv = Q + L + rd + ((g.index_head_dim + g.index_heads) if full else 0)
        n_qb = hl * g.qk_head_dim + (g.index_heads * g.index_head_dim if full else 0)
        w_q_b = torch.empty((n_qb, Q), dtype=torch.bfloat16, device=dev)
        native.fill_random_bf16(w_q_b[: hl * g.qk_head_dim], _seed_of(f"{p}.q_b@{r}", seed), 0.0, 0.02)
        if full:
            native.fill_random_bf16(w_q_b[hl * g.qk_head_dim :], _seed_of(f"{p}.idx_wq_b", seed), 0.0, 0.02)
        lw = LayerWeights(
            input_norm=bf16(p + ".in_norm", (H,), 1.0, 0.1),
            post_norm=bf16(p + ".post_norm", (H,), 1.0, 0.1),
            w_qkv_a=bf16(p + ".qkv_a", (n_qkv, H)),
            q_a_norm=bf16(p + ".q_a_norm", (Q,), 1.0, 0.1),
            kv_a_norm=bf16(p + ".kv_a_norm", (L,), 1.0, 0.1),
            w_q_b=w_q_b,
            kv_b=bf16(p + ".kv_b", (hl, g.kv_b_rows_per_head, L), sharded=True),
            w_o=bf16(p + ".o", (H, hl * g.v_head_dim), sharded=True),
        )
        if full:
            lw.k_norm_w = f32(p + ".k_norm_w", (g.index_head_dim,), 1.0, 0.1)
            lw.k_norm_b = f32(p + ".k_norm_b", (g.index_head_dim,), 0.0, 0.05)
        if g.mlp_layer_types[i] == "dense":
            c = layout.dense_cols_local
            lw.dense_gate = bf16(p + ".dense_gate", (c, H), sharded=True)
            lw.dense_up = bf16(p + ".dense_up", (c, H), sharded=True)
            lw.dense_down = bf16(p + ".dense_down", (H, c), sharded=True)
        else:
            c = layout.shared_cols_local
            lw.router_w = bf16(p + ".router", (g.num_routed_experts, H))
            lw.router_bias = f32(p + ".router_bias", (g.num_routed_experts,), 0.0, 0.02)
            lw.exp_gate_bits, lw.exp_gate_scale = fp8(p + ".exp_gate", routed_shape(layout, "gate_proj"))
            lw.exp_up_bits, lw.exp_up_scale = fp8(p + ".exp_up", routed_shape(layout, "up_proj"))
            lw.exp_down_bits, lw.exp_down_scale = fp8(p + ".exp_down", routed_shape(layout, "down_proj"))
            lw.shared_gate = bf16(p + ".shared_gate", (c, H), sharded=True)
            lw.shared_up = bf16(p + ".shared_up", (c, H), sharded=True)
            lw.shared_down = bf16(p + ".shared_down", (H, c), sharded=True)
        layers.append(lw)
    weights = DeviceWeights(
        geometry=g,
        layout=layout,
        embed=bf16("embed", (g.vocab_size, H)),
        layers=layers,
        final_norm=bf16("final_norm", (H,), 1.0, 0.1),
        lm_head=bf16("lm_head", (layout.vocab_local, H), sharded=True),
    )
    weights.count_bytes()
    weights.notes["init"] = f"random device init, seed {seed}"
    return weights
