"""Write a runtime-layout checkpoint as a Hugging Face style *source* directory.

Used for fixtures and synthetic benchmarks: the stacked routed experts are split back into per-expert tensors with the
Hugging Face names (``...experts.{e}.gate_proj.weight`` + ``.weight_scale_inv``), FP8 pairs become ``.weight`` /
``.weight_scale_inv``, tensors are distributed over ``shards`` safetensors files with a ``model.safetensors.index.json``,
and a ``config.json`` is written from which ``ModelGeometry.from_hf_config`` rebuilds the geometry.  The result goes
through the same inventory -> marker -> pack -> verify -> load path as a downloaded checkpoint.

No reference counterpart (the reference only consumes downloaded checkpoints); the names follow
``glm_tpu/model_loader/placement.py:75-196``.
"""

from __future__ import annotations

import json
from pathlib import Path

from glm_tpu_b200.config.model import ModelGeometry
from glm_tpu_b200.model_loader import source_inventory
from glm_tpu_b200.model_loader.sharded_state import format as fmt


def hf_config(g: ModelGeometry) -> dict:
    return {
        "model_type": "glm_moe_dsa", "architectures": ["GlmMoeDsaForCausalLM"], "vocab_size": g.vocab_size, "hidden_size": g.hidden_size,
        "num_hidden_layers": g.num_layers, "num_attention_heads": g.attention_heads, "q_lora_rank": g.q_lora_rank,
        "kv_lora_rank": g.kv_lora_rank, "qk_nope_head_dim": g.qk_nope_head_dim, "qk_rope_head_dim": g.qk_rope_head_dim,
        "v_head_dim": g.v_head_dim, "intermediate_size": g.dense_intermediate_size, "moe_intermediate_size": g.moe_intermediate_size,
        "n_routed_experts": g.num_routed_experts, "num_experts_per_tok": g.routed_top_k, "n_shared_experts": g.num_shared_experts,
        "routed_scaling_factor": g.routed_scaling_factor, "index_n_heads": g.index_heads, "index_head_dim": g.index_head_dim,
        "index_topk": g.index_top_k, "indexer_types": list(g.indexer_types), "mlp_layer_types": list(g.mlp_layer_types),
        "rope_parameters": {"rope_theta": g.rope_theta}, "rms_norm_eps": g.rms_norm_eps, "scoring_func": "sigmoid",
        "topk_method": "noaux_tc", "n_group": 1, "topk_group": 1, "eos_token_id": list(g.eos_ids),
        "quantization_config": {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": list(g.fp8_block_shape)},
    }


def source_tensors(arrays: dict) -> tuple[dict, set]:
    """Runtime layout -> Hugging Face names.  Returns ``(tensors, fp8_names)``."""
    out, fp8 = {}, set()
    for name, t in arrays.items():
        if name.endswith(".weight_bits") or name.endswith(".scale_inv"):
            prefix, role = name.rsplit(".", 1)
            suffix = "weight" if role == "weight_bits" else "weight_scale_inv"
            if ".mlp.experts." in prefix:
                stem, proj = prefix.rsplit(".", 1)
                for e in range(t.shape[0]):
                    out[f"{stem}.{e}.{proj}.{suffix}"] = t[e]
                    if role == "weight_bits":
                        fp8.add(f"{stem}.{e}.{proj}.{suffix}")
            else:
                out[f"{prefix}.{suffix}"] = t
                if role == "weight_bits":
                    fp8.add(f"{prefix}.{suffix}")
        else:
            out[name] = t
    return out, fp8


def export_source(arrays: dict, g: ModelGeometry, root: Path, shards: int = 2) -> Path:
    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    tensors, fp8 = source_tensors(arrays)
    names = sorted(tensors)
    weight_map = {}
    for s in range(shards):
        part = names[s::shards]
        if not part:
            continue
        file = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        fmt.write_file(root / file, {n: tensors[n] for n in part}, {"format": "pt"}, fp8 & set(part))
        weight_map.update({n: file for n in part})
    (root / source_inventory.INDEX_FILE).write_text(json.dumps({"metadata": {}, "weight_map": weight_map}, sort_keys=True))
    (root / "config.json").write_text(json.dumps(hf_config(g), sort_keys=True, indent=1))
    return root
