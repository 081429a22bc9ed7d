"""Frozen fixture v1: a small GLM-MoE-DSA model that exercises every branch (dense and MoE layers, own and shared indexers,
a selection smaller than the context) and whose weights depend only on a seed.

Parity: reference ``tools/equivalence/fixture.py:29-41,62-82`` (8 layers = 3 dense + 5 MoE, indexers F F F S S S F S, hidden 1024,
16 heads, 64 experts, seed 921); scaled down in width so the CPU oracle runs in seconds.
"""

from __future__ import annotations

from glm_tpu_b200.config.model import ModelGeometry

SEED = 921
PROMPT_SEED = 17
PROMPT_TOKENS = 40
NEW_TOKENS = 6
CAPACITY = 96


def fixture_geometry() -> ModelGeometry:
    return ModelGeometry(
        vocab_size=256, hidden_size=256, num_layers=8, attention_heads=4, q_lora_rank=64, kv_lora_rank=64, qk_nope_head_dim=32,
        qk_rope_head_dim=16, v_head_dim=32, dense_intermediate_size=512, moe_intermediate_size=128, num_routed_experts=16, routed_top_k=4,
        num_shared_experts=1, routed_scaling_factor=2.5, index_heads=4, index_head_dim=32, index_top_k=16,
        indexer_types=("full", "full", "full", "shared", "shared", "shared", "full", "shared"),
        mlp_layer_types=("dense", "dense", "dense", "sparse", "sparse", "sparse", "sparse", "sparse"),
        rope_theta=8000000.0, rms_norm_eps=1e-5, fp8_block_shape=(128, 128), eos_ids=(253, 254, 255),
    )


def fixture_checkpoint():
    from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint

    return random_checkpoint(fixture_geometry(), seed=SEED)


def fixture_prompt() -> list[int]:
    import torch

    gen = torch.Generator().manual_seed(PROMPT_SEED)
    return torch.randint(0, 250, (PROMPT_TOKENS,), generator=gen).tolist()
