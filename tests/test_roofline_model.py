"""The byte count behind the decode roofline: hand-computed figures for the GLM-5.3 geometry and the way they split over GPUs."""

import pytest

from glm_tpu_b200.benchmarks import roofline_model as rm
from glm_tpu_b200.config.model import glm53_geometry


def test_expert_and_layer_bytes_match_hand_computation():
    g = glm53_geometry()
    assert rm.expert_bytes(g) == 3 * 2048 * 6144 + 4 * (2 * 16 * 48 + 48 * 16)
    one = rm.decode_step_bytes(g.truncated(4), 1, chats=1, depth=1)  # 3 dense layers + 1 MoE layer, layer 0 and 2 carry an indexer
    full_layers = sum(1 for t in g.truncated(4).indexer_types if t == "full")
    qkv = lambda full: 2048 + 576 + ((128 + 32) if full else 0)  # noqa: E731
    qb = lambda full: 64 * 256 + (32 * 128 if full else 0)  # noqa: E731
    attention = sum(2 * (qkv(f) * 6144 + qb(f) * 2048 + 64 * (192 + 256) * 512 + 6144 * 64 * 256) for f in [True] * full_layers + [False] * (4 - full_layers))
    assert one["attention"] == attention
    assert one["dense_mlp"] == 3 * 2 * 3 * 12288 * 6144 and one["shared_expert"] == 2 * 3 * 2048 * 6144 and one["router"] == 2 * 256 * 6144
    assert one["lm_head"] == 2 * 154880 * 6144
    assert one["routed_mean"] == one["routed_busiest"] == 8 * rm.expert_bytes(g)  # one GPU, one chat: eight distinct experts
    assert one["caches"] == 4 * 1 * 576 * 2 + full_layers * 1 * 128 * 2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_parts_divide_and_the_busiest_gpu_reads_more_than_the_average(world):
    g = glm53_geometry().truncated(10)
    one, many = rm.decode_step_bytes(g, 1), rm.decode_step_bytes(g, world)
    for key in ("dense_mlp", "shared_expert", "lm_head"):
        assert many[key] * world == one[key]
    assert many["router"] == one["router"] and many["attention"] < one["attention"]  # replicated parts stay, head-split parts shrink
    assert abs(many["experts_per_layer_mean"] - 8 / world) < 0.05
    assert 8 / world < many["experts_per_layer_busiest"] <= 8
    assert many["total_busiest"] > many["total_mean"]
    striped = rm.decode_step_bytes(g, world, depth=30000, striped=True)
    replicated = rm.decode_step_bytes(g, world, depth=30000)
    assert striped["caches"] < replicated["caches"]


def test_four_chats_touch_fewer_than_four_times_the_experts():
    g = glm53_geometry().truncated(10)
    one, four = rm.decode_step_bytes(g, 1, chats=1), rm.decode_step_bytes(g, 1, chats=4)
    assert 3.5 * one["routed_mean"] < four["routed_mean"] < 4 * one["routed_mean"]  # some of 32 routes share an expert
    assert rm.main(["--gpus", "1,8", "--measured", "1:2.175"]) == 0


def test_prefill_flops_follow_the_shapes():
    g = glm53_geometry().truncated(4)
    f1, f8 = rm.prefill_flops(g, 1, 4096), rm.prefill_flops(g, 8, 4096)
    assert f1["routed_experts"] == 2 * 4096 * 8 * 3 * 2048 * 6144 and f8["routed_experts"] * 8 == f1["routed_experts"]
    keys = sum(min(p + 1, 2048) for p in range(4096))
    assert f1["attention"] == 4 * 2 * keys * 64 * (576 + 512) and f8["attention"] * 8 == f1["attention"]
    assert f8["indexer"] == f1["indexer"] > 0  # with a replicated cache every GPU scores every row
    assert f1["total"] == sum(v for k, v in f1.items() if k != "total")
    assert rm.main(["--gpus", "1", "--prefill", "1024", "--measured-prefill", "1:100"]) == 0
