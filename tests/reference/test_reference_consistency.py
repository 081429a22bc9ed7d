"""The contract oracle against the independent FP64 restatement, with the oracle's discrete decisions imposed and regret-checked."""

import numpy as np
import pytest

from glm_tpu_b200.oracle import contract
from tests.reference import independent as ind
from tools.equivalence import fixture as fx


@pytest.fixture(scope="module")
def both():
    g, ckpt = fx.fixture_geometry(), fx.fixture_checkpoint()
    tokens = fx.fixture_prompt()
    trace = contract.forward(contract.OracleWeights.from_checkpoint(g, ckpt), tokens, capacity=fx.CAPACITY)
    selected = {i: [r.numpy() for r in trace.selected[i]] for i in range(g.num_layers)}
    experts = {i: ids.numpy() for i, ids in trace.expert_ids.items()}
    return g, ckpt, tokens, trace, ind.forward(g, ckpt, tokens, selected, experts)


def test_weight_decode_matches_bit_for_bit():
    g, ckpt = fx.fixture_geometry(), fx.fixture_checkpoint()
    prefix = "model.layers.3.mlp.experts.gate_proj"
    mine = ind.table(ckpt, prefix, g.fp8_block_shape)
    theirs = contract.dequantize_fp8(ckpt[prefix + ".weight_bits"], ckpt[prefix + ".scale_inv"], g.fp8_block_shape).float().numpy()
    assert np.array_equal(mine.astype(np.float32), theirs)
    codes = np.arange(256, dtype=np.uint8)
    ok = (codes & 0x7F) != 0x7F  # the two NaN codes are refused by the loader
    import torch

    ref = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(ind.e4m3_to_f64(codes)[ok].astype(np.float32), ref[ok])


def test_logits_agree_within_bf16_noise(both):
    g, ckpt, tokens, trace, exact = both
    got, want = trace.logits.numpy().astype(np.float64), exact["logits"]
    span = np.abs(want).max()
    # ~50 bf16 roundings (2^-9 relative each) on the path of every logit: a few percent of the logit range is the floor
    assert np.abs(got - want).max() < 0.04 * span, np.abs(got - want).max() / span
    assert np.corrcoef(got.ravel(), want.ravel())[0, 1] > 0.999
    # the greedy token may only differ where the exact margin is within the noise
    top = want.argmax(-1)
    for r, t in enumerate(trace.tokens.tolist()):
        assert want[r, top[r]] - want[r, t] < 0.04 * span


def test_selections_have_no_regret(both):
    g, ckpt, tokens, trace, exact = both
    worst = 0.0
    for layer, scores in exact["index_scores"].items():
        scale = np.abs(scores[np.isfinite(scores)]).max()
        for r in range(len(tokens)):
            worst = max(worst, ind.selection_regret(scores[r], trace.selected[layer][r].numpy(), r + 1, g.index_top_k) / scale)
    assert worst < 0.02, worst


def test_routes_have_no_regret(both):
    g, ckpt, tokens, trace, exact = both
    worst = 0.0
    for layer, choice in exact["router_choice"].items():
        for r in range(len(tokens)):
            worst = max(worst, ind.routing_regret(choice[r], trace.expert_ids[layer][r].numpy()))
    assert worst < 0.01, worst  # sigmoid scores in (0, 1): a flip needs a gap under one percent


def test_a_wrong_rule_is_visible(both):
    """Sanity of the comparison itself: a restatement with another routed scale disagrees far beyond the noise floor."""
    import dataclasses

    g, ckpt, tokens, trace, exact = both
    selected = {i: [r.numpy() for r in trace.selected[i]] for i in range(g.num_layers)}
    experts = {i: ids.numpy() for i, ids in trace.expert_ids.items()}
    wrong = ind.forward(dataclasses.replace(g, routed_scaling_factor=1.0), ckpt, tokens, selected, experts)
    span = np.abs(exact["logits"]).max()
    assert np.abs(wrong["logits"] - exact["logits"]).max() > 0.1 * span
