"""Layer-unit tier on the CPU: every rule of the numerical contract that a kernel could silently get wrong is pinned by a case built so
that the wrong rule gives a different answer (rounding order, pairing, tie rules, where a bias or a scale enters).

Mirrors the reference's layer tests (`tests/layers/test_norm.py`, `test_rope.py`, `test_fp8.py`, `tests/layers/moe/test_router.py`,
`tests/layers/attention/test_dsa_indexer.py`): the same rules, restated against this repository's CPU oracle.
"""

import numpy as np
import pytest
import torch

from glm_tpu_b200.oracle import contract

F32, BF16 = torch.float32, torch.bfloat16


# --------------------------------------------------------------------------------------------------- FP8 weight decode
def test_fp8_decode_is_exact_for_all_256_codes():
    """Every e4m3fn code against the value computed from its bit fields; the two NaN codes stay NaN; there is no infinity."""
    codes = torch.arange(256, dtype=torch.uint8).reshape(1, 256)
    got = contract.dequantize_fp8(codes, torch.ones(1, 1), (1, 256)).to(F32)[0]
    for c in range(256):
        sign, exp, man = -1.0 if c & 0x80 else 1.0, (c >> 3) & 0xF, c & 7
        if exp == 15 and man == 7:
            assert torch.isnan(got[c])
            continue
        want = sign * (man / 8.0) * 2.0**-6 if exp == 0 else sign * (1 + man / 8.0) * 2.0 ** (exp - 7)
        assert float(got[c]) == want, c
    assert float(got[0x7E]) == 448.0 and not bool(torch.isinf(got).any())


def test_fp8_decode_rounds_after_the_scale_and_uses_the_block_of_each_element():
    bits = torch.tensor([[0x3F, 0x3F, 0x3F, 0x3F]], dtype=torch.uint8)  # 1.875 four times, blocks of two columns
    scale = torch.tensor([[1.0 / 7.0, 3.0]])
    got = contract.dequantize_fp8(bits, scale, (1, 2)).to(F32)[0]
    third = np.float32(1.875) * np.float32(1.0 / 7.0)
    assert float(got[0]) == float(torch.tensor(third).to(BF16)) and float(got[1]) == float(got[0])
    assert float(got[2]) == 5.625 and float(got[3]) == 5.625
    assert float(got[0]) != float(third)  # the product is not representable: the bf16 rounding is part of the contract


# --------------------------------------------------------------------------------------------------- norms
def test_rms_norm_rounds_before_the_weight():
    """bf16(bf16(x * inv) * w) differs from bf16(x * inv * w) on a value built for it."""
    torch.manual_seed(0)
    x = torch.randn(64, 256) * 3
    w = (1 + 0.3 * torch.randn(256)).to(BF16)
    got = contract.rms_norm(x, w, 1e-5)
    inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)
    single = contract.bf16_round(x * inv * w.to(F32))
    double = contract.bf16_round(contract.bf16_round(x * inv) * w.to(F32))
    assert torch.equal(got, double)
    assert not torch.equal(single, double)  # the fixture does see the rounding order


def test_add_rms_norm_feeds_the_unrounded_sum_and_carries_the_rounded_one():
    torch.manual_seed(1)
    update, residual = (torch.randn(32, 128) * 2).to(BF16), (torch.randn(32, 128) * 50).to(BF16)
    w = torch.ones(128, dtype=BF16)
    normed, carried = contract.add_rms_norm(update, residual, w, 1e-5)
    s = update.to(F32) + residual.to(F32)
    assert torch.equal(carried, contract.bf16_round(s))
    assert torch.equal(normed, contract.rms_norm(s, w, 1e-5))
    assert not torch.equal(normed, contract.rms_norm(contract.bf16_round(s), w, 1e-5))  # norm of the ROUNDED sum is a different function
    first, same = contract.add_rms_norm(None, residual, w, 1e-5)
    assert torch.equal(same, residual.to(F32)) and torch.equal(first, contract.rms_norm(residual, w, 1e-5))


# --------------------------------------------------------------------------------------------------- RoPE
def test_rope_pairs_are_interleaved_and_position_zero_is_identity():
    table = contract.rope_table(64, 8, 10000.0)
    x = torch.arange(1, 9, dtype=F32).reshape(1, 1, 8)
    assert torch.equal(contract.rope_interleaved_table(x, torch.tensor([0]), table), x)
    y = contract.rope_interleaved_table(x, torch.tensor([5]), table)[0, 0]
    cos, sin = table[5, :4].to(F32), table[5, 4:].to(F32)
    for j in range(4):  # pair (2j, 2j+1), not (j, j + 4)
        assert float(y[2 * j]) == float(contract.bf16_round(x[0, 0, 2 * j] * cos[j] - x[0, 0, 2 * j + 1] * sin[j]))
        assert float(y[2 * j + 1]) == float(contract.bf16_round(x[0, 0, 2 * j + 1] * cos[j] + x[0, 0, 2 * j] * sin[j]))


def test_rope_table_is_built_in_fp32_and_stored_in_bf16():
    table = contract.rope_table(4096, 64, 8e6)
    assert table.dtype == BF16 and table.shape == (4096, 64)
    j = np.arange(0, 64, 2, dtype=np.float32)
    inv = (np.float32(1) / np.power(np.float32(8e6), j / np.float32(64))).astype(np.float32)
    angle = np.float32(4095) * inv
    assert torch.equal(table[4095, :32], torch.from_numpy(np.cos(angle).astype(np.float32)).to(BF16))
    assert torch.equal(table[4095, 32:], torch.from_numpy(np.sin(angle).astype(np.float32)).to(BF16))


def test_indexer_rope_stays_fp32_and_touches_only_the_rope_features():
    torch.manual_seed(2)
    x = torch.randn(3, 4, 32)
    y = contract.rope_interleaved_fp32(x, torch.tensor([0, 7, 1000]), 8e6, 16)
    assert y.dtype == F32 and torch.equal(y[..., 16:], x[..., 16:]) and torch.equal(y[0], x[0])
    assert not torch.equal(contract.bf16_round(y[1:, :, :16]), y[1:, :, :16])  # no rounding to bf16 happened
    norms = (y[..., 0:16:2] ** 2 + y[..., 1:16:2] ** 2, x[..., 0:16:2] ** 2 + x[..., 1:16:2] ** 2)
    assert torch.allclose(*norms, rtol=1e-5)  # a rotation


# --------------------------------------------------------------------------------------------------- DSA top-k
def test_top_k_is_exact_ascending_and_breaks_ties_toward_the_lowest_position():
    scores = torch.tensor([1.0, 5.0, 5.0, -2.0, 5.0, 0.0, 5.0, 3.0])
    assert contract.top_k_positions(scores, 8, 3).tolist() == [1, 2, 4]          # four fives: the three lowest positions
    assert contract.top_k_positions(scores, 8, 5).tolist() == [1, 2, 4, 6, 7]
    assert contract.top_k_positions(scores, 3, 5).tolist() == [0, 1, 2]          # short context: everything
    assert contract.top_k_positions(scores, 6, 2).tolist() == [1, 2]             # positions past the context do not exist


def test_top_k_orders_signed_zeros_and_negative_values_like_the_bit_key():
    scores = torch.tensor([-0.0, 0.0, -1e-30, 1e-30, -3.0])
    key = contract.orderable_key(scores)
    assert key[3] > key[1] > key[0] > key[2] > key[4]  # +tiny > +0 > -0 > -tiny > -3
    assert contract.top_k_positions(scores, 5, 2).tolist() == [1, 3]
    assert contract.top_k_positions(torch.tensor([-0.0, 0.0, -0.0, 0.0]), 4, 1).tolist() == [1]


@pytest.mark.parametrize("seed", range(4))
def test_top_k_matches_a_sort_on_skewed_scores_with_many_ties(seed):
    gen = torch.Generator().manual_seed(seed)
    scores = torch.randint(0, 12, (3000,), generator=gen).to(F32) * 0.25 - 1.0  # twelve distinct values: the boundary is one big tie
    got = contract.top_k_positions(scores, 2900, 512).tolist()
    want = sorted(sorted(range(2900), key=lambda i: (-float(scores[i]), i))[:512])
    assert got == want


# --------------------------------------------------------------------------------------------------- router
def test_router_bias_chooses_but_does_not_weigh():
    x = torch.tensor([[1.0, 0.0, 0.0, 0.0]])
    weight = torch.tensor([[2.0, 0, 0, 0], [1.0, 0, 0, 0], [0.0, 0, 0, 0], [-1.0, 0, 0, 0]])
    bias = torch.tensor([0.0, 0.0, 0.0, 10.0])  # lifts the worst expert into the choice
    ids, weights, choice = contract.router(x, weight, bias, 2)
    assert ids.tolist() == [[3, 0]]
    s = torch.sigmoid(torch.tensor([2.0, 1.0, 0.0, -1.0]))
    assert torch.allclose(weights, torch.stack([s[3], s[0]])[None] / (s[3] + s[0]))  # unbiased scores, normalised over the chosen
    assert float(choice[0, 3]) == float(s[3] + 10.0)
    assert abs(float(weights.sum()) - 1.0) < 1e-6  # the routed scaling factor is not applied here


def test_router_ties_go_to_the_lowest_expert_id_and_imposed_ids_are_honoured():
    x = torch.ones(2, 3)
    weight = torch.zeros(6, 3)  # every expert scores sigmoid(0) = 0.5
    ids, weights, _ = contract.router(x, weight, torch.zeros(6), 3)
    assert ids.tolist() == [[0, 1, 2], [0, 1, 2]] and torch.allclose(weights, torch.full((2, 3), 1 / 3))
    imposed = torch.tensor([[5, 4, 0], [2, 2, 1]])
    ids2, weights2, _ = contract.router(x, weight, torch.zeros(6), 3, imposed=imposed)
    assert torch.equal(ids2, imposed.long()) and torch.allclose(weights2, torch.full((2, 3), 1 / 3))


# --------------------------------------------------------------------------------------------------- sampler, linear, activation
def test_greedy_ties_go_to_the_lowest_token_id():
    logits = torch.tensor([[0.5, 2.0, 2.0, -1.0], [3.0, 3.0, 3.0, 3.0], [-5.0, -7.0, -5.0, -6.0]]).to(BF16).to(F32)
    assert contract.greedy(logits).tolist() == [1, 0, 0]


def test_linear_accumulates_in_fp32_and_rounds_once():
    x = torch.tensor([[256.0, 1.0, 1.0, 1.0]]).to(BF16)
    w = torch.tensor([[1.0, 1.0, 1.0, 1.0]]).to(BF16)
    assert float(contract.linear(x, w, out_bf16=False)) == 259.0      # a bf16 accumulator would lose the ones
    assert float(contract.linear(x, w)) == 260.0                       # one rounding of 259 to 8 significant bits (even)


def test_swiglu_rounds_once_after_the_product():
    g, u = torch.tensor([1.7109375]), torch.tensor([0.33203125])
    want = contract.bf16_round(g * torch.sigmoid(g) * u)
    assert torch.equal(contract.swiglu_act(g, u), want)
    torch.manual_seed(4)
    gs, us = torch.randn(4096) * 3, torch.randn(4096)
    stepwise = contract.bf16_round(contract.bf16_round(gs * torch.sigmoid(gs)) * us)
    assert not torch.equal(contract.swiglu_act(gs, us), stepwise)  # rounding the SiLU first is a different function
    assert contract.swiglu_act(torch.zeros(1), u).item() == 0.0


# --------------------------------------------------------------------------------------------------- attention row
def test_attention_row_uses_only_the_selected_rows_in_any_order():
    torch.manual_seed(3)
    H, L, rd, n = 4, 16, 8, 40
    q_c, q_r = contract.bf16_round(torch.randn(H, L)), contract.bf16_round(torch.randn(H, rd))
    cache = contract.bf16_round(torch.randn(n, L + rd))
    sel = torch.tensor([3, 9, 17, 30])
    scale = float(np.float32((L + rd) ** -0.5))
    out = contract.absorbed_attention_row(q_c, q_r, cache, sel, scale)
    poisoned = cache.clone()
    poisoned[[i for i in range(n) if i not in sel.tolist()]] = float("nan")
    assert torch.equal(out, contract.absorbed_attention_row(q_c, q_r, poisoned, sel, scale))
    s = (q_c @ cache[sel, :L].T + q_r @ cache[sel, L:].T) * scale
    p = torch.softmax(s, dim=-1)
    assert torch.allclose(out.to(F32), p @ cache[sel, :L], rtol=2**-6, atol=2**-7)
    assert out.shape == (H, L)
