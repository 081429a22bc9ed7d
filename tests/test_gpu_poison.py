"""Poisoned padding and determinism (B200 only): NaN in cache rows that a kernel may touch but must not use never reaches an output,
and a kernel run twice on the same inputs gives the same bits.  Follows the reference's padded-panel test idea
(`tests/kernels/test_fp8_panel_matmul.py:48-50`): what lies outside the valid range is made toxic, not zero."""

import pytest
import torch

from glm_tpu_b200.oracle import contract

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf(x):
    return x.to(torch.bfloat16)


def test_attention_ignores_poisoned_unselected_rows_and_is_deterministic(native_lib):
    n = native_lib
    torch.manual_seed(12)
    H, L, rd, cap, top_k, rows = 64, 512, 64, 4096, 2048, 3
    W = L + rd
    q = _bf(torch.randn(rows, H, W) * 0.3)
    clean = _bf(torch.randn(1, 1, cap, W))
    sel = torch.full((rows, top_k), -1, dtype=torch.int32)
    counts = torch.zeros(rows, 2, dtype=torch.int32)
    picks = []
    for r, c in enumerate((2048, 130, 1)):
        p = torch.sort(torch.randperm(cap)[:c]).values
        sel[r, :c], counts[r] = p.to(torch.int32), c
        picks.append(p)
    used = torch.zeros(cap, dtype=torch.bool)
    used[torch.cat(picks)] = True
    poisoned = clean.clone()
    poisoned[0, 0, ~used] = float("nan")  # every cache row that no query selected
    lane = torch.zeros(rows, dtype=torch.int32, device=DEV)
    scale = float(torch.tensor(W**-0.5, dtype=torch.float32))
    chunks = -(-top_k // n.attn_chunk())
    outs = []
    for cache in (clean, poisoned, poisoned):
        part_o = torch.zeros(rows, chunks, H, L, device=DEV)
        part_ml = torch.zeros(rows, chunks, H, 2, device=DEV)
        o_split = torch.zeros(rows, H, L, dtype=torch.bfloat16, device=DEV)
        o_rows = torch.zeros(rows, H, L, dtype=torch.bfloat16, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        args = (q.to(DEV), cache.to(DEV), sel.to(DEV), counts.to(DEV), lane, rows, H, L, rd, 0, 1, cap, top_k)
        n.sparse_mla_partial(*args, chunks, scale, part_o, part_ml, status=status)
        n.attn_local_merge(part_o, part_ml, counts.to(DEV), rows, H, L, top_k, chunks, o_split, H)
        n.sparse_mla_rows(*args, scale, o_rows, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        outs.append((o_split.clone(), o_rows.clone()))
    for a, b in zip(outs[0], outs[1]):  # poison changes nothing, bit for bit
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    for a, b in zip(outs[1], outs[2]):  # and the same launch twice gives the same bits
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert not bool(torch.isnan(outs[1][1].float()).any())
    ref = contract.absorbed_attention_row(q[1, :, :L], q[1, :, L:], clean[0, 0], picks[1], scale)
    assert torch.allclose(outs[1][1][1].float().cpu(), ref.float(), rtol=2**-6, atol=4e-3)


@pytest.mark.parametrize("many", [False, True])
def test_indexer_ignores_poisoned_keys_past_the_context(native_lib, many):
    """The key tiles are 128 rows wide: a tile that straddles the end of a row's context also loads keys the row may not see."""
    n = native_lib
    torch.manual_seed(13)
    rows, IH, D, cap = 40, 32, 128, 2048
    q = (torch.randn(rows, IH, D) * 2.0).to(DEV)
    hw = (torch.randn(rows, IH) * 0.2).to(DEV)
    pos = torch.arange(700, 700 + rows, dtype=torch.int32, device=DEV)  # contexts 701..740: never a multiple of 128
    lane = torch.zeros(rows, dtype=torch.int32, device=DEV)
    clean = _bf(torch.randn(1, 1, cap, D))
    poisoned = clean.clone()
    poisoned[0, 0, 701:] = float("nan")  # everything at or past the smallest context's end... rows further on may see a few of them
    poisoned[0, 0, 701:741] = clean[0, 0, 701:741]  # ...so keep positions that some row of the chunk may legitimately use
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    res = []
    for keys in (clean, poisoned):
        out = torch.full((rows, cap), float("nan"), device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        extra = dict(pieces=torch.empty(n.indexer_rows_scratch_bytes(rows), dtype=torch.uint8, device=DEV), lane=0) if many else {}
        n.indexer_score(q, hw, keys.to(DEV), pos, lane, rows, IH, D, 0, 1, cap, 64, 1, 0, cap, cap, cap, scale, out, status=status, **extra)
        torch.cuda.synchronize()
        assert int(status.item()) == 0  # the non-finite check looks at scores inside the context only
        res.append(out)
    for r in range(rows):
        c = int(pos[r]) + 1
        assert torch.equal(res[0][r, :c], res[1][r, :c]) and not bool(torch.isnan(res[1][r, :c]).any())
        assert bool(torch.isnan(res[1][r, c:]).all())
