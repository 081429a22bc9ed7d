"""The many-rows tcgen05 indexer (prefill chunks) against the fp32 restatement and, bit for bit, against the one-row kernel (B200 only)."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference(q, hw, keys, scale):
    dots = torch.einsum("hd,td->ht", q.float(), keys.float()) * scale
    return (hw[:, None] * torch.relu(dots)).sum(0)


@pytest.mark.parametrize("stripe,world,rank", [(64, 1, 0), (64, 2, 1)])
def test_rows_indexer_matches_reference_and_one_row_kernel(native_lib, stripe, world, rank):
    n = native_lib
    torch.manual_seed(23)
    rows, IH, D, cap = 300, 32, 128, 4096
    lanes, slots, slot, lane_id = 2, 2, 1, 1
    local_cap = cap // world
    q = (torch.randn(rows, IH, D) * 2.0).to(DEV)
    hw = (torch.randn(rows, IH) * 0.2).to(DEV)
    keys = torch.randn(lanes, slots, local_cap, D).to(torch.bfloat16).to(DEV)
    # a chunk of a prompt (ascending positions) with a few out-of-order rows: the kernel may not rely on the order
    pos = torch.arange(1500, 1500 + rows, dtype=torch.int32)
    pos[7], pos[200], pos[299] = 3, 4095, 64
    pos = pos.to(DEV)
    lane = torch.full((rows,), lane_id, dtype=torch.int32, device=DEV)
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    max_ctx = cap
    one = torch.full((rows, cap), float("nan"), device=DEV)
    n.indexer_score(q, hw, keys, pos, lane, rows, IH, D, slot, slots, local_cap, stripe, world, rank, cap, max_ctx, cap, scale, one)
    many = torch.full((rows, cap), float("nan"), device=DEV)
    pieces = torch.empty(n.indexer_rows_scratch_bytes(rows), dtype=torch.uint8, device=DEV)
    n.indexer_score(q, hw, keys, pos, lane, rows, IH, D, slot, slots, local_cap, stripe, world, rank, cap, max_ctx, cap, scale, many,
                    pieces=pieces, lane=lane_id)
    torch.cuda.synchronize()
    assert torch.equal(torch.isnan(one), torch.isnan(many))          # the same positions are written, nothing else is touched
    assert torch.equal(one.nan_to_num(0.0), many.nan_to_num(0.0))    # and bit for bit the same scores
    page = stripe * world
    for r in (0, 7, 150, 200, 299):
        ctx = int(pos[r]) + 1
        mine = [g for g in range(ctx) if (g // stripe) % world == rank]
        if not mine:
            assert torch.isnan(many[r]).all()
            continue
        local = torch.tensor([(g // page) * stripe + g % stripe for g in mine], dtype=torch.long, device=DEV)
        ref = _reference(q[r], hw[r], keys[lane_id, slot, local], scale)
        assert torch.allclose(many[r, mine], ref, rtol=1e-4, atol=1e-4), (r, (many[r, mine] - ref).abs().max().item())


def test_rows_indexer_rotates_a_raw_query_like_the_one_row_kernel(native_lib):
    n = native_lib
    torch.manual_seed(29)
    rows, IH, D, cap, rd, lead = 64, 32, 128, 2048, 64, 96
    q_proj = (torch.randn(rows, lead + IH * D) * 0.7).to(DEV)
    inv_freq = torch.pow(torch.tensor(8e6), -torch.arange(0, rd, 2, dtype=torch.float32) / rd).to(DEV)
    hw = (torch.randn(rows, IH) * 0.2).to(DEV)
    keys = torch.randn(1, 1, cap, D).to(torch.bfloat16).to(DEV)
    pos = torch.arange(cap - rows, cap, dtype=torch.int32, device=DEV)
    lane = torch.zeros(rows, dtype=torch.int32, device=DEV)
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    one = torch.full((rows, cap), float("nan"), device=DEV)
    n.indexer_score(None, hw, keys, pos, lane, rows, IH, D, 0, 1, cap, 64, 1, 0, cap, cap, cap, scale, one, q_raw=q_proj, q_offset=lead,
                    inv_freq=inv_freq, rd=rd)
    many = torch.full((rows, cap), float("nan"), device=DEV)
    pieces = torch.empty(n.indexer_rows_scratch_bytes(rows), dtype=torch.uint8, device=DEV)
    n.indexer_score(None, hw, keys, pos, lane, rows, IH, D, 0, 1, cap, 64, 1, 0, cap, cap, cap, scale, many, q_raw=q_proj, q_offset=lead,
                    inv_freq=inv_freq, rd=rd, pieces=pieces, lane=0)
    torch.cuda.synchronize()
    assert torch.equal(torch.isnan(one), torch.isnan(many))
    assert torch.equal(one.nan_to_num(0.0), many.nan_to_num(0.0))
    assert bool((many[-1, :cap] != 0).any())


def test_rows_indexer_is_stable_over_many_launches(native_lib):
    """The accumulator ring is shared by several issuing threads and two epilogue groups: repeated launches on a deep context (every
    CTA walks 128 rows x 4 key tiles) must keep giving bit-identical scores and a clean status word."""
    n = native_lib
    torch.manual_seed(31)
    rows, IH, D, cap = 512, 32, 128, 8192
    q = (torch.randn(rows, IH, D) * 2.0).to(DEV)
    hw = (torch.randn(rows, IH) * 0.2).to(DEV)
    keys = torch.randn(1, 1, cap, D).to(torch.bfloat16).to(DEV)
    pos = torch.arange(cap - rows, cap, dtype=torch.int32, device=DEV)
    lane = torch.zeros(rows, dtype=torch.int32, device=DEV)
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pieces = torch.empty(n.indexer_rows_scratch_bytes(rows), dtype=torch.uint8, device=DEV)
    first = None
    noise = torch.empty(64 << 20, dtype=torch.uint8, device=DEV)
    for it in range(40):
        out = torch.full((rows, cap), float("nan"), device=DEV)
        if it % 3 == 0:
            noise.fill_(it)  # vary what is in L2 and how the CTAs' loads are timed
        n.indexer_score(q, hw, keys, pos, lane, rows, IH, D, 0, 1, cap, 64, 1, 0, cap, cap, cap, scale, out, status=status, pieces=pieces, lane=0)
        if first is None:
            first = out
        else:
            assert torch.equal(first.nan_to_num(0.0), out.nan_to_num(0.0)), it
    assert int(status.item()) == 0
    one = torch.full((64, cap), float("nan"), device=DEV)
    n.indexer_score(q[:64].contiguous(), hw[:64].contiguous(), keys, pos[:64].contiguous(), lane[:64].contiguous(), 64, IH, D, 0, 1, cap, 64, 1, 0, cap, cap,
                    cap, scale, one)
    assert torch.equal(one.nan_to_num(0.0), first[:64].nan_to_num(0.0))
