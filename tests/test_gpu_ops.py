"""Numerics of each CUDA kernel against the plain-PyTorch fp32 restatement of the same operation (B200 only)."""

import pytest
import torch

from glm_tpu_b200.oracle import contract

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bf(x):
    return x.to(torch.bfloat16)


def close(a, b, rtol=2**-7, atol=1e-5):
    a, b = a.float().cpu(), b.float().cpu()
    return torch.allclose(a, b, rtol=rtol, atol=atol), (a - b).abs().max().item()


@pytest.mark.parametrize("rows", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(96, 256), (2784, 6144), (37, 64)])
def test_skinny_bf16(native_lib, rows, N, K):
    n = native_lib
    torch.manual_seed(0)
    x = bf(torch.randn(rows, K, device=DEV))
    w = bf(torch.randn(N, K, device=DEV) * 0.05)
    ref = x.float() @ w.float().T
    out = torch.zeros(rows, N, device=DEV)
    n.skinny_bf16(x, w, out, n.SK_OUT_F32)
    ok, err = close(out, ref, rtol=1e-4, atol=1e-3)
    assert ok, err
    out16 = torch.zeros(rows, N, dtype=torch.bfloat16, device=DEV)
    n.skinny_bf16(x, w, out16, n.SK_OUT_BF16)
    ok, err = close(out16, bf(ref), rtol=2**-7, atol=1e-3)
    assert ok, err
    out_ar = torch.zeros(rows, N, dtype=torch.bfloat16, device=DEV)
    n.skinny_bf16(x, w, out_ar, n.SK_OUT_ALLREDUCE_BF16)  # single GPU: plain store
    assert torch.equal(out_ar, out16)


def test_skinny_batched_heads(native_lib):
    n = native_lib
    torch.manual_seed(1)
    rows, heads, L, v, nope = 4, 8, 128, 64, 64
    o_lat = bf(torch.randn(rows, heads, L, device=DEV))
    kv_b = bf(torch.randn(heads, nope + v, L, device=DEV) * 0.1)
    out = torch.zeros(rows, heads * v, dtype=torch.bfloat16, device=DEV)
    n.skinny_bf16(o_lat, kv_b[:, nope:, :], out, n.SK_OUT_BF16, rows=rows, N=v, K=L, xs=heads * L, ws=L, os_=heads * v, batch=heads,
                  xb=L, wb=(nope + v) * L, ob=v)
    ref = torch.einsum("rhc,hvc->rhv", o_lat.float(), kv_b[:, nope:, :].float()).reshape(rows, heads * v)
    ok, err = close(out, bf(ref), atol=1e-2)
    assert ok, err


def test_swiglu(native_lib):
    n = native_lib
    torch.manual_seed(2)
    rows, N, K = 4, 200, 512
    x = bf(torch.randn(rows, K, device=DEV))
    wg, wu = bf(torch.randn(N, K, device=DEV) * 0.05), bf(torch.randn(N, K, device=DEV) * 0.05)
    act = torch.zeros(rows, N, dtype=torch.bfloat16, device=DEV)
    n.skinny_bf16_swiglu(x, wg, wu, act)
    ref = contract.swiglu_act(contract.linear(x.cpu(), wg.cpu()), contract.linear(x.cpu(), wu.cpu()))
    ok, err = close(act, ref, rtol=2**-6, atol=2e-3)
    assert ok, err


def test_fp8_decode_is_bit_exact(native_lib):
    n = native_lib
    torch.manual_seed(3)
    bits = torch.randint(0, 256, (300, 520), dtype=torch.uint8)
    bits[(bits & 0x7F) == 0x7F] = 0x3C  # no NaN codes
    scale = torch.rand(3, 5) * 0.01 + 1e-4
    ref = contract.dequantize_fp8(bits, scale)
    out = torch.zeros(300, 520, dtype=torch.bfloat16, device=DEV)
    n.fp8_to_bf16(bits.to(DEV), scale.to(DEV), out)
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))


def test_add_rmsnorm(native_lib):
    n = native_lib
    torch.manual_seed(4)
    rows, H = 5, 6144
    upd, res, w = bf(torch.randn(rows, H)), bf(torch.randn(rows, H)), bf(torch.randn(H) * 0.1 + 1)
    ref_x, ref_res = contract.add_rms_norm(upd, res, w, 1e-5)
    d_res, out = res.to(DEV).clone(), torch.zeros(rows, H, dtype=torch.bfloat16, device=DEV)
    n.add_rmsnorm(upd.to(DEV), d_res, w.to(DEV), out, 1e-5)
    assert torch.equal(d_res.cpu().float(), ref_res)
    mism = (out.cpu().float() != ref_x).float().mean().item()
    ok, err = close(out, ref_x, rtol=2**-7, atol=1e-6)
    assert ok and mism < 0.01, (err, mism)
    d_res2 = res.to(DEV).clone()
    n.add_rmsnorm(None, d_res2, w.to(DEV), out, 1e-5)
    ref_x2, _ = contract.add_rms_norm(None, res, w, 1e-5)
    ok, err = close(out, ref_x2, rtol=2**-7, atol=1e-6)
    assert ok, err


def _routed_fixture(E, I, H, seed):
    from glm_tpu_b200.models.glm_moe_dsa.weights import quantize_fp8

    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in (("gate", (E, I, H)), ("up", (E, I, H)), ("down", (E, H, I))):
        bits, scale = quantize_fp8(torch.randn(shape, generator=gen) * 0.05, (128, 128), gen)
        out[name] = (bits, scale)
    return out


@pytest.mark.parametrize("mma", [1, 0], ids=["mma_sync", "fp32_fma"])
@pytest.mark.parametrize("rows,tiled", [(3, False), (40, True), (40, "sort_kernel"), (150, "sort_kernel")])
def test_routed_experts(native_lib, rows, tiled, mma):
    n = native_lib
    n.set_moe_mma(mma)
    torch.manual_seed(5)
    E, I, H, tk = 8, 256, 512, 2
    fx = _routed_fixture(E, I, H, 5)
    x = bf(torch.randn(rows, H) * 0.5)
    ids = torch.stack([torch.randperm(E)[:tk] for _ in range(rows)]).to(torch.int32)
    wts = torch.rand(rows, tk)
    wts = wts / wts.sum(-1, keepdim=True)
    deq = {k: contract.dequantize_fp8(*v) for k, v in fx.items()}
    ref = torch.zeros(rows * tk, H)
    for r in range(rows):
        for s in range(tk):
            e = int(ids[r, s])
            act = contract.swiglu_act(contract.linear(x[r : r + 1], deq["gate"][e]), contract.linear(x[r : r + 1], deq["up"][e]))
            ref[r * tk + s] = contract.bf16_round(contract.linear(act, deq["down"][e])[0] * contract.bf16_round(wts[r, s]))
    d = {k: (v[0].to(DEV), v[1].to(DEV)) for k, v in fx.items()}
    act = torch.zeros(rows * tk, I, dtype=torch.bfloat16, device=DEV)
    dw = torch.zeros(rows * tk, H, dtype=torch.bfloat16, device=DEV)
    ids_d, w_d, x_d = ids.to(DEV), wts.to(DEV), x.to(DEV)
    if tiled:
        from glm_tpu_b200.models.glm_moe_dsa.model import GlmMoeDsaModel

        te, tr, nt, tiles, rt = GlmMoeDsaModel._route_tiles(None, ids_d, E)
        if tiled == "sort_kernel":  # the one-launch sort gives the same tiles as the library-op sort
            te2 = torch.full((tiles,), -7, dtype=torch.int32, device=DEV)
            tr2 = torch.full((tiles, 8), -7, dtype=torch.int32, device=DEV)
            nt2, scratch = torch.zeros(1, dtype=torch.int32, device=DEV), torch.empty(rows * tk, dtype=torch.int32, device=DEV)
            n.route_sort8(ids_d, 0, E, te2, tr2, nt2, scratch)
            live = int(nt2)
            assert live == int(nt) and torch.equal(te2, te) and torch.equal(tr2[:live], tr[:live])
            te, tr, nt = te2, tr2, nt2
    else:
        te, tr, nt, tiles, rt = ids_d, None, None, rows * tk, 1
    n.moe_gateup_fp8(x_d, tk, te, tr, nt, tiles, rt, d["gate"][0], d["up"][0], d["gate"][1], d["up"][1], 0, act)
    n.moe_down_fp8(act, w_d, te, tr, nt, tiles, rt, d["down"][0], d["down"][1], 0, dw)
    n.set_moe_mma(1)
    ok, err = close(dw, ref, rtol=2**-5, atol=2e-3)
    assert ok, err
    # combine on one GPU: route sum, scale, shared
    shared = torch.randn(rows, H)
    out = torch.zeros(rows, H, dtype=torch.bfloat16, device=DEV)
    n.moe_combine(dw, ids_d, shared.to(DEV), rows, tk, H, 0, E, 2.5, False, out)
    routed = dw.float().cpu().reshape(rows, tk, H).sum(1)
    ref_out = contract.bf16_round(contract.bf16_round(contract.bf16_round(routed) * 2.5) + contract.bf16_round(shared))
    ok, err = close(out, ref_out, rtol=2**-7, atol=1e-3)
    assert ok, err


@pytest.mark.parametrize("rows,tk", [(1, 8), (4, 8), (8, 2), (11, 8)])
def test_down_combine_in_one_launch_equals_the_two_launches(native_lib, rows, tk):
    """Column-sliced experts: the fused down + route sum + shared + (one-GPU) all-reduce kernel against ``moe_down_fp8`` followed by
    ``moe_combine`` (same roundings; the fp32 sum over K runs in another order, so a value may land on the neighbouring bf16) and
    against a plain fp32 computation."""
    n = native_lib
    torch.manual_seed(9)
    E, I, H = 16, 256, 512
    fx = _routed_fixture(E, I, H, 9)
    d = {k: (v[0].to(DEV), v[1].to(DEV)) for k, v in fx.items()}
    ids = torch.stack([torch.randperm(E)[:tk] for _ in range(rows)]).to(torch.int32).to(DEV)
    wts = torch.rand(rows, tk)
    wts = (wts / wts.sum(-1, keepdim=True)).to(DEV)
    act = bf(torch.randn(rows * tk, I) * 0.3).to(DEV)
    shared = torch.randn(rows, H).to(DEV)
    dw = torch.zeros(rows * tk, H, dtype=torch.bfloat16, device=DEV)
    two = torch.zeros(rows, H, dtype=torch.bfloat16, device=DEV)
    one = torch.zeros(rows, H, dtype=torch.bfloat16, device=DEV)
    n.moe_down_fp8(act, wts, ids, None, None, rows * tk, 1, d["down"][0], d["down"][1], 0, dw)
    n.moe_combine(dw, ids, shared, rows, tk, H, 0, E, 2.5, False, two)
    n.moe_down_combine(act, wts, ids, d["down"][0], d["down"][1], shared, rows, tk, 2.5, one)
    torch.cuda.synchronize()
    ok, err = close(one, two.float().cpu(), rtol=2**-7, atol=2e-3)
    assert ok, err
    assert (one != two).float().mean().item() < 0.25  # a near-tie at one of the sixteen bf16 roundings per value
    deq = contract.dequantize_fp8(*fx["down"])
    routed = torch.zeros(rows, H)
    for r in range(rows):
        for s_ in range(tk):
            p = r * tk + s_
            routed[r] += (act[p].float().cpu() @ deq[int(ids[r, s_])].float().T) * float(wts[r, s_])
    ref = routed * 2.5 + shared.cpu()
    ok, err = close(one, ref, rtol=2**-6, atol=3e-2)  # sixteen bf16 roundings of terms around 0.5, scaled by 2.5
    assert ok, err


@pytest.mark.parametrize("rows,H,L,nope,v,counts", [(1, 8, 512, 192, 256, [2048]), (4, 8, 512, 192, 256, [2048, 70, 0, 1300]),
                                                     (2, 4, 128, 64, 64, [32, 17]), (1, 16, 64, 32, 34, [16])])
def test_merge_and_value_projection_in_one_launch(native_lib, rows, H, L, nope, v, counts):
    """``attn_merge_vproj`` against ``attn_local_merge`` followed by the batched ``skinny_bf16`` (the same bits), and against fp32."""
    n = native_lib
    torch.manual_seed(21)
    top_k = max(max(counts), 16)
    chunks = -(-top_k // n.attn_chunk())
    part_o = torch.randn(rows, chunks, H, L, device=DEV)
    part_ml = torch.stack([torch.randn(rows, chunks, H, device=DEV) * 3, torch.rand(rows, chunks, H, device=DEV) * 60 + 1], dim=-1).contiguous()
    cnt = torch.tensor([[c, c] for c in counts], dtype=torch.int32, device=DEV)
    kv_b = bf(torch.randn(H, nope + v, L, device=DEV) * 0.05)
    o_two = torch.full((rows, H, L), float("nan"), dtype=torch.bfloat16, device=DEV)
    v_two = torch.full((rows, H * v), float("nan"), dtype=torch.bfloat16, device=DEV)
    n.attn_local_merge(part_o, part_ml, cnt, rows, H, L, top_k, chunks, o_two, H)
    n.skinny_bf16(o_two, kv_b[:, nope:, :], v_two, n.SK_OUT_BF16, rows=rows, N=v, K=L, xs=H * L, ws=L, os_=H * v, batch=H, xb=L,
                  wb=(nope + v) * L, ob=v)
    o_one, v_one = torch.full_like(o_two, float("nan")), torch.full_like(v_two, float("nan"))
    n.attn_merge_vproj(part_o, part_ml, cnt, rows, H, L, top_k, chunks, kv_b, nope, o_one, v_one)
    torch.cuda.synchronize()
    assert torch.equal(o_one, o_two) and torch.equal(v_one, v_two)
    # plain fp32: softmax-style merge of the partials, then the projection
    used = torch.tensor([-(-c // n.attn_chunk()) for c in counts], device=DEV)
    live = torch.arange(chunks, device=DEV)[None, :, None] < used[:, None, None]
    m = torch.where(live, part_ml[..., 0], torch.full_like(part_ml[..., 0], -float("inf")))
    w = torch.where(live, torch.exp(m - m.amax(dim=1, keepdim=True).clamp_min(-1e30)), torch.zeros_like(m))
    den = (w * part_ml[..., 1]).sum(1)
    o_ref = torch.where(den[..., None] > 0, (w[..., None] * part_o).sum(1) / den[..., None].clamp_min(1e-30), torch.zeros(1, device=DEV))
    ok, err = close(o_one, o_ref, rtol=2**-7, atol=1e-3)
    assert ok, err
    v_ref = torch.einsum("rhc,hvc->rhv", bf(o_ref).float(), kv_b[:, nope:, :].float()).reshape(rows, H * v)
    ok, err = close(v_one, v_ref, rtol=2**-6, atol=2e-2)
    assert ok, err


def test_router_topk(native_lib):
    n = native_lib
    torch.manual_seed(6)
    rows, E, H, tk = 7, 256, 512, 8
    x, w = bf(torch.randn(rows, H)), bf(torch.randn(E, H) * 0.05)
    bias = torch.randn(E) * 0.02
    logits = (x.float() @ w.float().T)
    ids_ref, w_ref, _ = contract.router(x, w, bias, tk)
    ids = torch.zeros(rows, tk, dtype=torch.int32, device=DEV)
    wts = torch.zeros(rows, tk, device=DEV)
    n.router_topk(logits.to(DEV), bias.to(DEV), tk, ids, wts)
    assert torch.equal(ids.cpu().long(), ids_ref), (ids.cpu(), ids_ref)
    ok, err = close(wts, w_ref, rtol=1e-5, atol=1e-6)
    assert ok, err
    # exact ties go to the lowest expert id
    flat = torch.zeros(1, E)
    n.router_topk(flat.to(DEV), torch.zeros(E, device=DEV), tk, ids, wts)
    assert ids[0].cpu().tolist() == list(range(tk))


@pytest.fixture(params=[1, 0], ids=["cluster8", "single_cta"])
def topk_kernel(request, native_lib):
    """Both selection kernels behind the one entry point: the 8-CTA cluster (distributed shared memory) and the single CTA."""
    native_lib.set_topk_cluster(request.param)
    yield request.param
    native_lib.set_topk_cluster(1)


@pytest.mark.parametrize("n_ctx,top_k", [(10, 16), (100, 16), (5000, 2048), (32768, 2048), (2049, 2048), (7, 2048)])
def test_topk_select_exact_with_ties(native_lib, topk_kernel, n_ctx, top_k):
    n = native_lib
    torch.manual_seed(7)
    cap = 32768
    # coarse values force many ties at the boundary; include signed zeros
    scores = (torch.randn(2, cap) * 3).round() / 4
    scores[0, :50] = 0.0
    scores[0, 50:60] = -0.0
    pos = torch.tensor([n_ctx - 1, max(n_ctx // 2, 1) - 1], dtype=torch.int32)
    sel_g = torch.zeros(2, top_k, dtype=torch.int32, device=DEV)
    sel_l = torch.zeros(2, top_k, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(2, 2, dtype=torch.int32, device=DEV)
    n.topk_select(scores.to(DEV), pos.to(DEV), 2, cap, cap, top_k, 64, 1, 0, sel_g, sel_l, cnt)
    for r in range(2):
        ctx = int(pos[r]) + 1
        ref = contract.top_k_positions(scores[r], ctx, top_k)
        k = ref.numel()
        assert cnt[r].cpu().tolist() == [k, k]
        assert torch.equal(sel_g[r, :k].cpu().long(), ref)
        assert (sel_g[r, k:] == -1).all()
        assert torch.equal(sel_l[r, :k].cpu().long(), ref)  # one GPU: local row == position


def test_topk_select_striped_ownership(native_lib, topk_kernel):
    n = native_lib
    torch.manual_seed(8)
    cap, top_k, stripe, world = 4096, 256, 64, 4
    scores = torch.randn(1, cap)
    pos = torch.tensor([3000], dtype=torch.int32)
    ref = contract.top_k_positions(scores[0], 3001, top_k)
    for rank in range(world):
        sel_g = torch.zeros(1, top_k, dtype=torch.int32, device=DEV)
        sel_l = torch.zeros(1, top_k, dtype=torch.int32, device=DEV)
        cnt = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
        n.topk_select(scores.to(DEV), pos.to(DEV), 1, cap, cap, top_k, stripe, world, rank, sel_g, sel_l, cnt)
        assert torch.equal(sel_g[0].cpu().long(), ref)
        mine = ref[(ref // stripe) % world == rank]
        local = (mine // (stripe * world)) * stripe + mine % stripe
        assert int(cnt[0, 1]) == mine.numel()
        assert torch.equal(sel_l[0, : mine.numel()].cpu().long(), local)


def test_topk_select_long_context_all_equal(native_lib, topk_kernel):
    """A 166,912-slot row (beyond what one CTA can stage) where every score ties: the lowest positions win, in order."""
    n = native_lib
    cap, top_k = 166912, 2048
    scores = torch.full((1, cap), 0.25)
    scores[0, 100000:100010] = 0.5
    pos = torch.tensor([150000], dtype=torch.int32)
    sel_g = torch.zeros(1, top_k, dtype=torch.int32, device=DEV)
    sel_l = torch.zeros(1, top_k, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    n.topk_select(scores.to(DEV), pos.to(DEV), 1, cap, cap, top_k, 64, 1, 0, sel_g, sel_l, cnt)
    want = list(range(top_k - 10)) + list(range(100000, 100010))
    assert sel_g[0].cpu().tolist() == want and cnt[0].cpu().tolist() == [top_k, top_k]


def test_indexer_score(native_lib):
    n = native_lib
    torch.manual_seed(9)
    rows, IH, D, cap, ctx = 2, 32, 128, 4096, 3000
    q = torch.randn(rows, IH, D)
    hw = torch.randn(rows, IH) * 0.2
    keys = bf(torch.randn(1, 1, cap, D))
    pos = torch.tensor([ctx - 1, 700], dtype=torch.int32)
    lane = torch.zeros(rows, dtype=torch.int32)
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    scores = torch.full((rows, cap), float("nan"), device=DEV)
    n.indexer_score(q.to(DEV), hw.to(DEV), keys.to(DEV), pos.to(DEV), lane.to(DEV), rows, IH, D, 0, 1, cap, 64, 1, 0, cap, ctx, cap, scale,
                    scores)
    for r in range(rows):
        c = int(pos[r]) + 1
        dots = torch.einsum("hd,td->ht", q[r], keys[0, 0, :c].float()) * scale
        ref = (hw[r][:, None] * torch.relu(dots)).sum(0)
        ok, err = close(scores[r, :c], ref, rtol=1e-4, atol=1e-4)
        assert ok, err
        assert torch.isnan(scores[r, c:]).all()  # positions beyond the context are never written


@pytest.mark.parametrize("path", ["tcgen05", "cuda"])
def test_indexer_score_lanes_slots_and_stripes(native_lib, monkeypatch, path):
    """Both indexer kernels on a cache with several lanes and index slots, a striped layout (this GPU = rank 1 of 2) and ragged contexts."""
    monkeypatch.setenv("GLM_B200_INDEXER", path)
    n = native_lib
    torch.manual_seed(19)
    rows, IH, D, cap, stripe, world, rank = 3, 32, 128, 2048, 64, 2, 1
    lanes, slots, slot = 3, 2, 1
    local_cap = cap // world
    q = torch.randn(rows, IH, D) * 3.0
    hw = torch.randn(rows, IH) * 0.2
    keys = bf(torch.randn(lanes, slots, local_cap, D))
    pos = torch.tensor([1999, 130, 63], dtype=torch.int32)  # the last row owns nothing on rank 1 (positions 0..63 are rank 0's)
    lane = torch.tensor([2, 0, 1], dtype=torch.int32)
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    scores = torch.full((rows, cap), float("nan"), device=DEV)
    n.indexer_score(q.to(DEV), hw.to(DEV), keys.to(DEV), pos.to(DEV), lane.to(DEV), rows, IH, D, slot, slots, local_cap, stripe, world, rank, cap,
                    cap, cap, scale, scores)
    torch.cuda.synchronize()
    page = stripe * world
    for r in range(rows):
        ctx = int(pos[r]) + 1
        mine = [g for g in range(ctx) if (g // stripe) % world == rank]
        local = torch.tensor([(g // page) * stripe + g % stripe for g in mine], dtype=torch.long)
        got = scores[r].cpu()
        written = torch.zeros(cap, dtype=torch.bool)
        written[mine] = True
        assert torch.isnan(got[~written]).all()  # other ranks' positions and everything past the context stay untouched
        if mine:
            k = keys[int(lane[r]), slot, local].float()
            dots = torch.einsum("hd,td->ht", q[r], k) * scale
            ref = (hw[r][:, None] * torch.relu(dots)).sum(0)
            ok, err = close(got[mine], ref, rtol=1e-4, atol=1e-4)
            assert ok, (path, r, err)


@pytest.mark.parametrize("count", [0, 1, 31, 100, 2048])
def test_sparse_mla_attention(native_lib, count):
    n = native_lib
    torch.manual_seed(10)
    H, L, rd, cap, top_k = 64, 512, 64, 4096, 2048
    W = L + rd
    rows = 2
    q = bf(torch.randn(rows, H, W) * 0.3)
    cache = bf(torch.randn(1, 1, cap, W))
    sel = torch.full((rows, top_k), -1, dtype=torch.int32)
    counts = torch.zeros(rows, 2, dtype=torch.int32)
    picks = []
    for r in range(rows):
        c = count if r == 0 else min(count, 77)
        p = torch.sort(torch.randperm(cap)[:c]).values
        sel[r, :c] = p.to(torch.int32)
        counts[r] = c
        picks.append(p)
    chunks = -(-top_k // n.attn_chunk())
    part_o = torch.zeros(rows, chunks, H, L, device=DEV)
    part_ml = torch.zeros(rows, chunks, H, 2, device=DEV)
    o_lat = torch.zeros(rows, H, L, dtype=torch.bfloat16, device=DEV)
    lane = torch.zeros(rows, dtype=torch.int32, device=DEV)
    scale = float(torch.tensor((W - rd + rd) ** -0.5, dtype=torch.float32))
    n.sparse_mla_partial(q.to(DEV), cache.to(DEV), sel.to(DEV), counts.to(DEV), lane, rows, H, L, rd, 0, 1, cap, top_k, chunks, scale,
                         part_o, part_ml)
    n.attn_local_merge(part_o, part_ml, counts.to(DEV), rows, H, L, top_k, chunks, o_lat, H)
    # the one-kernel variant for many rows (running softmax statistics, no partials) against the same reference
    o_rows = torch.full((rows, H, L), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    n.sparse_mla_rows(q.to(DEV), cache.to(DEV), sel.to(DEV), counts.to(DEV), lane, rows, H, L, rd, 0, 1, cap, top_k, scale, o_rows, status)
    assert int(status.cpu()[0]) == 0
    for r in range(rows):
        ref = contract.absorbed_attention_row(q[r, :, :L], q[r, :, L:], cache[0, 0], picks[r], scale)
        ok, err = close(o_lat[r], ref, rtol=2**-6, atol=4e-3)
        assert ok, (r, err)
        ok, err = close(o_rows[r], ref, rtol=2**-6, atol=4e-3)
        assert ok, ("rows", r, err)


def test_wait_gives_up_and_reports(native_lib):
    """A wait on a flag that nothing sets runs out, sets the status word and leaves the context usable."""
    from glm_tpu_b200.parallel.peer import PeerGroup

    n = native_lib
    peer = PeerGroup(1, 0, wait_limit=2000)
    assert peer.read_status() == 0
    import ctypes as C

    code = n.lib().glmb_peer_wait_probe(C.byref(peer.comm), n.SIG_TEST, C.c_uint32(1), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code == 0
    assert peer.read_status() & n.STATUS_WAIT_TIMEOUT
    assert peer.read_status() == 0  # cleared by the read
    x = torch.ones(4, device=DEV) * 2
    assert float(x.sum()) == 8.0
    peer.close()


@pytest.mark.parametrize("shape", ["glm53", "small"])
def test_qkv_a_post_fast_equals_generic(native_lib, shape):
    """The single-round-trip kernel and the generic one must agree bit for bit (same rounding points, same reduction trees)."""
    n = native_lib
    Q, L, rd, D, IH = (2048, 512, 64, 128, 32) if shape == "glm53" else (128, 64, 16, 32, 4)
    rows, cap, lanes, layers, slots = 4, 256, 2, 3, 2
    W = L + rd
    torch.manual_seed(31)
    width = (Q + W + D + IH + 3) // 4 * 4
    proj = (torch.randn(rows, width) * 1.5).to(DEV)
    qw, kw = bf(torch.randn(Q) * 0.1 + 1).to(DEV), bf(torch.randn(L) * 0.1 + 1).to(DEV)
    knw, knb = (torch.randn(D) * 0.1 + 1).to(DEV), (torch.randn(D) * 0.05).to(DEV)
    table = contract.rope_table(cap, rd, 8e6).to(DEV)
    inv_freq = torch.pow(torch.tensor(8e6), -torch.arange(0, rd, 2, dtype=torch.float32) / rd).to(DEV)
    pos = torch.tensor([0, 17, 200, 255], dtype=torch.int32, device=DEV)
    lane = torch.tensor([0, 1, 1, 0], dtype=torch.int32, device=DEV)
    active = torch.tensor([1, 1, 0, 1], dtype=torch.int32, device=DEV)
    results = []
    for fast in (1, 0):
        n.set_qkv_fast(fast)
        out = {"q_resid": torch.zeros(rows, Q, dtype=torch.bfloat16, device=DEV), "kv_new": torch.zeros(rows, W, dtype=torch.bfloat16, device=DEV),
               "kv_cache": torch.zeros(lanes, layers, cap, W, dtype=torch.bfloat16, device=DEV),
               "index_cache": torch.zeros(lanes, slots, cap, D, dtype=torch.bfloat16, device=DEV),
               "head_w": torch.zeros(rows, IH, device=DEV), "idx_key_new": torch.zeros(rows, D, dtype=torch.bfloat16, device=DEV)}
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        a = n.QkvPostArgs()
        a.proj, a.proj_stride = proj.data_ptr(), proj.stride(0)
        a.q_norm_w, a.kv_norm_w = qw.data_ptr(), kw.data_ptr()
        a.rope_table, a.inv_freq = table.data_ptr(), inv_freq.data_ptr()
        a.k_norm_w, a.k_norm_b = knw.data_ptr(), knb.data_ptr()
        a.row_pos, a.row_lane, a.row_active = pos.data_ptr(), lane.data_ptr(), active.data_ptr()
        a.q_resid, a.kv_new = out["q_resid"].data_ptr(), out["kv_new"].data_ptr()
        a.kv_cache, a.index_cache = out["kv_cache"].data_ptr(), out["index_cache"].data_ptr()
        a.head_w, a.idx_key_new = out["head_w"].data_ptr(), out["idx_key_new"].data_ptr()
        a.Q, a.L, a.rd, a.D, a.IH = Q, L, rd, D, IH
        a.has_indexer = 1
        a.layer, a.layers, a.index_slot, a.full_layers = 1, layers, 1, slots
        a.local_cap, a.stripe, a.world, a.rank, a.capacity = cap, 64, 1, 0, cap
        a.eps, a.key_eps, a.head_scale = 1e-5, 1e-6, float(torch.tensor(IH**-0.5, dtype=torch.float32))
        a.status = status.data_ptr()
        n.qkv_a_post(a, rows)
        torch.cuda.synchronize()
        assert int(status.cpu()[0]) == 0
        results.append({k: v.cpu() for k, v in out.items()})
    n.set_qkv_fast(1)
    for key in results[0]:
        x, y = results[0][key], results[1][key]
        assert torch.equal(x.view(torch.int16) if x.dtype == torch.bfloat16 else x, y.view(torch.int16) if y.dtype == torch.bfloat16 else y), key
    # the inactive row wrote this step's row but not the cache; active rows wrote their cache rows
    assert bool((results[0]["kv_cache"][1, 1, 200] == 0).all()) and bool((results[0]["kv_cache"][1, 1, 17] != 0).any())
    assert bool((results[0]["kv_new"][2] != 0).any())


def test_q_post_fold_is_bit_identical(native_lib):
    """q_absorb fed with the raw q_b projection, and the tcgen05 indexer fed with the raw index query, against the two-kernel
    path (q_post first): the absorbed queries, their rope parts and the index scores must agree bit for bit."""
    n = native_lib
    torch.manual_seed(41)
    rows, hl, nope, rd, vd, L, IH, D, cap = 3, 8, 192, 64, 256, 512, 32, 128, 2048
    qk, W = nope + rd, L + rd
    q_proj = (torch.randn(rows, hl * qk + IH * D) * 0.7).to(DEV)
    kv_b = bf(torch.randn(hl, nope + vd, L) * 0.05).to(DEV)
    table = contract.rope_table(cap, rd, 8e6).to(DEV)
    inv_freq = torch.pow(torch.tensor(8e6), -torch.arange(0, rd, 2, dtype=torch.float32) / rd).to(DEV)
    pos = torch.tensor([5, 1000, 2047], dtype=torch.int32, device=DEV)
    lane = torch.zeros(rows, dtype=torch.int32, device=DEV)
    hw = (torch.randn(rows, IH) * 0.2).to(DEV)
    keys = bf(torch.randn(1, 1, cap, D)).to(DEV)
    scale = float(torch.tensor(D**-0.5, dtype=torch.float32))
    # two-kernel path
    q_nope = torch.zeros(rows, hl, nope, dtype=torch.bfloat16, device=DEV)
    q_full_a = torch.zeros(rows, hl, W, dtype=torch.bfloat16, device=DEV)
    q_idx = torch.zeros(rows, IH, D, device=DEV)
    b = n.QPostArgs()
    b.q, b.q_stride = q_proj.data_ptr(), q_proj.stride(0)
    b.rope_table, b.inv_freq, b.row_pos = table.data_ptr(), inv_freq.data_ptr(), pos.data_ptr()
    b.q_nope, b.q_full, b.q_idx = q_nope.data_ptr(), q_full_a.data_ptr(), q_idx.data_ptr()
    b.heads_local, b.head_base, b.heads_total = hl, 0, hl
    b.nope, b.rd, b.L, b.IH, b.D = nope, rd, L, IH, D
    b.has_indexer, b.capacity = 1, cap
    n.q_post(b, rows)
    n.q_absorb(q_nope, rows, kv_b, hl, 0, hl, nope, vd, L, rd, q_full_a)
    scores_a = torch.full((rows, cap), float("nan"), device=DEV)
    n.indexer_score(q_idx, hw, keys, pos, lane, rows, IH, D, 0, 1, cap, 64, 1, 0, cap, cap, cap, scale, scores_a)
    # folded path
    q_full_b = torch.zeros(rows, hl, W, dtype=torch.bfloat16, device=DEV)
    n.q_absorb(None, rows, kv_b, hl, 0, hl, nope, vd, L, rd, q_full_b, q_proj=q_proj, rope_table=table, row_pos=pos, capacity=cap)
    scores_b = torch.full((rows, cap), float("nan"), device=DEV)
    n.indexer_score(None, hw, keys, pos, lane, rows, IH, D, 0, 1, cap, 64, 1, 0, cap, cap, cap, scale, scores_b, q_raw=q_proj, q_offset=hl * qk,
                    inv_freq=inv_freq, rd=rd)
    torch.cuda.synchronize()
    assert torch.equal(q_full_a.view(torch.int16), q_full_b.view(torch.int16))
    assert bool((q_full_a[..., L:] != 0).any())
    for r in range(rows):
        c = int(pos[r]) + 1
        assert torch.equal(scores_a[r, :c], scores_b[r, :c])
        assert torch.isnan(scores_b[r, c:]).all()


def test_staging_canaries_catch_an_overrun(native_lib):
    """A write past the end of a staging region lands in its guard band and is reported (host-side check, no fault involved)."""
    from glm_tpu_b200.exceptions import DeviceStatusError
    from glm_tpu_b200.parallel.peer import PeerGroup

    peer = PeerGroup(1, 0, staging_bytes=8192)
    a = peer.region("a", 1000)
    b = peer.region("b", 512)
    peer.tensor(a, (250,), torch.float32).fill_(1.0)
    peer.tensor(b, (128,), torch.float32).fill_(2.0)
    peer.check_canaries()
    peer._bytes[a.offset + a.nbytes + 3] = 0  # one byte past region a (inside the staging buffer: nothing faults)
    with pytest.raises(DeviceStatusError, match="overrun"):
        peer.check_canaries()
    peer.close()
