"""The grouped expert GEMM with in-kernel FP8 decode (tcgen05) against a plain fp32 PyTorch restatement (B200 only)."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiles(local_ids, el):
    """Host restatement of the route sort: tiles, n_tiles, perm for routes whose local expert id is in [0, el)."""
    P = local_ids.numel()
    key = torch.where((local_ids >= 0) & (local_ids < el), local_ids, torch.full_like(local_ids, el))
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=el + 1)[:el]
    n_local = int(counts.sum())
    perm = torch.where(torch.arange(P) < n_local, order, torch.full_like(order, -1)).to(torch.int32)
    tiles, start = [], 0
    for e in range(el):
        c = int(counts[e])
        for r0 in range(start, start + c, 128):
            tiles.append([r0, start + c, e, 0])
        start += c
    n = len(tiles)
    tiles += [[0, 0, 0, 0]] * 5
    return torch.tensor(tiles, dtype=torch.int32), torch.tensor([n], dtype=torch.int32), perm


@pytest.mark.parametrize("rows,tk,E,el,H,I", [(64, 4, 8, 8, 512, 256), (300, 8, 16, 6, 1024, 384), (96, 8, 8, 4, 6144, 2048)])
def test_grouped_fp8_experts(native_lib, rows, tk, E, el, H, I):
    from glm_tpu_b200.models.glm_moe_dsa.weights import quantize_fp8
    from glm_tpu_b200.oracle.contract import dequantize_fp8

    n = native_lib
    gen = torch.Generator().manual_seed(rows + H)
    x = (torch.randn(rows, H, generator=gen) * 0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=gen)[:tk] for _ in range(rows)])  # [rows, tk], distinct per row
    ids[0] = ids[1]  # a repeated pattern, so one expert gets adjacent routes
    weight = torch.rand(rows, tk, generator=gen) + 0.1
    wg, sg = quantize_fp8(torch.randn(el, I, H, generator=gen) * 0.05, (128, 128), gen)
    wu, su = quantize_fp8(torch.randn(el, I, H, generator=gen) * 0.05, (128, 128), gen)
    wd, sd = quantize_fp8(torch.randn(el, H, I, generator=gen) * 0.05, (128, 128), gen)
    tiles, n_tiles, perm = _tiles(ids.reshape(-1).long(), el)
    P = rows * tk
    xs = torch.full((P, H), float("nan"), dtype=torch.bfloat16, device=DEV)  # poison: rows past this GPU's routes become zeros, never leak
    acts = torch.full((P, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    dw = torch.full((P, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    d = lambda t: t.to(DEV).contiguous()  # noqa: E731
    perm_d, tiles_d, n_d = d(perm), d(tiles), d(n_tiles)
    n.gather_rows(d(x), perm_d, tk, xs)
    n.moe_grouped_fp8w(xs, d(wg), d(wu), d(sg), d(su), tiles_d, n_d, 0, acts, status=status)
    n.moe_grouped_fp8w(acts, d(wd), None, d(sd), None, tiles_d, n_d, 1, dw, perm=perm_d, route_weight=d(weight), status=status)
    torch.cuda.synchronize()
    assert int(status.cpu()[0]) == 0
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    dq = [dequantize_fp8(w, s, (128, 128)).float() for w, s in ((wg, sg), (wu, su), (wd, sd))]
    got_x, got_act, got_dw = xs.cpu().float(), acts.cpu().float(), dw.cpu().float()
    checked = 0
    for pos in range(P):
        route = int(perm[pos])
        if route < 0:
            continue
        r, e = route // tk, int(ids.reshape(-1)[route])
        assert torch.equal(got_x[pos], x[r].float())
        g, u = bf(x[r].float() @ dq[0][e].T), bf(x[r].float() @ dq[1][e].T)
        act = bf(g * torch.sigmoid(g) * u)
        assert torch.allclose(got_act[pos], act, rtol=2**-6, atol=2**-8 * float(act.abs().max())), (pos, route)
        down = bf(bf(got_act[pos] @ dq[2][e].T) * bf(weight.reshape(-1)[route]))
        assert torch.allclose(got_dw[route], down, rtol=2**-6, atol=2**-8 * float(down.abs().max())), (pos, route)
        checked += 1
    assert checked == int((ids < el).sum())
    # routes of experts this GPU does not hold are never written
    foreign = (ids.reshape(-1) >= el).nonzero().flatten()
    assert bool(torch.isnan(got_dw[foreign]).all())
    # padding rows of the sorted activation buffer were overwritten with zeros, and no NaN reached a real route
    assert bool((got_x[checked:] == 0).all()) and not bool(torch.isnan(got_dw[(ids.reshape(-1) < el).nonzero().flatten()]).any())


@pytest.mark.parametrize("rows,tk,E,ebase,el", [(64, 4, 8, 0, 8), (300, 8, 16, 6, 6), (4096, 8, 256, 32, 32), (1000, 8, 256, 0, 256), (37, 8, 256, 224, 32)])
def test_route_sort_kernel_matches_the_stable_sort(native_lib, rows, tk, E, ebase, el):
    """One launch gives the permutation of a stable argsort by local expert, the 128-route tiles and their count."""
    n = native_lib
    gen = torch.Generator().manual_seed(rows * 7 + el)
    skew = torch.rand(E, generator=gen) ** 3 + 0.01  # some experts get many routes, some almost none
    ids = torch.multinomial(skew.expand(rows, E), tk, replacement=False, generator=gen).to(torch.int32)
    if rows == 37:
        ids[:] = torch.arange(tk, dtype=torch.int32)  # nothing for this GPU's experts [224, 256)
    P = rows * tk
    tiles_ref, n_ref, perm_ref = _tiles(ids.reshape(-1).long() - ebase, el)
    max_tiles = P // 128 + el
    tiles = torch.full((max_tiles, 4), 7, dtype=torch.int32, device=DEV)
    n_tiles = torch.full((1,), -5, dtype=torch.int32, device=DEV)
    perm = torch.full((P,), 12345, dtype=torch.int32, device=DEV)
    for _ in range(2):  # the second launch overwrites the first completely
        n.route_sort128(ids.to(DEV), ebase, el, tiles, n_tiles, perm)
    torch.cuda.synchronize()
    count = int(n_tiles.item())
    assert count == int(n_ref.item())
    assert torch.equal(perm.cpu(), perm_ref)
    assert torch.equal(tiles[:count].cpu(), tiles_ref[:count])
    assert bool((tiles[count:] == 0).all())


@pytest.mark.parametrize("rows,tk,E,ebase,el", [(64, 4, 8, 0, 8), (200, 8, 256, 0, 256), (256, 8, 256, 32, 32), (37, 8, 256, 224, 32), (1, 8, 256, 0, 256)])
def test_route_sort_in_tiles_of_eight(native_lib, rows, tk, E, ebase, el):
    """The same launch cut into 8-route tiles: per expert of this GPU, in expert order, its routes in route order, eight to a tile
    (global expert id per tile, -1 in the empty slots of an expert's last tile and in the tiles past the count)."""
    n = native_lib
    gen = torch.Generator().manual_seed(rows * 11 + el)
    skew = torch.rand(E, generator=gen) ** 3 + 0.01
    ids = torch.multinomial(skew.expand(rows, E), tk, replacement=False, generator=gen).to(torch.int32)
    if rows == 37:
        ids[:] = torch.arange(tk, dtype=torch.int32)  # nothing for this GPU's experts [224, 256)
    flat = ids.reshape(-1).tolist()
    want_expert, want_routes = [], []
    for e in range(ebase, ebase + el):
        mine = [i for i, x in enumerate(flat) if x == e]
        for j in range(0, len(mine), 8):
            want_expert.append(e)
            want_routes.append(mine[j : j + 8] + [-1] * (8 - len(mine[j : j + 8])))
    P = rows * tk
    max_tiles = P // 8 + el
    tile_expert = torch.full((max_tiles,), 7, dtype=torch.int32, device=DEV)
    tile_routes = torch.full((max_tiles, 8), 7, dtype=torch.int32, device=DEV)
    n_tiles = torch.full((1,), -5, dtype=torch.int32, device=DEV)
    scratch = torch.full((P,), 12345, dtype=torch.int32, device=DEV)
    for _ in range(2):
        n.route_sort8(ids.to(DEV), ebase, el, tile_expert, tile_routes, n_tiles, scratch)
    torch.cuda.synchronize()
    count = int(n_tiles.item())
    assert count == len(want_expert) <= max_tiles
    assert tile_expert[:count].cpu().tolist() == want_expert and bool((tile_expert[count:] == -1).all())
    assert tile_routes[:count].cpu().tolist() == want_routes


def test_swiglu_rows_matches_the_elementwise_expression(native_lib):
    n = native_lib
    gen = torch.Generator().manual_seed(5)
    gate = (torch.randn(300, 1024, generator=gen) * 3.0).to(torch.bfloat16).to(DEV)
    up = torch.randn(300, 1024, generator=gen).to(torch.bfloat16).to(DEV)
    gate[0, :4] = torch.tensor([0.0, -0.0, 80.0, -80.0], dtype=torch.bfloat16)
    g32, u32 = gate.float(), up.float()
    ref = (g32 * torch.sigmoid(g32) * u32).to(torch.bfloat16)
    out = n.swiglu_rows(gate.clone(), up)
    assert torch.allclose(out.float(), ref.float(), rtol=2**-7, atol=1e-30)
    assert float((out != ref).float().mean()) < 1e-3  # at most a last-place difference of the exponential here and there
    inplace = gate.clone()
    assert n.swiglu_rows(inplace, up, inplace) is inplace and torch.equal(inplace, out)
