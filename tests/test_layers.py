"""The layer-level functions: CPU path against hand-made cases, and (on a B200) the CUDA path against the CPU path."""

import pytest
import torch

from glm_tpu_b200.layers import embed, fp8, linear, mlp, norm, sampler
from glm_tpu_b200.layers.attention import dsa_indexer, kv_cache, mla
from glm_tpu_b200.layers.contracts import RouterOutput
from glm_tpu_b200.layers.moe import routed_experts, router
from glm_tpu_b200.models.glm_moe_dsa.weights import quantize_fp8


def _inputs(device):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(3, 256, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(128, 256, generator=g) * 0.05).to(torch.bfloat16)
    return x.to(device), w.to(device), g


def _run_all(device):
    x, w, g = _inputs(device)
    out = {}
    nw = (torch.randn(256, generator=g) * 0.1 + 1).to(torch.bfloat16).to(device)
    out["norm"], out["residual"] = norm.add_rms_norm(x, x * 2, nw, 1e-5)
    out["linear"] = linear.linear(x, w)
    w2 = (torch.randn(128, 256, generator=g) * 0.05).to(torch.bfloat16).to(device)
    wd = (torch.randn(256, 128, generator=g) * 0.05).to(torch.bfloat16).to(device)
    out["mlp"] = mlp.dense_mlp(x, w, w2, wd)
    bits, scale = quantize_fp8(torch.randn(256, 256, generator=g) * 0.05, (128, 128), g)
    out["fp8"] = fp8.decode(bits.to(device), scale.to(device))
    table = (torch.randn(50, 256, generator=g)).to(torch.bfloat16).to(device)
    out["embed"] = embed.embed(torch.tensor([3, 49, 0]), table)
    logits = torch.randn(3, 1000, generator=g).to(torch.bfloat16)
    logits[1, 10] = logits[1, 500] = 9.0
    out["greedy"] = sampler.greedy(logits.to(device))
    routes = router.route((torch.randn(3, 256, generator=g)).to(device), (torch.randn(256, generator=g) * 0.1).to(device), 8)
    out["route_ids"], out["route_w"] = routes.expert_ids, routes.weights
    q = torch.randn(2, 32, 128, generator=g)
    keys = torch.randn(300, 128, generator=g).to(torch.bfloat16)
    lengths = torch.tensor([300, 120])
    sc = dsa_indexer.scores(q.to(device), (torch.randn(2, 32, generator=g) * 0.2).to(device), keys.to(device), lengths)
    out["scores"] = torch.nan_to_num(sc, nan=-7.0)
    sel = dsa_indexer.select(sc, lengths, 64)
    out["selected"], out["counts"] = sel.positions, sel.counts
    qa = (torch.randn(2, 16, 576, generator=g) * 0.3).to(torch.bfloat16)
    cache = torch.randn(300, 576, generator=g).to(torch.bfloat16)
    out["attention"] = mla.sparse_attention(qa.to(device), cache.to(device), sel, 512, 576**-0.5)
    gate = quantize_fp8(torch.randn(4, 128, 256, generator=g) * 0.05, (128, 128), g)
    up = quantize_fp8(torch.randn(4, 128, 256, generator=g) * 0.05, (128, 128), g)
    down = quantize_fp8(torch.randn(4, 256, 128, generator=g) * 0.05, (128, 128), g)
    ids = torch.tensor([[0, 3], [2, 5], [1, 1]], dtype=torch.int32)
    ro = RouterOutput(ids.to(device), torch.tensor([[0.6, 0.4], [0.5, 0.5], [0.9, 0.1]]).to(device))
    dev = lambda pair: (pair[0].to(device), pair[1].to(device))  # noqa: E731
    out["dw"] = routed_experts.routed_experts(x, ro, dev(gate), dev(up), dev(down))
    return {k: v.detach().cpu() for k, v in out.items()}


def test_cpu_path_basic_rules():
    out = _run_all("cpu")
    assert out["greedy"].tolist()[1] == 10  # ties go to the lowest id
    assert out["counts"].tolist() == [[64, 64], [64, 64]] and bool((out["selected"][:, 1:] > out["selected"][:, :-1]).all())
    assert bool((out["dw"][3] == 0).all()) and bool((out["dw"][0] != 0).any())  # expert 5 is not among this GPU's four
    assert torch.allclose(out["route_w"].sum(-1), torch.ones(3), atol=1e-6)
    assert kv_cache.owner(torch.tensor([0, 63, 64, 130]), 64, 2).tolist() == [0, 0, 1, 0]
    assert kv_cache.local_row(torch.tensor([0, 64, 128, 130]), 64, 2).tolist() == [0, 0, 64, 66]
    assert [kv_cache.owned_count(130, 64, 2, r) for r in (0, 1)] == [66, 64]
    assert kv_cache.owner_subset(torch.tensor([1, 70, 129, -1]), 64, 2, 0).tolist() == [1, 65]


@pytest.mark.gpu
def test_cuda_path_matches_cpu_path(native_lib):
    cpu, gpu = _run_all("cpu"), _run_all("cuda:0")
    for key in ("greedy", "route_ids", "selected", "counts", "embed", "fp8", "residual"):
        assert torch.equal(cpu[key], gpu[key]), key
    for key, tol in (("norm", 2**-7), ("linear", 2**-7), ("mlp", 2**-6), ("route_w", 1e-6), ("scores", 1e-4), ("attention", 2**-6), ("dw", 2**-5)):
        a, b = cpu[key].float(), gpu[key].float()
        assert torch.allclose(a, b, rtol=tol, atol=tol * float(a.abs().max())), (key, float((a - b).abs().max()))
