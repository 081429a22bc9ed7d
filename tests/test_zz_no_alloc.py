"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of this library may not call cudaMalloc at all (a process with memory fixed at start-up, a plug-in living
in another framework's pool, a loop that cannot afford the allocator's implicit synchronisation).  For them
``glmb_sparse_mla_attention_noalloc`` keeps the attention intermediates in an array inside the library image.  This
test checks that it returns exactly what the ordinary two-call path returns (and what a plain fp32 softmax attention
gives, within bf16), on consecutive calls that share that array; that the driver's free-memory figure does not move
across a call; that the status word reports a clamped index; and that it refuses problems larger than the array or of a
shape the kernels do not take, with codes that cannot be mistaken for CUDA errors.  It is collected last on purpose (the file name sorts behind every
other test file): the free-memory comparison is only meaningful once everything that allocates lazily in this process --
the CUDA context, the library's module image on the device, handles other tests create -- already exists, and a test
that leaked device memory before it would show up here as a moving baseline rather than hide.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOO_LARGE, BAD_SHAPE = -1, -2


def _problem(seed, counts, H=64, L=512, rd=64, cap=4096, top_k=2048):
    gen = torch.Generator().manual_seed(seed)
    rows, W = len(counts), L + rd
    q = (torch.randn(rows, H, W, generator=gen) * 0.3).to(torch.bfloat16)
    cache = torch.randn(1, 1, cap, W, generator=gen).to(torch.bfloat16)
    sel = torch.full((rows, top_k), -1, dtype=torch.int32)
    cnt = torch.zeros(rows, 2, dtype=torch.int32)
    for r, c in enumerate(counts):
        sel[r, :c] = torch.sort(torch.randperm(cap, generator=gen)[:c]).values.to(torch.int32)
        cnt[r] = c
    return dict(q=q.to(DEV), cache=cache.to(DEV), sel=sel.to(DEV), cnt=cnt.to(DEV), lane=torch.zeros(rows, dtype=torch.int32, device=DEV),
                rows=rows, H=H, L=L, rd=rd, cap=cap, top_k=top_k, scale=float(torch.tensor((L // 2) ** -0.5, dtype=torch.float32)))


def _ordinary(n, p):
    chunks = -(-p["top_k"] // n.attn_chunk())
    part_o = torch.zeros(p["rows"], chunks, p["H"], p["L"], device=DEV)
    part_ml = torch.zeros(p["rows"], chunks, p["H"], 2, device=DEV)
    out = torch.zeros(p["rows"], p["H"], p["L"], dtype=torch.bfloat16, device=DEV)
    n.sparse_mla_partial(p["q"], p["cache"], p["sel"], p["cnt"], p["lane"], p["rows"], p["H"], p["L"], p["rd"], 0, 1, p["cap"], p["top_k"],
                         chunks, p["scale"], part_o, part_ml)
    n.attn_local_merge(part_o, part_ml, p["cnt"], p["rows"], p["H"], p["L"], p["top_k"], chunks, out, p["H"])
    return out


def _no_alloc(n, p, out, status=None):
    fn = n.lib().glmb_sparse_mla_attention_noalloc
    fn.restype = C.c_int
    ptr = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    return fn(ptr(p["q"]), ptr(p["cache"]), ptr(p["sel"]), ptr(p["cnt"]), ptr(p["lane"]), p["rows"], p["H"], p["L"], p["rd"], 0, 1, p["cap"],
              p["top_k"], C.c_float(p["scale"]), ptr(out), None if status is None else ptr(status),
              C.c_void_p(torch.cuda.current_stream().cuda_stream))


def _fp32_reference(p):
    """Plain softmax attention over the selected cache rows in fp32: scores over latent + rope, values = the latent part."""
    q, cache = p["q"].float().cpu(), p["cache"].float().cpu()[0, 0]
    out = torch.zeros(p["rows"], p["H"], p["L"])
    for r in range(p["rows"]):
        count = int(p["cnt"][r, 1])
        if count == 0:
            continue
        keys = cache[p["sel"][r, :count].cpu().long()]
        prob = torch.softmax(q[r] @ keys.T * p["scale"], dim=-1)
        out[r] = prob @ keys[:, : p["L"]]
    return out


def test_no_alloc_attention_matches_ordinary_path_twice(native_lib):
    n = native_lib
    # the second problem is smaller, so stale intermediates of the first call sit right behind the ones it uses
    for seed, counts in ((11, [2048, 700]), (12, [65, 0])):
        p = _problem(seed, counts)
        expect = _ordinary(n, p)
        out = torch.full_like(expect, float("nan"))
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        reference = _fp32_reference(p)
        assert _no_alloc(n, p, torch.empty_like(out)) == 0  # a warm call: module load and the symbol lookup happen once
        torch.cuda.synchronize()
        free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        code = _no_alloc(n, p, out, status)
        assert code == 0, code
        torch.cuda.synchronize()
        # the driver's own figure: a cudaMalloc inside the library would show here, whoever's allocator made it
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == allocated_before
        assert int(status.item()) == 0
        assert torch.equal(out, expect)  # the same kernels on the same inputs: the same bits
        assert torch.allclose(out.float().cpu(), reference, rtol=2**-6, atol=4e-3), (out.float().cpu() - reference).abs().max()
        if counts[1] == 0:  # an empty row gives zeros
            assert torch.equal(out[1], torch.zeros_like(out[1]))


def test_no_alloc_attention_reports_a_clamped_index(native_lib):
    n = native_lib
    p = _problem(15, [130, 40])
    p["sel"][1, 7] = p["cap"] + 5  # beyond the cache: the kernel clamps it (no fault) and says so
    out = torch.zeros(2, p["H"], p["L"], dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert _no_alloc(n, p, out, status) == 0
    torch.cuda.synchronize()
    assert int(status.item()) & n.STATUS_BAD_INDEX
    assert bool(torch.isfinite(out.float()).all())


def test_no_alloc_attention_refuses_what_does_not_fit(native_lib):
    n = native_lib
    p = _problem(13, [10, 10, 10])
    out = torch.zeros(3, p["H"], p["L"], dtype=torch.bfloat16, device=DEV)
    assert _no_alloc(n, p, out) == TOO_LARGE
    p = _problem(14, [10], top_k=4096, cap=8192)
    out = torch.zeros(1, p["H"], p["L"], dtype=torch.bfloat16, device=DEV)
    assert _no_alloc(n, p, out) == TOO_LARGE
    # shapes the kernels do not take: refused before anything is launched, never reported as a CUDA error
    for change in (dict(rd=-64), dict(rd=8), dict(L=256), dict(top_k=0)):
        p = _problem(14, [10])
        p.update(change)
        assert _no_alloc(n, p, torch.zeros(1, p["H"], 512, dtype=torch.bfloat16, device=DEV)) == BAD_SHAPE, change
    p = _problem(14, [10])
    p["rd"] = 1024
    assert _no_alloc(n, p, torch.zeros(1, p["H"], p["L"], dtype=torch.bfloat16, device=DEV)) == TOO_LARGE
    n.lib().glmb_noalloc_strerror.restype = C.c_char_p
    assert b"at most 2 rows" in n.lib().glmb_noalloc_strerror(TOO_LARGE)
    assert b"unsupported shape" in n.lib().glmb_noalloc_strerror(BAD_SHAPE)
    assert b"CUDA error" in n.lib().glmb_noalloc_strerror(700) and b"CUDA error" not in n.lib().glmb_noalloc_strerror(-9)
