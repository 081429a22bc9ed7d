"""The tcgen05/TMEM/TMA GEMM against a plain fp32 PyTorch product (B200 only)."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(params=[1, 2], ids=["tile128x128", "persistent128x256"])
def variant(request, native_lib):
    """Both kernels behind the one entry point: 128x128 tile per CTA, and the persistent 128x256 kernel."""
    native_lib.set_gemm_variant(request.param)
    yield request.param
    native_lib.set_gemm_variant(0)


@pytest.mark.parametrize("rows,N,K", [(128, 128, 64), (300, 256, 512), (1000, 384, 6144), (64, 2048, 200), (2500, 1288, 136)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_dense_gemm(native_lib, variant, rows, N, K, out_dtype):
    n = native_lib
    torch.manual_seed(rows + N + K)
    a = (torch.randn(rows, K, device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, device=DEV) * 0.5).to(torch.bfloat16)
    out = torch.full((rows, N), float("nan"), dtype=out_dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    n.gemm_bf16_tc(a, b, out, status=status)
    ref = a.float() @ b.float().T
    assert int(status.cpu()[0]) == 0
    tol = 2**-7 if out_dtype == torch.bfloat16 else 1e-4
    err = (out.float() - ref).abs().max().item()
    assert torch.allclose(out.float(), ref, rtol=tol, atol=tol * float(ref.abs().max())), err


@pytest.mark.parametrize("N", [256, 328])
def test_grouped_gemm(native_lib, variant, N):
    n = native_lib
    torch.manual_seed(5)
    E, K = 4, 512
    counts = [130, 0, 257, 5]
    rows = sum(counts)
    a = (torch.randn(rows, K, device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn(E, N, K, device=DEV) * 0.5).to(torch.bfloat16)
    tiles, start = [], 0
    for e, c in enumerate(counts):
        for r0 in range(start, start + c, 128):
            tiles.append([r0, start + c, e, 0])
        start += c
    max_tiles = len(tiles) + 3
    tiles += [[0, 0, 0, 0]] * 3
    tiles_t = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    n_tiles = torch.tensor([max_tiles - 3], dtype=torch.int32, device=DEV)
    out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    n.gemm_bf16_tc(a, b, out, experts=E, tiles=tiles_t, n_tiles=n_tiles, status=status)
    assert int(status.cpu()[0]) == 0
    start = 0
    for e, c in enumerate(counts):
        ref = a[start : start + c].float() @ b[e].float().T
        assert torch.allclose(out[start : start + c].float(), ref, rtol=2**-7, atol=2**-7 * 8), e
        start += c


def test_gemm_throughput_is_tensor_core_class(native_lib):
    """A 8192^3 product must run far above what CUDA cores could do (sanity check, not a benchmark)."""
    n = native_lib
    M = N = K = 8192
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    b = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    n.set_gemm_variant(0)
    for _ in range(2):
        n.gemm_bf16_tc(a, b, out)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(5):
        n.gemm_bf16_tc(a, b, out)
    e.record()
    torch.cuda.synchronize()
    tflops = 5 * 2 * M * N * K / (s.elapsed_time(e) * 1e-3) / 1e12
    print(f"tcgen05 gemm 8192^3: {tflops:.0f} TFLOP/s")
    assert tflops > 150


def test_many_tiles_per_cta(native_lib, variant):
    """More tiles than SMs: the persistent kernel reuses both accumulators and wraps the operand ring many times."""
    n = native_lib
    torch.manual_seed(11)
    rows, N, K = 4096, 2560, 320
    a = (torch.randn(rows, K, device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, device=DEV) * 0.5).to(torch.bfloat16)
    out = torch.full((rows, N), float("nan"), dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    n.gemm_bf16_tc(a, b, out, status=status)
    ref = a.float() @ b.float().T
    assert int(status.cpu()[0]) == 0
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-4 * float(ref.abs().max()))
