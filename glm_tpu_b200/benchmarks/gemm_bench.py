"""tcgen05 GEMM against the library GEMM at square and at prefill shapes.

    python -m glm_tpu_b200.benchmarks.gemm_bench [--shapes 8192x8192x8192,512x6144x2048] [--iters 10] [--out gemm.md]

Each shape ``MxNxK`` computes ``C[M,N] = A[M,K] . B[N,K]^T`` (bf16 in, fp32 accumulate, bf16 out).  Timing: CUDA events
around each launch after 3 warm-ups, the best and the median of ``--iters`` runs, with a 256 MB buffer written between
runs so that no operand is left in the 126 MB L2.  Fractions are against the measured library bf16 throughput
(``MEASURED_PEAKS.json`` at the repository root when present, else 1,590 TFLOP/s).
"""

from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

DEFAULT_SHAPES = "8192x8192x8192,4096x4096x4096,2048x6144x2048,512x6144x2048,512x2784x6144,4096x12288x6144,256x19360x6144"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shapes", default=DEFAULT_SHAPES)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-library", action="store_true", help="skip the library GEMM (profiling runs)")
    ap.add_argument("--variant", type=int, default=0, help="0 auto, 1 one 128x128 tile per CTA, 2 persistent 128x256 kernel")
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)

    import torch

    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.ops import native

    build()
    native.set_gemm_variant(args.variant)
    dev = torch.device("cuda", 0)
    peaks_file = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak = json.loads(peaks_file.read_text())["bf16_tflops"] if peaks_file.exists() else 1590.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        out = []
        for _ in range(args.iters):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return min(out), statistics.median(out)

    lines = [f"bf16 GEMM C[M,N] = A[M,K] . B[N,K]^T, fp32 accumulate; kernel variant {args.variant} (0 = chosen by size); library peak (measured burst) {peak:.0f} TFLOP/s; L2 flushed between runs",
             "", "| M x N x K | tcgen05 best us | median us | TFLOP/s (best) | of measured library peak | library best us | library TFLOP/s | max abs diff |",
             "|---|---|---|---|---|---|---|---|"]
    for shape in args.shapes.split(","):
        M, N, K = (int(v) for v in shape.split("x"))
        a = torch.randn(M, K, device=dev, dtype=torch.float32).mul_(0.5).to(torch.bfloat16)
        b = torch.randn(N, K, device=dev, dtype=torch.float32).mul_(0.5).to(torch.bfloat16)
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        best, med = timed(lambda: native.gemm_bf16_tc(a, b, c, status=status.data_ptr()))
        flops = 2.0 * M * N * K
        row = f"| {M} x {N} x {K} | {best * 1e3:.1f} | {med * 1e3:.1f} | {flops / best / 1e9:.0f} | {flops / best / 1e9 / peak:.2f} |"
        if args.no_library:
            row += " - | - | - |"
        else:
            ref = torch.empty_like(c)
            lbest, _ = timed(lambda: torch.mm(a, b.t(), out=ref))
            row += f" {lbest * 1e3:.1f} | {flops / lbest / 1e9:.0f} | {(c.float() - ref.float()).abs().max().item():.3g} |"
        lines.append(row)
        del a, b, c
    if int(status[0]) != 0:
        raise SystemExit(f"device status {int(status[0])}")
    text = "\n".join(lines) + "\n"
    print(text)
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
