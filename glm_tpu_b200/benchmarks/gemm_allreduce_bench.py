"""GEMM followed by an all-reduce of the K-split partial products: one fused kernel against GEMM + library all-reduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 \\
        -m glm_tpu_b200.benchmarks.gemm_allreduce_bench [--shapes 1024x6144x2048,...] [--iters 20] [--out file.md]

Each rank holds its own ``A_r [M, K]`` and ``B_r [N, K]`` (bf16); the result on every rank is ``bf16(sum_r A_r . B_r^T)``.

* fused: the persistent tcgen05 kernel whose epilogue pushes each fp32 partial tile to the tile's owner over NVLink, sums in
  rank order, and pushes the bf16 tile to every rank, plus the one-CTA kernel that waits for every rank's completion signal;
* baseline: the same tcgen05 GEMM with an fp32 result, ``torch.distributed.all_reduce`` (NCCL), and the cast to bf16.

Timing: CUDA events on the launching stream around each iteration after a barrier, the maximum over ranks per iteration,
best and median of ``--iters`` after 3 warm-ups; a 256 MB buffer is written between iterations (operands leave L2).  The
roofline time is the larger of FLOPs / measured library GEMM peak and the bytes each GPU must send (fp32 partials to the
owners + bf16 results to the others) / 770 GB/s (measured peer copy bandwidth per direction).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shapes", default="1024x6144x2048,1024x6144x1536,4096x6144x2048,256x6144x2048")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist

    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.ops import native
    from glm_tpu_b200.parallel.peer import PeerGroup

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if rank == 0:
        build()
    dist.init_process_group("nccl", device_id=dev)
    dist.barrier()
    peaks_file = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak = json.loads(peaks_file.read_text())["bf16_tflops"] if peaks_file.exists() else 1590.0
    link_gbs = 770.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    lines = [f"GEMM + all-reduce over {world} GPUs: fused tcgen05/NVLink kernel vs tcgen05 GEMM + NCCL all-reduce + cast; max over ranks; "
             f"roofline = max(FLOPs / {peak:.0f} TFLOP/s, bytes sent per GPU / {link_gbs:.0f} GB/s)",
             "", "| M x N x K (per rank) | fused best us | fused median us | baseline best us | baseline median us | speed-up (median) | roofline us | fused / roofline |",
             "|---|---|---|---|---|---|---|---|"]
    for shape in args.shapes.split(","):
        M, N, K = (int(v) for v in shape.split("x"))
        part_bytes = native.gemm_allreduce_part_bytes(M, N, world)
        peer = PeerGroup(world, rank, staging_bytes=part_bytes + M * N * 2 + 8192, device=dev)
        r_out, r_part = peer.region("out", M * N * 2), peer.region("part", part_bytes)
        a = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        b = (torch.randn(N, K, device=dev) * 0.5).to(torch.bfloat16)
        part = torch.empty(M, N, dtype=torch.float32, device=dev)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

        def fused():
            native.gemm_bf16_tc_allreduce(a, b, peer.comm, r_part.offset, r_out.offset, status=peer.status_ptr)
            native.wait_signal(peer.comm, native.SIG_GEMM)

        def baseline():
            native.gemm_bf16_tc(a, b, part)
            dist.all_reduce(part)
            out.copy_(part)

        def timed(fn):
            for _ in range(3):
                fn()
            samples = []
            for _ in range(args.iters):
                flush.fill_(1)
                torch.cuda.synchronize()
                dist.barrier()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                fn()
                e.record()
                torch.cuda.synchronize()
                t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                samples.append(float(t[0]))
            return min(samples), statistics.median(samples)

        fb, fm = timed(fused)
        bb, bm = timed(baseline)
        status = peer.read_status()
        sent = M * N * (4 + 2) * (world - 1) / world
        roof = max(2.0 * M * N * K / (peak * 1e12), sent / (link_gbs * 1e9)) * 1e6
        lines.append(f"| {M} x {N} x {K} | {fb * 1e3:.1f} | {fm * 1e3:.1f} | {bb * 1e3:.1f} | {bm * 1e3:.1f} | {bm / fm:.2f}x | {roof:.1f} | "
                     f"{fm * 1e3 / roof:.2f} |" + ("" if status == 0 else f" status {status}"))
        dist.barrier()
        peer.close()
    if rank == 0:
        text = "\n".join(lines) + "\n"
        print(text)
        if args.out:
            args.out.parent.mkdir(parents=True, exist_ok=True)
            args.out.write_text(text)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
