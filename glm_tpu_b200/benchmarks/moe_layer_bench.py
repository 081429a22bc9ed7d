"""One MoE layer at GLM-5.3 dimensions: router -> routed FP8 experts (+ shared expert) -> combine, expert-parallel over the GPUs.

    python -m glm_tpu_b200.benchmarks.moe_layer_bench [--tokens 1,4,64,512,4096] [--iters 20] [--out moe.md]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29547 -m glm_tpu_b200.benchmarks.moe_layer_bench

Hidden 6,144, 256 routed experts (FFN 2,048) top-8 + 1 shared expert, routed weights random e4m3 with 128 x 128 fp32 block scales,
activations bf16 N(0, 1), router bias skewed so that the per-expert load varies about 4x.  1-8 tokens take the decode kernels (route-list
FP8 GEMVs, combine with the in-kernel all-reduce); more tokens take the prefill path (expert sort, grouped tcgen05 GEMM with in-kernel
FP8 decode).  Timing: CUDA events around one layer call, barrier before, maximum over ranks, median of --iters after 3 warm-ups; a 256 MB
buffer is written between calls (weights leave L2).  Roofline per GPU = max(distinct local expert bytes + shared + router bytes over the
measured copy bandwidth, FLOPs over the measured library GEMM peak); the busiest GPU sets the time, so its numbers are reported.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokens", default="1,4,64,512,4096")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist

    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.models.glm_moe_dsa.model import Workspace
    from glm_tpu_b200.runner.gpu_runner import build_runner

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if rank == 0:
        build()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    full = glm53_geometry()
    g = dataclasses.replace(full, num_layers=1, indexer_types=("full",), mlp_layer_types=("sparse",), vocab_size=1024 * world, eos_ids=(1, 2, 3))
    counts = [int(v) for v in args.tokens.split(",")]
    runner = build_runner(g, world=world, rank=rank, device=dev, seed=0, context_capacity=256, lanes=min(8, max(c for c in counts if c <= 8) if any(c <= 8 for c in counts) else 1),
                          prefill_chunk=max(counts), use_graphs=False)
    model, lw = runner.model, runner.model.w.layers[0]
    # skewed expert bias: a linear ramp in shuffled expert order, its amplitude bisected until the 95th-percentile expert gets about 4x the
    # routes of the 5th-percentile one over the largest token count (every rank routes all tokens, so every rank finds the same amplitude)
    gen = torch.Generator().manual_seed(3)
    ramp = torch.linspace(-1.0, 1.0, g.num_routed_experts)[torch.randperm(g.num_routed_experts, generator=gen)].to(dev)
    cal, n_cal = runner._ensure_prefill_ws(), max(counts)
    cal.x[:n_cal].copy_(torch.randn(n_cal, g.hidden_size, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16))

    def load_ratio(amplitude: float) -> float:
        lw.router_bias.copy_(ramp * amplitude)
        model._mlp(cal, lw, 0, n_cal, False)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()  # ranks stay in step: the in-kernel exchanges assume ranks at most one exchange apart
        load = torch.bincount(cal.topk_ids[:n_cal].flatten().long(), minlength=g.num_routed_experts).float().sort().values
        return float(load[int(0.95 * (len(load) - 1))] / load[int(0.05 * (len(load) - 1))].clamp_min(1.0))

    lo_a, hi_a = 0.0, 0.5
    for _ in range(12):
        mid = 0.5 * (lo_a + hi_a)
        lo_a, hi_a = (mid, hi_a) if load_ratio(mid) < 4.0 else (lo_a, mid)
    skew = load_ratio(hi_a)
    peaks_file = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, I, tk, E = g.hidden_size, g.moe_intermediate_size, g.routed_top_k, g.num_routed_experts
    el, ebase = E // world, rank * (E // world)
    expert_bytes = 3 * I * H
    shared_bytes = 3 * model.layout.shared_cols_local * H * 2
    lines = [f"MoE layer at GLM-5.3 dims on {world} GPU(s): hidden {H}, {E} experts x FFN {I} top-{tk} ({el} per GPU, FP8) + shared expert; router bias skewed to a {skew:.1f}x p95/p5 expert load; "
             f"roofline vs {peaks['hbm_gbs']:.0f} GB/s and {peaks['bf16_tflops']:.0f} TFLOP/s (measured)", "",
             "| tokens | path | median us | best us | busiest GPU: distinct experts | routes | MB streamed | GFLOP | roofline us | achieved / roofline |",
             "|---|---|---|---|---|---|---|---|---|---|"]
    for tokens in counts:
        decode = tokens <= 8
        ws = runner.decode_ws if decode and tokens <= runner.lanes else (runner._ensure_prefill_ws() if not decode else Workspace(model, tokens, f"moe{tokens}"))
        ws.x[:tokens].copy_(torch.randn(tokens, H, generator=torch.Generator().manual_seed(tokens)).to(torch.bfloat16))

        def step():
            model._mlp(ws, lw, 0, tokens, decode)

        for _ in range(3):
            step()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        launch = step
        if decode:  # decode steps are replayed from a CUDA graph, as the engine's decode program is
            graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
            with torch.cuda.graph(graph, stream=side):
                step()
            launch = graph.replay
            launch()
            torch.cuda.synchronize()
        ids = ws.topk_ids[:tokens].clone().cpu()
        mine = ids[(ids >= ebase) & (ids < ebase + el)]
        stats = torch.tensor([float(mine.unique().numel()), float(mine.numel())], dtype=torch.float64, device=dev)
        samples = []
        for _ in range(args.iters):
            flush.fill_(1)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            launch()
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            samples.append(float(t[0]))
        if world > 1:
            dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        distinct, routes = int(stats[0]), int(stats[1])
        streamed = distinct * expert_bytes + shared_bytes + E * H * 2
        flops = 2.0 * routes * 3 * I * H + 2.0 * tokens * 3 * model.layout.shared_cols_local * H
        roof = max(streamed / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)) * 1e6
        med, best = statistics.median(samples) * 1e3, min(samples) * 1e3
        if rank == 0:
            lines.append(f"| {tokens} | {'decode kernels, graph' if decode else 'grouped tcgen05'} | {med:.1f} | {best:.1f} | {distinct} | {routes} | {streamed / 1e6:.1f} | "
                         f"{flops / 1e9:.1f} | {roof:.1f} | {med / roof:.2f} |")
    runner.peer.check_status()
    if rank == 0:
        text = "\n".join(lines) + "\n"
        print(text)
        if args.out:
            args.out.parent.mkdir(parents=True, exist_ok=True)
            args.out.write_text(text)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
