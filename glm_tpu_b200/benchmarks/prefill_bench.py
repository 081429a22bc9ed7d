"""Prefill throughput and time to first token.

    python -m glm_tpu_b200.benchmarks.prefill_bench --layers 12 --prompt 4096 --chunk 1024 [--repeat 3] [--out prefill.md]
    python -m torch.distributed.run --nproc-per-node 8 ... -m glm_tpu_b200.benchmarks.prefill_bench --layers 78 --prompt 16384

Random-init GLM-5.3 architecture (FP8 experts), uniform random prompt ids.  One prefill = host token ids (pinned) ->
device, every chunk through every layer (tcgen05 projections, DSA indexer + sparse attention, grouped FP8 expert GEMM),
the first token read back by the host: the time measured is the whole of that, by wall clock around a synchronize,
the maximum over ranks, best and median of ``--repeat`` runs after one warm-up.
"""

from __future__ import annotations

import argparse
import os
import statistics
import time
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--chunk", type=int, default=1024)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--kv-layout", default="auto")
    ap.add_argument("--shard", type=int, default=1, help="emulate one GPU of this many: experts and vocabulary divided (small profiling runs)")
    ap.add_argument("--timeline", action="store_true", help="after the timed runs, one more prefill with every launch of the library bracketed by CUDA events")
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist

    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.runner.gpu_runner import build_runner

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if rank == 0:
        build()
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()
    g = glm53_geometry().truncated(args.layers)
    if args.shard > 1:
        import dataclasses

        g = dataclasses.replace(g, num_routed_experts=g.num_routed_experts // args.shard, vocab_size=g.vocab_size // args.shard,
                                eos_ids=tuple(e % (g.vocab_size // args.shard) for e in g.eos_ids))
    runner = build_runner(g, world=world, rank=rank, device=device, seed=0, context_capacity=args.context, lanes=1,
                          prefill_chunk=args.chunk, kv_layout=args.kv_layout)
    gen = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, g.vocab_size, (args.prompt,), generator=gen).tolist()
    times = []
    for i in range(args.repeat + 1):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        token = runner.prefill(0, prompt)
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        if i > 0:
            times.append(float(dt[0]))
    runner.peer.check_status()
    timeline_text = ""
    if args.timeline:
        from glm_tpu_b200.ops import native

        with native.kernel_timeline() as tl:
            t0 = time.perf_counter()
            runner.prefill(0, prompt)
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            rows = tl.rows()
        agg: dict = {}
        for name, _, ms in rows:
            agg.setdefault(name, [0, 0.0])
            agg[name][0] += 1
            agg[name][1] += ms
        total = sum(v[1] for v in agg.values())
        timeline_text = (f"\nbracketed prefill: wall {wall * 1e3:.1f} ms, library kernels {total:.1f} ms over {len(rows)} launches (the rest is framework glue: "
                         f"route sorting, copies, casts)\n| kernel | launches | total ms | share of kernel time |\n|---|---|---|---|\n"
                         + "".join(f"| {k} | {c} | {t:.2f} | {t / total:.1%} |\n" for k, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])))
    if rank == 0:
        best, med = min(times), statistics.median(times)
        text = (f"prefill: GLM-5.3 architecture, {args.layers} of 78 layers, {g.num_routed_experts} experts, {world} GPU(s), kv layout {runner.kv_layout}, prompt {args.prompt} tokens in "
                f"chunks of {args.chunk}, context capacity {args.context}\n"
                f"time to first token: best {best * 1e3:.1f} ms, median {med * 1e3:.1f} ms ({args.repeat} runs after a warm-up)\n"
                f"prefill rate: {args.prompt / best:.0f} tokens/s (best), {args.prompt / med:.0f} tokens/s (median); first token {token}\n" + timeline_text)
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
