"""Decode step time of ONE rank of an N-GPU layout, measured on one GPU.

The process holds the shard rank ``--rank`` of ``--emulate-world`` GPUs would hold (the same weight bytes, the same launches, the
same grids) and skips every exchange, so the figure is a rank's own work per step without the waiting for peers: what is left when
it is subtracted from a real N-GPU step is the cost of the exchanges.  The step is replayed from a CUDA graph and timed with CUDA
events over ``--steps`` steps after ``--warmup``; one row per (decode path, expert split, chats).

    python -m glm_tpu_b200.benchmarks.shard_step_bench --layers 24 --emulate-world 8 --paths kernels --splits sliced,whole --chats 1,4

``--prefill-rows N`` times the prefill of an N-token prompt the same way instead (eager launches, CUDA events over ``--steps``
prefills after ``--warmup``; wall clock beside it, so a host-bound launch sequence shows as wall > device):

    python -m glm_tpu_b200.benchmarks.shard_step_bench --layers 6 --emulate-world 8 --splits sliced --prefill-rows 200 --steps 5 --warmup 3

No counterpart in the reference (its decode step exists only as one compiled program per profile).
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="shard_step_bench")
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--chats", default="1", help="comma separated lane counts")
    ap.add_argument("--emulate-world", type=int, default=8)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--depth", type=int, default=30000)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--paths", default="kernels", help="comma separated: kernels, phases, mega")
    ap.add_argument("--splits", default="sliced,whole", help="comma separated expert splits")
    ap.add_argument("--prefill-rows", type=int, default=0, help="time the prefill of a prompt of this many tokens instead of the decode step")
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)

    import torch

    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.runner.gpu_runner import build_runner

    torch.cuda.set_device(0)
    g = glm53_geometry().truncated(args.layers)
    world, emulate = args.emulate_world, args.emulate_world > 1
    if args.prefill_rows:
        return prefill(args, g, world, emulate)
    lines = [f"decode step of rank {args.rank} of {world} GPU(s) on one GPU (exchanges skipped): GLM-5.3 architecture, {args.layers} layers, "
             f"chats {args.depth} tokens deep in a {args.context}-slot context, CUDA-graph replay, CUDA events over {args.steps} steps", "",
             "| decode path | expert split | chats | launches per step | us per step | us per layer |", "|---|---|---|---|---|---|"]
    for path in args.paths.split(","):
        for split in args.splits.split(","):
            for chats in (int(c) for c in args.chats.split(",")):
                runner = build_runner(g, world=world, rank=args.rank, device="cuda:0", seed=0, context_capacity=args.context, lanes=chats,
                                      use_graphs=True, decode_path=path, emulate_shard=emulate, expert_split=split if world > 1 else None,
                                      kv_layout="replicated" if emulate else "auto")
                try:
                    for lane in range(chats):
                        runner.synthetic_context(lane, args.depth - 97 * lane, seed=lane)
                    record = runner.build_decode_program()
                    for _ in range(args.warmup):
                        runner.decode_step()
                    torch.cuda.synchronize()
                    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    for _ in range(args.steps):
                        runner.decode_step()
                    end.record()
                    torch.cuda.synchronize()
                    us = start.elapsed_time(end) * 1e3 / args.steps
                    runner.peer.check_status()
                    lines.append(f"| {runner.decode_path} | {runner.model.layout.expert_split} | {chats} | {record.launches} | {us:.0f} | {us / args.layers:.1f} |")
                    print(lines[-1], flush=True)
                finally:
                    runner.close()
                    del runner
                    torch.cuda.empty_cache()
    text = "\n".join(lines) + "\n"
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(text)
    else:
        print(text)
    return 0


def prefill(args, g, world: int, emulate: bool) -> int:
    import time

    import torch

    from glm_tpu_b200.runner.gpu_runner import build_runner

    lines = [f"prefill of a {args.prefill_rows}-token prompt by rank {args.rank} of {world} GPU(s) on one GPU (exchanges skipped): GLM-5.3 architecture, "
             f"{args.layers} layers, chunks of {args.prefill_chunk} rows, {args.steps} prefills after {args.warmup}", "",
             "| expert split | device ms per prefill | wall ms per prefill | device us per layer |", "|---|---|---|---|"]
    prompt = torch.randint(0, g.vocab_size, (args.prefill_rows,), generator=torch.Generator().manual_seed(0)).tolist()
    for split in args.splits.split(","):
        runner = build_runner(g, world=world, rank=args.rank, device="cuda:0", seed=0, context_capacity=args.context, lanes=1, use_graphs=True,
                              prefill_chunk=args.prefill_chunk, emulate_shard=emulate, expert_split=split if world > 1 else None,
                              kv_layout="replicated" if emulate else "auto")
        try:
            for _ in range(args.warmup):
                runner.prefill(0, prompt)
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            for _ in range(args.steps):
                runner.prefill(0, prompt)
            end.record()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) * 1e3 / args.steps
            ms = start.elapsed_time(end) / args.steps
            runner.peer.check_status()
            lines.append(f"| {runner.model.layout.expert_split} | {ms:.2f} | {wall:.2f} | {ms * 1e3 / args.layers:.0f} |")
            print(lines[-1], flush=True)
        finally:
            runner.close()
            del runner
            torch.cuda.empty_cache()
    text = "\n".join(lines) + "\n"
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(text)
    else:
        print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
