"""Per-kernel device time of one decode step, with a bytes model and the fraction of the memory roofline.

    python -m glm_tpu_b200.benchmarks.decode_breakdown --layers 6 --depth 30000 --chats 1 --steps 20 --out breakdown.md

Builds the GLM-5.3 architecture (random FP8 weights) truncated to ``--layers`` layers on one GPU, makes the lane(s)
``--depth`` tokens deep (``synthetic_context``), and runs eager decode steps with every launch bracketed by CUDA events
(programmatic dependent launch off, so the brackets do not overlap).  ``--shard 8`` shrinks the expert count and the
vocabulary to what one GPU of eight holds (32 experts, 19,360 vocabulary rows) while each kernel keeps its per-GPU
shape; attention still runs all 64 heads unless ``--heads`` cuts them.

Per entry point and shape it prints launches per step, mean microseconds, the share of the step, the bytes the kernel
has to stream (weights or cache rows: each step touches different weights, far more than the 126 MB L2 in total) and
the achieved bandwidth as a fraction of the measured copy bandwidth (``MEASURED_PEAKS.json`` next to the repository
root when present, else 6,650 GB/s).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
from collections import OrderedDict
from pathlib import Path


def bytes_model(name: str, ints: tuple, g, depth: int, lanes: int):
    """Bytes a launch must stream from HBM (None: latency-bound helper kernels)."""
    H, I = g.hidden_size, g.moe_intermediate_size
    if name == "skinny_bf16":
        _, rows, _, N, K, _, _, batch = ints[:8]
        return N * K * 2 * batch
    if name == "skinny_bf16_swiglu":
        _, rows, _, N, K = ints[:5]
        return 2 * N * K * 2
    if name == "moe_gateup_fp8":
        tiles = ints[2]
        return tiles * 2 * I * H
    if name == "moe_down_fp8":
        tiles = ints[0]
        return tiles * I * H
    if name == "sparse_mla_partial":
        rows = ints[0]
        return rows * min(depth + 1, g.index_top_k) * g.kv_row_width * 2
    if name == "indexer_score":
        rows = ints[0]
        return rows * (depth + 1) * g.index_head_dim * 2
    if name == "topk_select":
        rows = ints[0]
        return rows * (depth + 1) * 4
    return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--depth", type=int, default=30000)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--chats", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--shard", type=int, default=1, help="emulate one GPU of this many: experts and vocabulary divided")
    ap.add_argument("--kv-layout", default="auto", choices=["auto", "striped", "replicated"])
    ap.add_argument("--tail", type=int, default=48, help="also list this many of the step's last launches in order")
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)
    os.environ["GLM_B200_PDL"] = "0"

    import torch

    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.ops import native
    from glm_tpu_b200.runner.gpu_runner import build_runner

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if rank == 0:
        build()
    if world > 1:  # one process per GPU (torch.distributed.run): in-kernel collectives, times include the waits on peers
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
    g = glm53_geometry().truncated(args.layers)
    if args.shard > 1:
        g = dataclasses.replace(g, num_routed_experts=g.num_routed_experts // args.shard, vocab_size=g.vocab_size // args.shard,
                                eos_ids=tuple(e % (g.vocab_size // args.shard) for e in g.eos_ids))
    peaks_file = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks_file.read_text())["hbm_gbs"] if peaks_file.exists() else 6650.0
    runner = build_runner(g, world=world, rank=rank, device=torch.device("cuda", local_rank), seed=0, context_capacity=args.context,
                          lanes=args.chats, use_graphs=False, kv_layout=args.kv_layout)
    for lane in range(args.chats):
        runner.synthetic_context(lane, args.depth - lane * 97, seed=lane)
    for _ in range(args.warmup):
        runner.decode_step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        runner.decode_step()
    stop.record()
    torch.cuda.synchronize()
    eager_ms = start.elapsed_time(stop) / args.steps
    with native.kernel_timeline() as tl:
        for _ in range(args.steps):
            runner.decode_step()
        rows = tl.rows()
    runner.peer.check_status()
    if world > 1:
        dist.barrier()
        if rank != 0:
            dist.destroy_process_group()
            return 0

    groups: OrderedDict = OrderedDict()
    for name, ints, ms in rows:
        model = bytes_model(name, ints, g, args.depth, args.chats)
        key = (name, model)
        groups.setdefault(key, []).append(ms)
    total_us = sum(sum(v) for v in groups.values()) / args.steps * 1e3
    lines = [
        f"decode step breakdown: GLM-5.3 architecture, {args.layers} layers ({g.mlp_layer_types.count('dense')} dense + "
        f"{g.mlp_layer_types.count('sparse')} MoE; {len(g.full_layers)} with their own indexer), {g.num_routed_experts} experts, "
        f"vocabulary {g.vocab_size}, {args.chats} chat(s) at depth {args.depth} of {args.context} slots, {world} GPU(s) (rank 0 shown, "
        f"kv layout {runner.kv_layout}), eager launches, "
        f"programmatic dependent launch off",
        f"eager step {eager_ms * 1e3:.0f} us; sum of bracketed kernels {total_us:.0f} us over {len(rows) // args.steps} launches; "
        f"memory roofline = {hbm:.0f} GB/s (measured copy bandwidth)",
        "",
        "| kernel | launches/step | median us | share | MB streamed | GB/s | of measured HBM |",
        "|---|---|---|---|---|---|---|",
    ]
    for (name, model), times in sorted(groups.items(), key=lambda kv: -sum(kv[1])):
        per_step = len(times) / args.steps
        med = statistics.median(times) * 1e3
        share = sum(times) / args.steps * 1e3 / total_us
        if model:
            gbs = model / (med * 1e-6) / 1e9
            lines.append(f"| {name} | {per_step:g} | {med:.1f} | {share:.1%} | {model / 1e6:.2f} | {gbs:.0f} | {gbs / hbm:.2f} |")
        else:
            lines.append(f"| {name} | {per_step:g} | {med:.1f} | {share:.1%} | - | - | - |")
    per_step = len(rows) // args.steps
    if args.tail > 0:
        lines += ["", f"launch order of the last {min(args.tail, per_step)} launches of the last step (us): "
                  + ", ".join(f"{name} {ms * 1e3:.1f}" for name, _, ms in rows[-min(args.tail, per_step):])]
    text = "\n".join(lines) + "\n"
    print(text)
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(text)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
