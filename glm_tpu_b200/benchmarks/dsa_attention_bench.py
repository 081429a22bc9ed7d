"""DSA sparse MLA attention block at GLM-5.3 dimensions: decode with 1 and 4 chats at ~32k tokens of context, and a 4,096-token prefill chunk.

    python -m glm_tpu_b200.benchmarks.dsa_attention_bench [--kv-layout striped|replicated] [--iters 20] [--out dsa.md]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29548 -m glm_tpu_b200.benchmarks.dsa_attention_bench

One attention block (64 heads, q_lora 2,048, latent 512 + rope 64, 32 index heads of 128, top-2,048) on a 32,768-slot cache of random
bf16 rows: q_a/kv_a projection -> norms, RoPE, cache write -> q_b -> absorbed query -> indexer scores -> exact top-2,048 -> sparse MLA ->
merge -> value projection -> o_proj (+ all-reduce).  With --kv-layout striped on several GPUs the cache is striped by position and the
queries, scores and (o, m, l) partials are exchanged inside the kernels; replicated keeps a full cache per GPU and attends local heads.
Timing: CUDA events around the block, barrier before, maximum over ranks, median of --iters after 3 warm-ups, 256 MB written in between.
"""

from __future__ import annotations

import argparse
import dataclasses
import os
import statistics
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kv-layout", default="striped", choices=["striped", "replicated", "auto"])
    ap.add_argument("--depth", type=int, default=30000)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--topk-cluster", type=int, choices=[0, 1], help="force the 8-CTA-cluster (1) or the single-CTA (0) top-k kernel (A/B runs)")
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist

    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.runner.gpu_runner import build_runner

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if rank == 0:
        build()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    g = dataclasses.replace(glm53_geometry(), num_layers=1, indexer_types=("full",), mlp_layer_types=("dense",), vocab_size=1024 * world, eos_ids=(1, 2, 3))
    runner = build_runner(g, world=world, rank=rank, device=dev, seed=0, context_capacity=32768, lanes=4, prefill_chunk=4096, use_graphs=False,
                          kv_layout=args.kv_layout)
    model, st, lw = runner.model, runner.state, runner.model.w.layers[0]
    if args.topk_cluster is not None:
        from glm_tpu_b200.ops import native as _native

        _native.set_topk_cluster(args.topk_cluster)
    for lane in range(4):
        runner.synthetic_context(lane, args.depth - 97 * lane, seed=lane)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        # every call is fenced by a synchronize and a barrier, warm-ups included: the in-kernel exchanges assume ranks at most one
        # exchange apart (in the model the MLP's all-reduce between two attention blocks sees to that), and their waits give up
        # after about a second, less than the skew of ranks that have just filled their caches at their own pace
        for _ in range(3):
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            fn()
        samples = []
        for _ in range(args.iters):
            flush.fill_(1)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            samples.append(float(t[0]))
        if rank == 0 and max(samples) > 5 * min(samples):
            print("uneven samples (ms):", " ".join(f"{v:.2f}" for v in samples), flush=True)
        return statistics.median(samples) * 1e3, min(samples) * 1e3

    flagged = []

    def status_of(case: str) -> str:
        """The device status word after a case (0 = clean); a wait that ran out or a clamped index is reported beside its case."""
        torch.cuda.synchronize()
        value = runner.peer.read_status()
        if value:
            flagged.append((case, value))
        return "ok" if not value else f"status {value:#x}"

    lines = [f"DSA attention block at GLM-5.3 dims on {world} GPU(s), kv layout {runner.kv_layout}, 32,768-slot cache, chats {args.depth} tokens deep, eager launches", "",
             "| case | rows | median us | best us | device status |", "|---|---|---|---|---|"]
    ws = runner.decode_ws
    frozen = torch.zeros(4, dtype=torch.int32, device=dev)  # inactive rows: the block runs in full but writes no cache row and advances nothing
    for rows in (1, 4):
        ws.x[:rows].copy_(torch.randn(rows, g.hidden_size, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16))

        def decode_block(rows=rows):
            model._attention(ws, lw, 0, rows, st.positions, st.lane_ids, frozen, st, True, runner.cache.context_capacity)

        med, best = timed(decode_block)
        lines.append(f"| decode, {rows} chat(s) at depth {args.depth} | {rows} | {med:.1f} | {best:.1f} | {status_of(f'decode {rows}')} |")
    pws = runner._ensure_prefill_ws()
    rows = 4096
    pws.x[:rows].copy_(torch.randn(rows, g.hidden_size, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16))
    start = 32768 - rows - 1
    pos = torch.arange(start, start + rows, dtype=torch.int32, device=dev)
    lane_t = torch.zeros(rows, dtype=torch.int32, device=dev)

    def prefill_block():
        model._attention(pws, lw, 0, rows, pos, lane_t, None, st, False, start + rows, 0)

    med, best = timed(prefill_block)
    lines.append(f"| prefill chunk of 4,096 rows at positions {start}..{start + rows - 1} (every row selects 2,048 of > 28k keys) | {rows} | {med:.1f} | {best:.1f} | "
                 f"{status_of('prefill chunk')} |")
    from glm_tpu_b200.ops import native

    with native.kernel_timeline() as tl:  # one more pass with every launch bracketed by events: where the chunk's time goes
        prefill_block()
        torch.cuda.synchronize()
        agg: dict = {}
        for name, _, ms in tl.rows():
            agg.setdefault(name, [0, 0.0])
            agg[name][0] += 1
            agg[name][1] += ms
    lines += ["", "| kernel of the prefill chunk | launches | total ms |", "|---|---|---|"]
    lines += [f"| {k} | {c} | {t:.2f} |" for k, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])]
    status_of("timeline pass")
    if flagged:
        print(f"rank {rank}: device status raised in {flagged}", flush=True)
    if rank == 0:
        text = "\n".join(lines) + "\n"
        print(text)
        if args.out:
            args.out.parent.mkdir(parents=True, exist_ok=True)
            args.out.write_text(text)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 1 if flagged else 0


if __name__ == "__main__":
    raise SystemExit(main())
