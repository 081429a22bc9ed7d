"""Time of every phase of the persistent decode kernel, from the device's own clock.

    python -m glm_tpu_b200.benchmarks.mega_phases --layers 12 --depth 30000 --chats 1 --steps 20
    python -m torch.distributed.run --nproc-per-node 8 ... -m glm_tpu_b200.benchmarks.mega_phases --layers 78

CTA 0 of the persistent kernel stamps ``%globaltimer`` after every phase and its grid barrier (``MegaDecoder.enable_timeline``);
the step is replayed from its CUDA graph, so the figures are those of the production launch sequence.  The indexer and top-k
kernels between two stretches show up as the gap before a stretch's first stamp.  Printed per phase kind: occurrences per step,
median and total microseconds, the bytes of weights the phase streams on this GPU and the bandwidth that amounts to.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
from pathlib import Path

PHASES = {1: "qkv_a", 2: "q_b", 3: "absorb", 4: "attn", 5: "merge", 6: "vproj", 7: "oproj", 8: "mlp_a", 9: "mlp_b", 10: "moe_down", 11: "combine"}
HEAD = {1: "lm_head", 2: "finalize"}


def phase_bytes(g, layout, layer: int, phase: int, routes_local: float) -> int | None:
    """Weight bytes phase ``phase`` of ``layer`` streams on one GPU (None: no weight stream)."""
    H, hl = g.hidden_size, layout.heads_local
    full = g.indexer_types[layer] == "full"
    dense = g.mlp_layer_types[layer] == "dense"
    if phase == 1:
        return (g.q_lora_rank + g.kv_row_width + ((g.index_head_dim + g.index_heads) if full else 0)) * H * 2
    if phase == 2:
        return (hl * g.qk_head_dim + (g.index_heads * g.index_head_dim if full else 0)) * g.q_lora_rank * 2
    if phase == 3:
        return hl * g.qk_nope_head_dim * g.kv_lora_rank * 2
    if phase == 6:
        return hl * g.v_head_dim * g.kv_lora_rank * 2
    if phase == 7:
        return H * hl * g.v_head_dim * 2
    if phase == 8:
        return 2 * layout.dense_cols_local * H * 2 if dense else (g.num_routed_experts + 2 * layout.shared_cols_local) * H * 2
    if phase == 9:
        if dense:
            return H * layout.dense_cols_local * 2
        return int(routes_local * 2 * g.moe_intermediate_size * H) + H * layout.shared_cols_local * 2
    if phase == 10 and not dense:
        return int(routes_local * g.moe_intermediate_size * H)
    return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--depth", type=int, default=30000)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--chats", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--emulate-world", type=int, default=1,
                    help="on ONE GPU: hold rank 0's shard of a layout over this many GPUs and skip every exchange (what a GPU of the box "
                         "spends outside the exchanges; the outputs mean nothing)")
    ap.add_argument("--repeat", action="store_true", help="run every phase twice in a row (world 1 only): the second run has warm code and operands")
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)

    import torch

    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.runner.gpu_runner import build_runner

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if rank == 0:
        build()
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
    g = glm53_geometry().truncated(args.layers)
    emulate = args.emulate_world > 1 and world == 1
    peaks_file = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks_file.read_text())["hbm_gbs"] if peaks_file.exists() else 6650.0
    runner = build_runner(g, world=args.emulate_world if emulate else world, rank=rank, device=torch.device("cuda", local_rank), seed=0,
                          context_capacity=args.context, lanes=args.chats, use_graphs=True, decode_path="mega", emulate_shard=emulate,
                          kv_layout="replicated" if emulate else "auto")
    for lane in range(args.chats):
        runner.synthetic_context(lane, args.depth - lane * 97, seed=lane)
    if args.repeat:
        runner.mega.args.compat_ksplit = 2
    runner.mega.enable_timeline(4 * (12 * args.layers + 8) * (args.steps + 1))
    rec = runner.build_decode_program()
    for _ in range(args.warmup):
        runner.decode_step()
    runner.mega.read_timeline()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        runner.decode_step()
    stop.record()
    torch.cuda.synchronize()
    step_ms = start.elapsed_time(stop) / args.steps
    stamps = runner.mega.read_timeline()
    barrier_ns = {v: runner.mega.barrier_nanoseconds(2000, v) for v in (0, 1, 2)}
    runner.peer.check_status()
    if world > 1:
        dist.barrier()
        if rank != 0:
            runner.close()
            dist.destroy_process_group()
            return 0

    routes_local = args.chats * g.routed_top_k / max(world, args.emulate_world if emulate else 1)
    groups: dict = {}
    for layer, code, us in stamps:
        phase, before_barrier, inner = code & 127, bool(code & 128), code >> 16
        if inner or before_barrier:
            name = (HEAD if layer >= g.num_layers else PHASES).get(phase, str(phase))
            if inner == 7:
                key = f"  {name}: own work of CTA 0, first run"
            elif inner == 8:
                key = f"  {name}: barrier before the second run"
            else:
                key = f"  {name}: " + (f"up to step {inner}" if inner else "own work of CTA 0 (last run; the rest of the phase is the wait for the slowest CTA + barrier)")
            groups.setdefault(key, {"us": [], "bytes": None})["us"].append(us)
            continue
        if layer >= g.num_layers:
            key, nbytes = ("head." + HEAD.get(phase, str(phase))) if phase else "gap before a stretch (indexer + top-k, launch)", None
            if phase == 1:
                nbytes = runner.layout.vocab_local * g.hidden_size * 2
        elif phase == 0:
            key, nbytes = "gap before a stretch (indexer + top-k, launch)", None
        else:
            kind = ("dense." if g.mlp_layer_types[layer] == "dense" and phase >= 8 else "") + PHASES[phase]
            if phase in (1, 2) and g.indexer_types[layer] == "full":
                kind += " (full)"
            key, nbytes = kind, phase_bytes(g, runner.layout, layer, phase, routes_local)
        groups.setdefault(key, {"us": [], "bytes": nbytes})["us"].append(us)
    total = sum(sum(v["us"]) for v in groups.values()) / args.steps
    lines = [
        f"persistent decode kernel, per phase: GLM-5.3 architecture, {args.layers} layers, {g.num_routed_experts} experts, {args.chats} chat(s) at depth "
        f"{args.depth}, {world} GPU(s) (rank 0 shown{', holding the shard of one GPU of ' + str(args.emulate_world) + ' with the exchanges skipped' if emulate else ''}), CUDA-graph replay, {rec.launches} launches per step, grid {runner.mega.grid()} CTAs",
        f"step {step_ms * 1e3:.0f} us (CUDA events over {args.steps} steps); sum of stamped intervals {total:.0f} us; HBM {hbm:.0f} GB/s measured copy bandwidth",
        "grid barrier alone (2,000 back to back): " + ", ".join(f"variant {v}: {ns / 1e3:.2f} us" for v, ns in barrier_ns.items())
        + " (1 = counter and generation on separate lines, relaxed polling: the one in use; 0 = first form; 2 = per-CTA arrival words)",
        "",
        "| phase (+ its barrier) | per step | median us | us per step | share | weight MB | GB/s | of measured HBM |",
        "|---|---|---|---|---|---|---|---|",
    ]
    for key, v in sorted(groups.items(), key=lambda kv: -sum(kv[1]["us"])):
        med, per = statistics.median(v["us"]), len(v["us"]) / args.steps
        tot = sum(v["us"]) / args.steps
        if v["bytes"]:
            gbs = v["bytes"] / (med * 1e-6) / 1e9
            lines.append(f"| {key} | {per:g} | {med:.1f} | {tot:.0f} | {tot / total:.1%} | {v['bytes'] / 1e6:.2f} | {gbs:.0f} | {gbs / hbm:.2f} |")
        else:
            lines.append(f"| {key} | {per:g} | {med:.1f} | {tot:.0f} | {tot / total:.1%} | - | - | - |")
    text = "\n".join(lines) + "\n"
    print(text)
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(text)
    runner.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
