"""Bytes a decode step must stream from HBM on one GPU, and the time the measured copy bandwidth allows for them.

    python -m glm_tpu_b200.benchmarks.roofline_model [--gpus 1,2,4,8] [--chats 1] [--depth 200] [--measured 1:2.175,2:3.788,8:11.02]

Decode is weight streaming: with 1-8 rows every matrix a step touches is read once and used for a handful of FLOPs per byte, so the
lower bound of a step is (bytes the busiest GPU reads) / (copy bandwidth).  The bytes are counted from the geometry and the parallel
layout, tensor by tensor, exactly as `models/glm_moe_dsa/weights.py` lays them out on a GPU:

* attention, per layer: the fused q_a | kv_a (| indexer key | indexer weights) projection (replicated), q_b of this GPU's heads (| the
  indexer query projection), kv_b and the o_proj slice of this GPU's heads, all bf16;
* dense layers: this GPU's columns of gate / up / down (bf16); MoE layers: the router (bf16, replicated), this GPU's columns of the
  shared expert (bf16) and, per route that lands on one of this GPU's experts, the three FP8 matrices of that expert with their
  block scales (a repeated expert is read once; the busiest GPU is found by sampling routes uniformly);
* caches: min(depth, top-k) latent rows per layer and chat, and on full-indexer layers the index keys of the whole context (all of
  them with a replicated cache, a 1 / N slice with a striped one);
* once per step: this GPU's rows of the lm_head (bf16).

N GPUs hold `round(78 N / 8)` layers when `--layers` is not given, as `bench.py` runs them.  No GPU is needed to run this module.
"""

from __future__ import annotations

import argparse
import json
import random
from pathlib import Path

from glm_tpu_b200.config.model import ModelGeometry, glm53_geometry
from glm_tpu_b200.config.parallel import ParallelLayout

FALLBACK_HBM_GBS = 6650.0


def measured_hbm_gbs() -> tuple[float, str]:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def expert_bytes(g: ModelGeometry) -> int:
    """One routed expert: gate, up, down in FP8 plus their fp32 block scales."""
    bn, bk = g.fp8_block_shape
    cells = 3 * g.moe_intermediate_size * g.hidden_size
    scales = 2 * (-(-g.moe_intermediate_size // bn)) * (-(-g.hidden_size // bk)) + (-(-g.hidden_size // bn)) * (-(-g.moe_intermediate_size // bk))
    return cells + 4 * scales


def busiest_gpu_experts(g: ModelGeometry, world: int, chats: int, samples: int = 4000, seed: int = 0) -> tuple[float, float]:
    """(mean over GPUs, expected maximum over GPUs) of the distinct local experts one step touches, routes drawn uniformly."""
    rng = random.Random(seed)
    per = g.num_routed_experts // world
    total_mean = total_max = 0.0
    for _ in range(samples):
        touched = set()
        for _ in range(chats):
            touched.update(rng.sample(range(g.num_routed_experts), g.routed_top_k))
        counts = [0] * world
        for e in touched:
            counts[e // per] += 1
        total_mean += sum(counts) / world
        total_max += max(counts)
    return total_mean / samples, total_max / samples


def decode_step_bytes(g: ModelGeometry, world: int, *, chats: int = 1, depth: int = 200, striped: bool = False,
                      expert_split: str = "whole") -> dict:
    """``expert_split='sliced'``: every GPU streams ``1 / world`` of every touched expert, so mean and busiest coincide."""
    lay = ParallelLayout(g, world, 0)
    H, Q, L, rd = g.hidden_size, g.q_lora_rank, g.kv_lora_rank, g.qk_rope_head_dim
    hl = lay.heads_local
    attention = caches = dense = shared = router = 0
    for layer in range(g.num_layers):
        full = g.indexer_types[layer] == "full"
        n_qkv = Q + L + rd + ((g.index_head_dim + g.index_heads) if full else 0)
        n_qb = hl * g.qk_head_dim + (g.index_heads * g.index_head_dim if full else 0)
        attention += 2 * (n_qkv * H + n_qb * Q + hl * g.kv_b_rows_per_head * L + H * hl * g.v_head_dim)
        caches += chats * min(depth, g.index_top_k) * g.kv_row_width * 2
        if full:
            caches += chats * (depth // (world if striped else 1)) * g.index_head_dim * 2
        if g.mlp_layer_types[layer] == "dense":
            dense += 2 * 3 * lay.dense_cols_local * H
        else:
            router += 2 * g.num_routed_experts * H
            shared += 2 * 3 * lay.shared_cols_local * H
    moe_layers = sum(1 for t in g.mlp_layer_types if t != "dense")
    mean_e, max_e = busiest_gpu_experts(g, world, chats)
    if expert_split == "sliced" and world > 1:
        mean_e = max_e = mean_e  # the touched experts of the whole box, divided evenly: what `mean` already is
    routed_mean, routed_max = moe_layers * mean_e * expert_bytes(g), moe_layers * max_e * expert_bytes(g)
    head = 2 * lay.vocab_local * H
    fixed = attention + caches + dense + shared + router + head
    return {"attention": attention, "caches": caches, "dense_mlp": dense, "shared_expert": shared, "router": router, "lm_head": head,
            "routed_mean": routed_mean, "routed_busiest": routed_max, "total_mean": fixed + routed_mean, "total_busiest": fixed + routed_max,
            "experts_per_layer_mean": mean_e, "experts_per_layer_busiest": max_e}


def measured_tflops() -> tuple[float, str]:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def prefill_flops(g: ModelGeometry, world: int, tokens: int) -> dict:
    """Floating-point operations one GPU performs to prefill a fresh prompt of ``tokens`` (2 per multiply-add; the three-piece index
    query counts once: it is the useful work that is reported, not the issued one).  Routed work is spread evenly over the GPUs."""
    lay = ParallelLayout(g, world, 0)
    H, Q, L = g.hidden_size, g.q_lora_rank, g.kv_lora_rank
    hl = lay.heads_local
    keys = sum(min(p + 1, g.index_top_k) for p in range(tokens))  # attended keys, summed over the rows
    context = tokens * (tokens + 1) // 2                           # scored keys, summed over the rows
    proj = attn = index = mlp = routed = 0
    for layer in range(g.num_layers):
        full = g.indexer_types[layer] == "full"
        n_qkv = Q + L + g.qk_rope_head_dim + ((g.index_head_dim + g.index_heads) if full else 0)
        n_qb = hl * g.qk_head_dim + (g.index_heads * g.index_head_dim if full else 0)
        proj += 2 * tokens * (n_qkv * H + n_qb * Q + hl * g.kv_b_rows_per_head * L + H * hl * g.v_head_dim)
        attn += 2 * keys * hl * (g.kv_row_width + L)
        if full:
            index += 2 * context * g.index_heads * g.index_head_dim  # replicated cache: every GPU scores every row
        if g.mlp_layer_types[layer] == "dense":
            mlp += 2 * tokens * 3 * lay.dense_cols_local * H
        else:
            mlp += 2 * tokens * (3 * lay.shared_cols_local * H + g.num_routed_experts * H)
            routed += 2 * tokens * g.routed_top_k * 3 * g.moe_intermediate_size * H // world
    head = 2 * lay.vocab_local * H
    return {"projections": proj, "attention": attn, "indexer": index, "dense_shared_router": mlp, "routed_experts": routed, "lm_head": head,
            "total": proj + attn + index + mlp + routed + head}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", default="1,2,4,8")
    ap.add_argument("--chats", type=int, default=1)
    ap.add_argument("--depth", type=int, default=200)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--striped", action="store_true")
    ap.add_argument("--expert-split", default="sliced", choices=["sliced", "whole"], help="routed experts per GPU (several GPUs)")
    ap.add_argument("--small-box-layers", type=int, default=12, help="layers on fewer than 8 GPUs (0: round(78 N / 8), the earlier scheme)")
    ap.add_argument("--measured", default="", help="N:ms per step, comma separated, to print the achieved fraction")
    ap.add_argument("--prefill", type=int, default=0, help="also print the compute bound of prefilling a fresh prompt of this many tokens")
    ap.add_argument("--measured-prefill", default="", help="N:ms of that prefill, comma separated")
    args = ap.parse_args(argv)
    bw, kind = measured_hbm_gbs()
    measured = {int(k): float(v) for k, v in (item.split(":") for item in args.measured.split(",") if item)}
    print(f"decode step, {args.chats} chat(s) at depth {args.depth}, routed experts {args.expert_split}; roofline = bytes of the busiest GPU / {bw:.0f} GB/s ({kind} copy bandwidth)\n")
    print("| GPUs | layers | attention MB | dense + shared + router MB | routed experts MB (mean / busiest) | caches MB | lm_head MB | total GB (busiest) | roofline ms | measured ms | roofline / measured |")
    print("|---|---|---|---|---|---|---|---|---|---|---|")
    for world in (int(v) for v in args.gpus.split(",")):
        layers = args.layers or (78 if world >= 8 else (args.small_box_layers or max(4, round(78 * world / 8))))
        g = glm53_geometry() if layers == 78 else glm53_geometry().truncated(layers)
        b = decode_step_bytes(g, world, chats=args.chats, depth=args.depth, striped=args.striped, expert_split=args.expert_split)
        roof_ms = b["total_busiest"] / (bw * 1e9) * 1e3
        got = measured.get(world)
        mb = lambda x: f"{x / 1e6:,.0f}"  # noqa: E731
        print(f"| {world} | {layers} | {mb(b['attention'])} | {mb(b['dense_mlp'] + b['shared_expert'] + b['router'])} | {mb(b['routed_mean'])} / {mb(b['routed_busiest'])} | "
              f"{mb(b['caches'])} | {mb(b['lm_head'])} | {b['total_busiest'] / 1e9:.2f} | {roof_ms:.3f} | {'' if got is None else f'{got:.3f}'} | "
              f"{'' if got is None else f'{roof_ms / got:.2f}'} |")
    if args.prefill:
        tf, kind = measured_tflops()
        got_p = {int(k): float(v) for k, v in (item.split(":") for item in args.measured_prefill.split(",") if item)}
        print(f"\nprefill of a fresh {args.prefill}-token prompt; bound = FLOPs of one GPU / {tf:.0f} TFLOP/s ({kind} library GEMM peak)\n")
        print("| GPUs | layers | projections | attention | indexer | dense + shared + router | routed experts | total TFLOP per GPU | bound ms | measured ms | bound / measured |")
        print("|---|---|---|---|---|---|---|---|---|---|---|")
        for world in (int(v) for v in args.gpus.split(",")):
            layers = args.layers or (78 if world >= 8 else (args.small_box_layers or max(4, round(78 * world / 8))))
            g = glm53_geometry() if layers == 78 else glm53_geometry().truncated(layers)
            f = prefill_flops(g, world, args.prefill)
            bound = f["total"] / (tf * 1e12) * 1e3
            got = got_p.get(world)
            t = lambda x: f"{x / 1e12:.1f}"  # noqa: E731
            print(f"| {world} | {layers} | {t(f['projections'])} | {t(f['attention'])} | {t(f['indexer'])} | {t(f['dense_shared_router'])} | {t(f['routed_experts'])} | "
                  f"{t(f['total'])} | {bound:.1f} | {'' if got is None else f'{got:.1f}'} | {'' if got is None else f'{bound / got:.3f}'} |")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
