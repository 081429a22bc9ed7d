"""One rank of the multi-GPU model test (launched by ``tests/test_gpu_multi.py`` through torch.distributed.run).

Every rank shards the same small checkpoint, runs prefill + greedy decode with the in-kernel (peer-memory) collectives
and again with the NCCL baseline, and rank 0 writes the tokens and the discrete decisions to ``--out`` as JSON.
"""

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def run(g, ckpt, prompt, new_tokens, capacity, stripe, comm, use_graphs, record, world, rank, device, lanes=1, kv_layout="striped",
        expert_split=None):
    from glm_tpu_b200.runner.gpu_runner import build_runner

    runner = build_runner(g, world=world, rank=rank, device=device, checkpoint=ckpt, context_capacity=capacity, lanes=lanes,
                          stripe=stripe, use_graphs=use_graphs, prefill_chunk=32, comm=comm, wait_limit=4_000_000, kv_layout=kv_layout,
                          expert_split=expert_split)
    split = runner.model.layout.expert_split
    decisions = {"selected": {i: [] for i in g.full_layers}, "experts": {i: [] for i in g.sparse_layers}}
    if record:
        inner = runner.model.run_rows

        def recording(*a, **k):
            runner.model.trace = {}
            out = inner(*a, **k)
            t = runner.model.trace
            for layer in g.full_layers:
                for row in t["sel_global"][layer].cpu():
                    decisions["selected"][layer].append(row[row >= 0].tolist())
            for layer in g.sparse_layers:
                decisions["experts"][layer] += t["topk_ids"][layer].cpu().tolist()
            runner.model.trace = None
            return out

        runner.model.run_rows = recording
    firsts = [runner.prefill(lane, prompt[lane]) for lane in range(lanes)]
    runner.build_decode_program()
    if record:
        for layer in g.full_layers:
            del decisions["selected"][layer][-lanes:]
        for layer in g.sparse_layers:
            del decisions["experts"][layer][-lanes:]
    out = [[t] for t in firsts]
    for step in range(new_tokens - 1):
        runner.decode_step()
        for lane, tok in enumerate(runner.read_step_tokens(step)):
            out[lane].append(tok)
    runner.peer.check_status()
    kind = runner.report.programs[-1].kind
    runner.close()
    run.last_split = split
    return out, decisions, kind


def gemm_allreduce_check(world, rank, device):
    """The tcgen05 GEMM with the fused NVLink all-reduce against fp32 partial products summed by the library all-reduce."""
    from glm_tpu_b200.ops import native
    from glm_tpu_b200.parallel.peer import PeerGroup

    out = {}
    for rows, N, K in ((300, 1024, 512), (1000, 6144, 256), (128, 520, 2048)):
        part_bytes = native.gemm_allreduce_part_bytes(rows, N, world)
        peer = PeerGroup(world, rank, staging_bytes=part_bytes + rows * N * 2 + 8192, device=device)
        r_out = peer.region("out", rows * N * 2)
        r_part = peer.region("part", part_bytes)
        got = peer.tensor(r_out, (rows, N), torch.bfloat16)
        gen = torch.Generator().manual_seed(100 * rank + rows)
        a = (torch.randn(rows, K, generator=gen) * 0.5).to(torch.bfloat16).to(device)
        b = (torch.randn(N, K, generator=gen) * 0.5).to(torch.bfloat16).to(device)
        worst = 0.0
        for round_ in range(3):  # several rounds through the same slots and flags
            got.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            native.gemm_bf16_tc_allreduce(a, b, peer.comm, r_part.offset, r_out.offset, status=peer.status_ptr)
            native.wait_signal(peer.comm, native.SIG_GEMM)
            ref = a.float() @ b.float().T
            dist.all_reduce(ref)
            torch.cuda.synchronize()
            err = (got.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
            worst = max(worst, err if err == err else 1e9)
            a = (a.float() * -0.5 + 0.25).to(torch.bfloat16)
        peer.check_canaries()  # the pushes of both ranks stayed inside their regions
        out[f"{rows}x{N}x{K}"] = {"rel_err": worst, "status": peer.read_status()}
        dist.barrier()
        peer.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)

    from glm_tpu_b200.config.model import small_geometry
    from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint

    import dataclasses

    # the routed experts' width grows with the GPU count so that a column slice stays a whole FP8 block at every world size
    g = dataclasses.replace(small_geometry(4), moe_intermediate_size=128 * world)
    ckpt = random_checkpoint(g, seed=5)
    gen = torch.Generator().manual_seed(5)
    prompt = [torch.randint(0, g.vocab_size, (70,), generator=gen).tolist()]
    result = {"world": world, "moe_intermediate_size": g.moe_intermediate_size}
    fused, decisions, _ = run(g, ckpt, prompt, 10, 128, 16, "fused", False, True, world, rank, device)
    result["fused_eager"] = fused[0]
    result["default_split"] = run.last_split
    # the other split of the routed experts (whole experts per GPU), eager with recorded decisions and as a graph
    other = "whole" if run.last_split == "sliced" else "sliced"
    alt, alt_dec, _ = run(g, ckpt, prompt, 10, 128, 16, "fused", False, True, world, rank, device, expert_split=other)
    result["other_split"], result["other_split_eager"] = other, alt[0]
    result["other_split_decisions"] = {"selected": {str(k): v for k, v in alt_dec["selected"].items()},
                                       "experts": {str(k): v for k, v in alt_dec["experts"].items()}}
    alt_graph, _, _ = run(g, ckpt, prompt, 10, 128, 16, "fused", True, False, world, rank, device, expert_split=other)
    result["other_split_graph"] = alt_graph[0]
    result["decisions"] = {"selected": {str(k): v for k, v in decisions["selected"].items()},
                           "experts": {str(k): v for k, v in decisions["experts"].items()}}
    graph, _, kind = run(g, ckpt, prompt, 10, 128, 16, "fused", True, False, world, rank, device)
    result["fused_graph"], result["fused_graph_kind"] = graph[0], kind
    nccl, _, _ = run(g, ckpt, prompt, 10, 128, 16, "nccl", False, False, world, rank, device)
    result["nccl"] = nccl[0]
    # two concurrent chats with different prompts through the batched decode program
    prompts2 = [prompt[0][:40], prompt[0][20:65]]
    both, _, _ = run(g, ckpt, prompts2, 6, 128, 16, "fused", True, False, world, rank, device, lanes=2)
    result["two_lanes"] = both
    # the same chat with a full cache replica per GPU (no attention exchange), graph and NCCL-baseline variants
    rep_eager, rep_dec, _ = run(g, ckpt, prompt, 10, 128, 16, "fused", False, True, world, rank, device, kv_layout="replicated")
    result["replicated_eager"] = rep_eager[0]
    result["replicated_decisions"] = {"selected": {str(k): v for k, v in rep_dec["selected"].items()},
                                      "experts": {str(k): v for k, v in rep_dec["experts"].items()}}
    rep, _, _ = run(g, ckpt, prompt, 10, 128, 16, "fused", True, False, world, rank, device, kv_layout="replicated")
    result["replicated_graph"] = rep[0]
    result["prompt"] = prompt[0]
    result["gemm_allreduce"] = gemm_allreduce_check(world, rank, device)
    gathered = [None] * world
    dist.all_gather_object(gathered, result["fused_graph"])
    result["all_ranks_agree"] = all(x == gathered[0] for x in gathered)
    if rank == 0:
        Path(args.out).write_text(json.dumps(result))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
