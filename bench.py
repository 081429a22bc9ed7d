"""Headline benchmark: greedy decode rate of one chat at a 32,768-slot context, GLM-5.3 FP8 architecture.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 64 --warmup 8

A *step* is one decode step (one new token for every live chat).  With 8 GPUs the model is the full 78-layer
GLM-5.3; with 1, 2 or 4 GPUs it is the 12-layer truncation of the same architecture (the full model does not fit),
which the JSON line states in ``config``.  Weights are random-init in the FP8 checkpoint layout, the prompt is 200
uniform random token ids, decoding is greedy with a fresh cache.

Two measurements are reported:
* ``value`` / ``ms_per_step``: K steps enqueued back to back, timed with CUDA events on the launching stream, maximum
  over ranks.
* ``e2e``: the same K steps through the engine's session loop: every step copies the step's input token from pinned
  host memory to the device and reads the produced token back before the next step is issued.

``--impl reference`` reports why the JAX/Pallas TPU reference cannot run on this machine.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_SINGLE_CHAT_TOK_S = 13.57
BASELINE_FOUR_CHAT_TOK_S = 5.12


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.samples: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx.append(float(s[2]))
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[4:8]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


class _SkipExtras(Exception):
    pass


def reference_arm() -> int:
    line = {
        "impl": "reference",
        "unavailable": "the reference is JAX 0.10.1 + Pallas/Mosaic TPU kernels on a 32-chip TPU v4 slice; jax, jaxlib and libtpu are not "
                       "installed and cannot be installed offline, and there is no TPU; compare with its published 13.57 tok/s",
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0: all 78 on 8 GPUs; on N < 8 GPUs round(78 * N / 8), the depth whose weights fill a GPU as the full model fills eight)")
    ap.add_argument("--chats", type=int, default=1, help="concurrent chats (lanes): 1 or 4")
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--prompt", type=int, default=200)
    ap.add_argument("--depth", type=int, default=0,
                    help="instead of a real prefill, make every chat this many tokens deep with a synthetic (random) cache: decode cost at depth")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra measurements after the timed region (time to first token, and four concurrent chats when --chats 1)")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--kv-layout", default="auto", choices=["auto", "striped", "replicated"],
                    help="latent cache: a replica per GPU (no attention exchange) or striped by position over the GPUs")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.runner.gpu_runner import build_runner

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if rank == 0:
        build()
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()

    layers = args.layers or (78 if world >= 8 else max(4, round(78 * world / 8)))
    geometry = glm53_geometry()
    if layers != geometry.num_layers:
        geometry = geometry.truncated(layers)
    t0 = time.perf_counter()
    runner = build_runner(geometry, world=world, rank=rank, device=device, seed=0, context_capacity=args.context, lanes=args.chats,
                          comm=args.comm, use_graphs=not args.no_graphs, prefill_chunk=1024, kv_layout=args.kv_layout)
    torch.cuda.synchronize()
    load_s = time.perf_counter() - t0

    gen = torch.Generator().manual_seed(1234)
    t0 = time.perf_counter()
    first = []
    for lane in range(args.chats):
        if args.depth:
            runner.synthetic_context(lane, args.depth - 97 * lane, seed=lane)
            first.append(-1)
            continue
        n = args.prompt if args.chats == 1 else (150, 200, 250, 300, 200, 200, 200, 200)[lane]
        prompt = torch.randint(0, geometry.vocab_size, (n,), generator=gen).tolist()
        first.append(runner.prefill(lane, prompt))
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    rec = runner.build_decode_program()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed: K steps back to back --------------------------------------------------------
    for _ in range(args.warmup):
        runner.decode_step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        runner.decode_step()
    stop.record()
    barrier()
    device_ms = start.elapsed_time(stop)

    # ---- end to end: session loop with the per-step host round trip ---------------------------------
    lanes = args.chats
    host_in = torch.zeros(lanes, dtype=torch.int32).pin_memory()
    host_out = torch.zeros(lanes, dtype=torch.int32).pin_memory()
    host_in.copy_(runner.state.tokens.cpu())
    from glm_tpu_b200.models.glm_moe_dsa.model import RING

    step0 = int(runner.state.step_counter.cpu()[0])
    for i in range(3):
        runner.state.tokens.copy_(host_in, non_blocking=True)
        runner.decode_step()
        host_out.copy_(runner.state.out_tokens[(step0 + i) % RING], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        host_in.copy_(torch.where(host_out >= 0, host_out, host_in))
    step0 += 3
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        runner.state.tokens.copy_(host_in, non_blocking=True)  # H2D of this step's input tokens (pinned)
        runner.decode_step()
        host_out.copy_(runner.state.out_tokens[(step0 + i) % RING], non_blocking=True)  # D2H of the step's result
        torch.cuda.current_stream().synchronize()
        host_in.copy_(torch.where(host_out >= 0, host_out, host_in))
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    e2e_wall_ms = (time.perf_counter() - wall0) * 1e3
    clocks = sampler.stop() if rank == 0 else None
    runner.peer.check_status()

    times = torch.tensor([device_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    device_ms, e2e_ms = float(times[0]), float(times[1])
    ms_per_step = device_ms / args.steps
    tok_s = args.chats * 1000.0 / ms_per_step
    e2e_tok_s = args.chats * 1000.0 / (e2e_ms / args.steps)

    # ---- the rest of the headline metric, outside the timed region: time to first token, four concurrent chats ----------
    extras = {}
    weights, kv_layout = runner.weights, runner.kv_layout
    try:
        if args.no_extras:
            raise _SkipExtras
        def timed_prefill(r, lane, n):
            prompt = torch.randint(0, geometry.vocab_size, (n,), generator=gen).tolist()
            barrier()
            w0 = time.perf_counter()
            r.prefill(lane, prompt)  # returns after the first token has reached the host
            torch.cuda.synchronize()
            ms = torch.tensor([(time.perf_counter() - w0) * 1e3], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms[0])

        ttft = {}
        for n in (args.prompt, 4096):
            if n + 8 < args.context:
                timed_prefill(runner, 0, n)  # first call at this length: allocations, tensor maps
                ttft[str(n)] = round(min(timed_prefill(runner, 0, n) for _ in range(2)), 2)
        extras["ttft_ms_by_prompt_tokens"] = ttft
        extras["ttft_note"] = "wall clock, token ids on the host -> first token on the host, max over ranks, best of 2 after a warm-up; the reference publishes 965 ms for 85 tokens"
        if args.chats == 1:
            from glm_tpu_b200.runner.gpu_runner import GpuModelRunner

            runner.close()
            runner = None
            torch.cuda.empty_cache()
            barrier()
            r4 = GpuModelRunner(weights, context_capacity=args.context, lanes=4, comm=args.comm, use_graphs=not args.no_graphs, prefill_chunk=1024,
                                kv_layout=args.kv_layout)
            for lane, n in enumerate((150, 200, 250, 300)):
                r4.prefill(lane, torch.randint(0, geometry.vocab_size, (n,), generator=gen).tolist())
            rec4 = r4.build_decode_program()
            for _ in range(args.warmup):
                r4.decode_step()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(args.steps):
                r4.decode_step()
            a1.record()
            barrier()
            r4.peer.check_status()
            ms4 = torch.tensor([a0.elapsed_time(a1)], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(ms4, op=dist.ReduceOp.MAX)
            step4 = float(ms4[0]) / args.steps
            extras["four_chats"] = {"tok_s_total": round(4000.0 / step4, 3), "tok_s_per_chat": round(1000.0 / step4, 3), "ms_per_step": round(step4, 4),
                                    "vs_baseline_per_chat": round(1000.0 / step4 / BASELINE_FOUR_CHAT_TOK_S, 3), "launches_per_step": rec4.launches,
                                    "timing": "CUDA events around the same number of steps, max over ranks"}
            runner = r4
    except _SkipExtras:
        pass
    except Exception as exc:  # the timed figures above stand on their own: an extra that fails is reported, not fatal
        extras["error"] = f"{type(exc).__name__}: {exc}"[:300]

    baseline = BASELINE_SINGLE_CHAT_TOK_S if args.chats == 1 else BASELINE_FOUR_CHAT_TOK_S * args.chats
    if rank == 0:
        line = {
            "metric": "decode tok/s/chat (1 and 4 chats, 32k ctx), TTFT, GLM-5.3 FP8 on 8xB200",
            "metric_detail": f"value = greedy decode tokens/s with {args.chats} chat(s) at a 32k-slot context; four-chat rate and time to first token are under 'extras'",
            "value": round(tok_s, 3),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": round(tok_s / baseline, 3),
            "dtype": "bf16 activations, fp8 e4m3 routed experts (block-scaled), fp32 accumulate",
            "data": "synthetic: random-init weights in the FP8 checkpoint layout, uniform random prompt ids",
            "config": {
                "model": f"GLM-5.3 architecture, {layers} of 78 layers" + ("" if layers == 78 else " (the full model needs 8 GPUs: depth cut to keep the per-GPU weight bytes of the 8-GPU run)"),
                "layers": layers,
                "layer_tokens_per_s": round(tok_s * layers, 1),
                "scaling_note": "per-GPU work is fixed as N grows (layers = 78 N / 8), so the job-level figure that should grow with N is layers x tokens/s",
                "global_batch": args.chats,
                "seq_len": args.context,
                "prompt_tokens": args.prompt if not args.depth else None,
                "context_depth": args.depth or args.prompt,
                "context_fill": "synthetic random cache rows (no prefill)" if args.depth else "real prefill of the prompt",
                "parallelism": f"tp{world}(heads,mlp)+ep{world}(experts)" if world > 1 else "single gpu",
                "comm": args.comm,
                "kv_layout": kv_layout,
                "decode_program": rec.kind,
                "l2": "each step streams more weight bytes than the 126 MB L2 (inputs larger than L2)",
                "per_chat_tok_s": round(tok_s / args.chats, 3),
            },
            "e2e": {
                "value": round(e2e_tok_s, 3),
                "unit": "tokens/s",
                "h2d_bytes_per_step": 4 * lanes,
                "d2h_bytes_per_step": 4 * lanes,
                "ms_per_step": round(e2e_ms / args.steps, 4),
                "wall_ms_per_step_rank0": round(e2e_wall_ms / args.steps, 4),
            },
            "gpu_launches": rec.launches * args.steps,
            "launches_per_step": rec.launches,
            "clocks": clocks,
            "load_seconds": round(load_s, 2),
            "prefill_seconds": round(prefill_s, 3),
            "resident_bytes_per_gpu": weights.bytes_resident,
            "first_tokens": first,
            "extras": extras,
        }
        print(json.dumps(line))
    if runner is not None:
        runner.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
