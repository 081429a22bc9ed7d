"""Headline benchmark: greedy decode rate of one chat at a 32,768-slot context, GLM-5.3 FP8 architecture.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 64 --warmup 8

A *step* is one decode step (one new token for every live chat).  With 8 GPUs the model is the full 78-layer GLM-5.3;
with 1, 2 or 4 GPUs it is the 12-layer truncation of the same architecture (the full model does not fit), the same 12
layers at every such N, so those runs are one configuration under strong scaling.  The JSON line states the layer count
and gives ``vs_baseline`` only for the full model (a 12-layer rate is not comparable with the published 78-layer one); the
8-GPU run also reports the 12-layer rate under ``extras`` so that the curve over 1, 2, 4 and 8 GPUs exists on one
configuration.  Weights are random-init in the FP8 checkpoint layout, the prompt is 200 uniform random token ids, decoding
is greedy with a fresh cache.

Two measurements:

* ``value`` / ``ms_per_step``: ``--steps`` decode steps enqueued back to back, timed with CUDA events on the launching
  stream between barriers, maximum over ranks; repeated ``--repeats`` times, the median block is reported and the spread
  beside it.
* ``e2e``: the same model through the engine's public call, ``LLMEngine.generate`` (``generate_concurrent`` for several
  chats): a fresh request whose prompt is copied from pinned host memory, then per token the feed of the committed token
  (host to device), the decode step, the read of the produced token and of the status word (device to host), two all-rank
  votes over gloo and the token line written and flushed by rank 0.  The rate is the engine's own report (decode tokens /
  decode wall seconds, slowest rank), which is how the published 13.57 tokens/s is defined.

``--impl reference`` reports why the JAX/Pallas TPU reference cannot run on this machine.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
from pathlib import Path
import tempfile
import threading
import time

BASELINE_SINGLE_CHAT_TOK_S = 13.57
BASELINE_FOUR_CHAT_TOK_S = 5.12
FULL_LAYERS = 78
SMALL_BOX_LAYERS = 12


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


def reference_arm() -> int:
    line = {
        "impl": "reference",
        "unavailable": "the reference is JAX 0.10.1 + Pallas/Mosaic TPU kernels on a 32-chip TPU v4 slice; jax, jaxlib and libtpu are not "
                       "installed and cannot be installed offline, and there is no TPU; compare with its published 13.57 tok/s",
    }
    if int(os.environ.get("RANK", "0")) == 0:  # one line however many ranks the launcher started
        print(json.dumps(line))
    return 0


class Bench:
    """One process of the benchmark (one GPU): the distributed plumbing and the two timing methods."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.gloo = None
        self._vote_dir, self._votes = None, 0
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # the version banner would share stdout with the JSON line
        if self.world > 1:
            from datetime import timedelta

            # bounded waits everywhere: a rank that fails must cost its peers minutes at most, never the default half hour
            # the library announces its version on file descriptor 1 when the first communicator comes up: that line belongs on
            # stderr, stdout carries the one JSON line
            sys.stdout.flush()
            saved_stdout = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group("nccl", device_id=self.device, timeout=timedelta(seconds=300))
                self.gloo = dist.new_group(backend="gloo", timeout=timedelta(seconds=120))  # host barriers, the vote's rendezvous
                dist.barrier()
                torch.cuda.synchronize()
            finally:
                os.dup2(saved_stdout, 1)
                os.close(saved_stdout)
        self.gen = torch.Generator().manual_seed(1234)

    def barrier(self):
        """Device idle on every rank, then a host barrier (gloo: a peer that never arrives raises here after two minutes)."""
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier(group=self.gloo)

    def max_over_ranks(self, values: list[float]) -> list[float]:
        t = self.torch.tensor(values, dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def prompt(self, n: int, vocab: int) -> list[int]:
        return self.torch.randint(0, vocab, (n,), generator=self.gen).tolist()

    # ------------------------------------------------------------------ device-timed blocks
    def timed_blocks(self, runner, steps: int, warmup: int, repeats: int) -> list[float]:
        """Milliseconds of ``repeats`` blocks of ``steps`` decode steps each (CUDA events, barrier + synchronize on both sides,
        maximum over ranks)."""
        torch = self.torch
        for _ in range(warmup):
            runner.decode_step()
        out = []
        for _ in range(repeats):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            start.record()
            for _ in range(steps):
                runner.decode_step()
            stop.record()
            self.barrier()
            out.append(start.elapsed_time(stop))
        runner.peer.check_status()
        return self.max_over_ranks(out)

    # ------------------------------------------------------------------ through the engine
    def engine_run(self, runner, geometry, prompts: list[list[int]], new_tokens: int, capacity: int) -> dict:
        """``LLMEngine.generate`` / ``generate_concurrent`` with the fleet vote (shared memory between the ranks of the box, as the
        workers use it) and a flushed token file on rank 0."""
        from glm_tpu_b200.engine import request as rq
        from glm_tpu_b200.engine.llm_engine import LLMEngine
        from glm_tpu_b200.engine.request_session import LocalVote, fleet_vote
        from glm_tpu_b200.worker.gpu_worker import profile_for

        profile = profile_for(geometry, capacity)
        if self.world > 1:
            if self._vote_dir is None:
                made = [tempfile.mkdtemp(prefix="glm_b200_bench_vote_") if self.rank == 0 else None]
                self.dist.broadcast_object_list(made, src=0, group=self.gloo)
                self._vote_dir = made[0]
            self._votes += 1
            vote = fleet_vote(self.gloo, self.rank, self.world, self._vote_dir, name=f"vote{self._votes}.shm", timeout=60.0)
        else:
            vote = LocalVote()
        vote_seconds = [0.0]
        inner = vote.all

        def timed_vote(ok, point):
            t0 = time.perf_counter()
            try:
                return inner(ok, point)
            finally:
                vote_seconds[0] += time.perf_counter() - t0

        vote.all = timed_vote

        def consensus(digest: str) -> bool:
            if self.world == 1:
                return True
            gathered = [None] * self.world
            self.dist.all_gather_object(gathered, digest, group=self.gloo)
            return all(d == gathered[0] for d in gathered)

        engine = LLMEngine(runner, vote=vote, profile=profile, digest_consensus=consensus)
        requests = [rq.from_token_ids(p, request_id=f"bench-{i}", max_new_tokens=new_tokens + 1, context_capacity=capacity, profile=profile)
                    for i, p in enumerate(prompts)]
        sink_file = tempfile.NamedTemporaryFile("w", suffix=".jsonl", delete=False) if self.rank == 0 else None

        def sink(event):
            if sink_file is not None:
                sink_file.write(json.dumps(event.wire(), sort_keys=True, separators=(",", ":")) + "\n")
                sink_file.flush()

        self.barrier()
        vote_seconds[0] = 0.0
        if len(requests) == 1:
            reports = [engine.generate(requests[0], sink)]
        else:
            reports = engine.generate_concurrent(rq.batch(requests, concurrent=True, profile=profile), sink)
        self.barrier()
        if sink_file is not None:
            sink_file.close()
            os.unlink(sink_file.name)
        timed = sum(r["timed_decode_tokens"] for r in reports)
        wall = max(r["decode_wall_seconds"] for r in reports)
        wall, votes, prefill = self.max_over_ranks([wall, vote_seconds[0], max(r["prefill_seconds"] for r in reports)])
        lanes = len(requests)
        return {
            "value": round(timed / wall, 3) if wall > 0 else None,
            "unit": "tokens/s",
            "api": "LLMEngine.generate" if lanes == 1 else "LLMEngine.generate_concurrent",
            "timed_decode_tokens": timed,
            "decode_wall_seconds": round(wall, 4),
            "ms_per_step": round(wall * 1e3 / max(timed // lanes, 1), 4),
            "h2d_bytes_per_step": runner.fed_bytes_per_step,
            "d2h_bytes_per_step": 4 * runner.lanes + 4,
            "prompt_h2d_bytes": sum(4 * len(p) for p in prompts),
            "prefill_seconds": round(prefill, 4),
            "vote_seconds": round(votes, 4),
            "vote_share_of_decode": round(votes / wall, 4) if wall > 0 else None,
            "finish_reasons": [r["finish_reason"] for r in reports],
            "per_token": "feed of the committed token (pinned host -> device), decode step (CUDA graph), token + status read (device -> host), "
                         "validity vote, commit, token line written and flushed on rank 0, delivery vote",
        }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5, help="timed blocks of --steps steps; the median block is the headline, min and max are reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0: all 78 on 8 GPUs, the 12-layer truncation below)")
    ap.add_argument("--chats", type=int, default=1, help="concurrent chats (lanes): 1 or 4")
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--prompt", type=int, default=200)
    ap.add_argument("--tokens", type=int, default=0, help="decode tokens of the engine run (0: --steps x --repeats; 2048 is the full published decode length)")
    ap.add_argument("--depth", type=int, default=0,
                    help="instead of a real prefill, make every chat this many tokens deep with a synthetic (random) cache: decode cost at depth")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra measurements after the timed region (time to first token, four concurrent chats, depth 30,000, 12 layers)")
    ap.add_argument("--prefill-chunk", type=int, default=2048, help="rows per prefill pass (what the serving worker uses at a 32k context)")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--kv-layout", default="auto", choices=["auto", "striped", "replicated"],
                    help="latent cache: a replica per GPU (no attention exchange) or striped by position over the GPUs")
    ap.add_argument("--decode-path", default="auto", choices=["auto", "kernels", "phases", "mega"])
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)

    b = Bench(args)
    torch = b.torch
    from glm_tpu_b200.config.model import glm53_geometry
    from glm_tpu_b200.csrc.build import build
    from glm_tpu_b200.runner.gpu_runner import GpuModelRunner, build_runner

    if b.rank == 0:
        build()
    b.barrier()
    layers = args.layers or (FULL_LAYERS if b.world >= 8 else SMALL_BOX_LAYERS)
    full = glm53_geometry()
    geometry = full if layers == full.num_layers else full.truncated(layers)
    common = dict(context_capacity=args.context, comm=args.comm, use_graphs=not args.no_graphs, prefill_chunk=args.prefill_chunk, kv_layout=args.kv_layout,
                  decode_path=args.decode_path)
    t0 = time.perf_counter()
    runner = build_runner(geometry, world=b.world, rank=b.rank, device=b.device, seed=0, lanes=args.chats, **common)
    torch.cuda.synchronize()
    load_s = time.perf_counter() - t0

    def fill(r, lanes: int, depth: int) -> tuple[list, float]:
        """Give every lane its context: a real prefill of a random prompt, or (``depth``) a synthetic cache of that depth."""
        t = time.perf_counter()
        first = []
        for lane in range(lanes):
            if depth:
                r.synthetic_context(lane, depth - 97 * lane, seed=lane)
                first.append(-1)
            else:
                n = args.prompt if lanes == 1 else (150, 200, 250, 300, 200, 200, 200, 200)[lane]
                first.append(r.prefill(lane, b.prompt(n, geometry.vocab_size)))
        torch.cuda.synchronize()
        return first, time.perf_counter() - t

    first, prefill_s = fill(runner, args.chats, args.depth)
    rec = runner.build_decode_program()

    # ---- device-timed: blocks of K steps back to back ------------------------------------------------
    sampler = ClockSampler(b.local_rank)
    if b.rank == 0:
        sampler.start()
    blocks = b.timed_blocks(runner, args.steps, args.warmup, args.repeats)
    device_ms = statistics.median(blocks)
    ms_per_step = device_ms / args.steps
    tok_s = args.chats * 1000.0 / ms_per_step

    # ---- end to end: the engine's public call ---------------------------------------------------------
    incomplete = False
    new_tokens = args.tokens or args.steps * args.repeats
    prompts = [b.prompt(args.prompt if args.chats == 1 else (150, 200, 250, 300, 200, 200, 200, 200)[i], geometry.vocab_size) for i in range(args.chats)]
    try:
        e2e = b.engine_run(runner, geometry, prompts, new_tokens, args.context)
    except Exception as exc:  # the device-timed figure stands, but the line says that it is not the whole story
        e2e, incomplete = {"value": None, "error": f"{type(exc).__name__}: {exc}"[:300]}, True
    clocks = sampler.stop() if b.rank == 0 else None

    # ---- the rest of the published metrics, outside the timed regions -----------------------------------
    extras: dict = {}
    r4 = None
    weights, kv_layout = runner.weights, runner.kv_layout
    layout, fallbacks = runner.model.layout, runner.model.fallbacks  # the line below names them even if an extra loses the runner
    if not args.no_extras and not incomplete:
        try:
            def timed_prefill(r, lane, n):
                prompt = b.prompt(n, geometry.vocab_size)
                b.barrier()
                w0 = time.perf_counter()
                r.prefill(lane, prompt)  # returns after the first token has reached the host
                torch.cuda.synchronize()
                return b.max_over_ranks([(time.perf_counter() - w0) * 1e3])[0]

            ttft = {}
            for n in (args.prompt, 4096, 16384):
                if n + 8 < args.context:
                    timed_prefill(runner, 0, n)  # first call at this length: allocations, tensor maps
                    ttft[str(n)] = round(min(timed_prefill(runner, 0, n) for _ in range(2)), 2)
            extras["ttft_ms_by_prompt_tokens"] = ttft
            extras["ttft_note"] = (f"wall clock, token ids on the host -> first token on the host, chunks of {args.prefill_chunk} rows, max over ranks, best of 2 after a warm-up; "
                                   "the reference publishes 965 ms for 85 tokens")
            if args.chats == 1 and not args.depth:
                # the same chat 30,000 tokens deep: what a decode step costs late in a long answer
                runner.synthetic_context(0, 30000, seed=0)
                deep = b.timed_blocks(runner, args.steps, 3, min(args.repeats, 3))
                extras["depth_30000"] = {"tok_s": round(1000.0 * args.steps / statistics.median(deep), 3),
                                         "ms_per_step": round(statistics.median(deep) / args.steps, 4), "context_fill": "synthetic random cache rows"}
            if args.chats == 1:
                runner.close()
                runner = None
                torch.cuda.empty_cache()
                b.barrier()
                r4 = GpuModelRunner(weights, lanes=4, **common)
                fill(r4, 4, 0)
                rec4 = r4.build_decode_program()
                blocks4 = b.timed_blocks(r4, args.steps, args.warmup, min(args.repeats, 3))
                step4 = statistics.median(blocks4) / args.steps
                four = {"tok_s_total": round(4000.0 / step4, 3), "tok_s_per_chat": round(1000.0 / step4, 3), "ms_per_step": round(step4, 4),
                        "launches_per_step": rec4.launches, "timing": "CUDA events around the same number of steps, max over ranks, median block"}
                if layers == FULL_LAYERS:
                    four["vs_baseline_per_chat"] = round(1000.0 / step4 / BASELINE_FOUR_CHAT_TOK_S, 3)
                prompts4 = [b.prompt(n, geometry.vocab_size) for n in (150, 200, 250, 300)]
                four["e2e"] = b.engine_run(r4, geometry, prompts4, min(new_tokens, 256), args.context)
                extras["four_chats"] = four
                runner = r4
            if layers == FULL_LAYERS and b.world >= 8:
                # the 12-layer truncation on this box too: the configuration the 1-, 2- and 4-GPU runs use
                runner.close()
                runner = r4 = weights = None  # noqa: F841 - drop the full model before the small one is built
                torch.cuda.empty_cache()
                b.barrier()
                small = build_runner(full.truncated(SMALL_BOX_LAYERS), world=b.world, rank=b.rank, device=b.device, seed=0, lanes=1, **common)
                small.prefill(0, b.prompt(args.prompt, full.vocab_size))
                small.build_decode_program()
                blocks12 = b.timed_blocks(small, args.steps, args.warmup, min(args.repeats, 3))
                extras["layers12"] = {"tok_s": round(1000.0 * args.steps / statistics.median(blocks12), 3),
                                      "ms_per_step": round(statistics.median(blocks12) / args.steps, 4), "layers": SMALL_BOX_LAYERS}
                runner = small
        except Exception as exc:
            import traceback

            where = traceback.extract_tb(exc.__traceback__)[-1]
            extras["error"] = f"{type(exc).__name__}: {exc}"[:300] + f" ({Path(where.filename).name}:{where.lineno})"
            print(f"[bench rank {b.rank}] extras failed: {extras['error']}", file=sys.stderr, flush=True)
            incomplete = True

    baseline = BASELINE_SINGLE_CHAT_TOK_S if args.chats == 1 else BASELINE_FOUR_CHAT_TOK_S * args.chats
    comparable = layers == FULL_LAYERS and args.context == 32768 and args.chats in (1, 4)
    if b.rank == 0:
        line = {
            "metric": "decode tok/s/chat (1 and 4 chats, 32k ctx), TTFT, GLM-5.3 FP8 on 8xB200",
            "metric_detail": f"value = greedy decode tokens/s with {args.chats} chat(s) at a 32k-slot context; four-chat rate, time to first token and "
                             "the rate at depth 30,000 are under 'extras'",
            "value": round(tok_s, 3),
            "unit": "tokens/s",
            "n_gpus": b.world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": round(tok_s / baseline, 3) if comparable else None,
            "dtype": "bf16 activations, fp8 e4m3 routed experts (block-scaled), fp32 accumulate",
            "data": "synthetic: random-init weights in the FP8 checkpoint layout, uniform random prompt ids",
            "repeats": {"blocks": args.repeats, "ms_per_step_min": round(min(blocks) / args.steps, 4), "ms_per_step_median": round(ms_per_step, 4),
                        "ms_per_step_max": round(max(blocks) / args.steps, 4)},
            "config": {
                "model": f"GLM-5.3 architecture, {layers} of {FULL_LAYERS} layers"
                         + ("" if layers == FULL_LAYERS else " (the 12-layer truncation used on 1, 2 and 4 GPUs: the full model needs 8)"),
                "layers": layers,
                "scaling_note": "1, 2 and 4 GPUs run the same 12 layers (strong scaling); 8 GPUs run all 78 and report the 12-layer rate under extras.layers12",
                "global_batch": args.chats,
                "seq_len": args.context,
                "prompt_tokens": args.prompt if not args.depth else None,
                "context_depth": args.depth or args.prompt,
                "context_fill": "synthetic random cache rows (no prefill)" if args.depth else "real prefill of the prompt",
                "parallelism": (f"tp{b.world}(heads, mlp, shared expert" + (", routed experts by column)" if layout.sliced
                                else f")+ep{b.world}(routed experts)")) if b.world > 1 else "single gpu",
                "expert_split": layout.expert_split,
                "all_reduce": ("(value, sequence) pairs" if os.environ.get("GLM_B200_AR", "pairs") != "flags" else "values + fence + flag") if b.world > 1 else "none",
                "fallbacks": dict(fallbacks),
                "comm": args.comm,
                "kv_layout": kv_layout,
                "decode_program": rec.kind,
                "decode_path": rec.name,
                "l2": "each step streams more weight bytes than the 126 MB L2 (inputs larger than L2)",
                "per_chat_tok_s": round(tok_s / args.chats, 3),
            },
            "e2e": e2e,
            "gpu_launches": rec.launches * args.steps,
            "launches_per_step": rec.launches,
            "clocks": clocks,
            "load_seconds": round(load_s, 2),
            "prefill_seconds": round(prefill_s, 3),
            "first_tokens": first,
            "extras": extras,
        }
        if incomplete:
            line["incomplete"] = True
        print(json.dumps(line))
    if runner is not None:
        runner.close()
    if b.world > 1:
        try:
            b.barrier()
        except Exception:  # noqa: BLE001 - a peer that failed earlier must not keep this rank from finishing
            pass
        b.dist.destroy_process_group()
    return 0  # an incomplete run says so in its line ('incomplete': true); the device-timed figure above still stands


if __name__ == "__main__":
    sys.exit(main())
