"""The per-GPU worker process: preflight, load, run queued / concurrent requests, resident loop.

One worker drives one GPU (``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` from the environment; the controller or
``torch.distributed.run`` starts them).  Every phase ends in an all-rank vote so that a rank that failed takes the
others down at the same point instead of stranding them.

    python -m glm_tpu_b200.worker.gpu_worker --run-dir DIR --request FILE [--keep-loaded] --model random:tiny ...

Phases: preflight (environment flag, run directory, request identity) -> runtime (process groups, vote channel) ->
load (weights: random init or a packed checkpoint) -> programs (decode program capture) -> warm-up (2 tokens, nothing
delivered) -> requests.  Rank 0 writes ``tokens.jsonl`` (one TokenEvent per line, flushed per token) and
``answer.txt``; every rank persists ``runner.rank<r>.json``.  With ``--keep-loaded`` the worker then serves resident
commands from stdin (one canonical JSON line per request; ``{"stop":true}`` ends the session).

Parity: reference ``glm_tpu/worker/tpu_worker.py:29-385`` (preflight, phases, run_queued, run_concurrent,
resident_loop, records).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

from glm_tpu_b200.engine import request as request_schema
from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.engine.llm_engine import LLMEngine
from glm_tpu_b200.engine.outputs import final_channel
from glm_tpu_b200.engine.request_session import LocalVote, fleet_vote
from glm_tpu_b200.utils.io_utils import persist_json


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="glm_tpu_b200.worker.gpu_worker")
    ap.add_argument("--run-dir", required=True)
    ap.add_argument("--request", help="prepared request or batch (JSON file); optional with --keep-loaded")
    ap.add_argument("--request-sha256", help="expected request_sha256 of --request")
    ap.add_argument("--keep-loaded", action="store_true")
    ap.add_argument("--model", default="random:tiny", help="random:<tiny|small|glm53>[:layers] or a packed checkpoint directory")
    ap.add_argument("--backend", default="gpu", choices=["gpu", "oracle"], help="'oracle' runs the CPU contract reference")
    ap.add_argument("--context", type=int, default=0, help="context capacity (0: the request's)")
    ap.add_argument("--lanes", type=int, default=1)
    ap.add_argument("--comm", default=None, choices=["fused", "nccl"], help="default: GLM_B200_COMM, else fused")
    ap.add_argument("--kv-layout", default="auto")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--site-json", help="the controller's resolved site (staged in the run directory)")
    ap.add_argument("--site-sha256", help="digest of --site-json as the controller computed it")
    ap.add_argument("--source-manifest", help="digest of every source file, taken by the controller")
    ap.add_argument("--source-manifest-sha256")
    ap.add_argument("--binding", help="topology binding: which physical GPU each rank uses")
    ap.add_argument("--binding-sha256")
    ap.add_argument("--preflight-only", action="store_true")
    ap.add_argument("--no-warmup", action="store_true")
    return ap.parse_args(argv)


# ------------------------------------------------------------------------------------------------ preflight
REPO = Path(__file__).resolve().parents[2]
SELF = Path(__file__).resolve().relative_to(REPO).as_posix()


def authenticate_launch(args) -> dict:
    """What binds this worker to its controller, checked before a device is opened: the staged site (digest given on the
    command line; its run root must be where the run directory is), the source manifest (every listed file re-hashed, this
    file among them) and the topology binding (self-digest, the command line's digest, the site's pin).  Returns
    ``{"site", "pins", "binding"}`` (None where nothing was staged: a launch without a site file pins nothing)."""
    from glm_tpu_b200.utils.io_utils import read_bounded

    out: dict = {"site": None, "pins": None, "binding": None}
    for flag, digest in (("site_json", "site_sha256"), ("source_manifest", "source_manifest_sha256"), ("binding", "binding_sha256")):
        if bool(getattr(args, flag)) != bool(getattr(args, digest)):
            raise SystemExit(f"--{flag.replace('_', '-')} and --{digest.replace('_', '-')} come together")
    if args.site_json:
        from glm_tpu_b200.config.site import SiteConfig

        site = SiteConfig.from_staged(Path(args.site_json), args.site_sha256)
        if Path(args.run_dir).resolve().parent != site.paths.run_root.resolve():
            raise SystemExit("the run directory is not under the staged site's run_root")
        out["site"], out["pins"] = site, site.checkpoint_pins
    if args.source_manifest:
        import hashlib

        from glm_tpu_b200.executor import source_manifest

        raw = read_bounded(Path(args.source_manifest), 4 << 20)
        if hashlib.sha256(raw).hexdigest() != args.source_manifest_sha256:
            raise SystemExit("the source manifest is not the controller's (digest differs)")
        source_manifest.verify(REPO, json.loads(raw), must_contain=SELF)
    if args.binding:
        from glm_tpu_b200.parallel import topology as topo

        binding = topo.load_topology_binding(Path(args.binding), args.binding_sha256)
        pinned = out["site"].topology_binding_sha256 if out["site"] is not None else ""
        if pinned and binding["binding_sha256"] != pinned:
            raise SystemExit("the topology binding is not the one the site pins")
        out["binding"] = binding
    elif out["site"] is not None and out["site"].topology_binding_sha256 and args.backend == "gpu":
        raise SystemExit("the site pins a topology binding but the controller staged none")
    return out


def preflight(args) -> dict:
    """Checks that need no device.  Returns the validated payload (or None)."""
    if os.environ.get(proto.WORKER_ENV_FLAG) != "1":
        raise SystemExit(f"{proto.WORKER_ENV_FLAG}=1 is required: workers are started by the controller")
    run_dir = Path(args.run_dir)
    if not run_dir.is_dir():
        raise SystemExit(f"run directory {run_dir} does not exist")
    args.launch = authenticate_launch(args)
    payload = None
    if args.request:
        raw = Path(args.request).read_bytes()
        payload = json.loads(raw)
        if args.request_sha256 and payload.get("request_sha256") != args.request_sha256:
            raise SystemExit("the staged request is not the one the controller prepared")
    elif not args.keep_loaded:
        raise SystemExit("--request is required unless the worker only serves resident commands")
    return payload


def resolve_model(spec: str):
    """``(geometry, source)``: source is ('random', seed-less) or ('checkpoint', Path)."""
    from glm_tpu_b200.config import model as mc

    if spec.startswith("random:"):
        parts = spec.split(":")
        base = {"tiny": mc.tiny_geometry, "small": mc.small_geometry, "glm53": mc.glm53_geometry}[parts[1]]()
        if len(parts) > 2:
            base = base.truncated(int(parts[2]))
        return base, ("random", None)
    path = Path(spec)
    from glm_tpu_b200.model_loader.sharded_state import loader

    return loader.read_geometry(path), ("checkpoint", path)


def profile_for(geometry, capacity: int, tokenizer=None) -> request_schema.RequestProfile:
    from glm_tpu_b200.config import model as mc

    if geometry.vocab_size == mc.glm53_geometry().vocab_size:
        return request_schema.GLM53_PROFILE
    caps = tuple(sorted({capacity}))
    return request_schema.RequestProfile.for_geometry(geometry, caps, concurrent_capacity=capacity)


# ------------------------------------------------------------------------------------------------ worker
class Worker:
    def __init__(self, args, payload):
        self.args, self.payload = args, payload
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        self.run_dir = Path(args.run_dir)
        self.record: dict = {"rank": self.rank, "world": self.world, "phases": {}, "requests": [], "programs": []}
        self.vote = LocalVote()
        self.gloo = None
        self.engine = None
        self.tokenizer = None
        self.launch = getattr(args, "launch", None) or {"site": None, "pins": None, "binding": None}

    def phase(self, name: str, fn):
        """Run ``fn``; whatever happens, all ranks vote on the outcome before anyone continues."""
        t0 = time.perf_counter()
        error = None
        result = None
        try:
            result = fn()
        except BaseException as exc:  # noqa: BLE001
            error = exc
        self.record["phases"][name] = time.perf_counter() - t0
        if not self.vote.all(error is None, f"phase:{name}"):
            self.record["failure_type"] = type(error).__name__ if error else "PeerFailure"
            self.persist()
            if error:
                raise error
            raise SystemExit(f"a peer failed in phase {name}")
        return result

    def init_runtime(self):
        if self.world > 1:
            import torch
            import torch.distributed as dist

            if self.args.backend == "gpu":
                torch.cuda.set_device(self.local_rank)
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
                self.gloo = dist.new_group(backend="gloo")
            else:
                dist.init_process_group("gloo")
                self.gloo = dist.group.WORLD
            # the ranks of one box vote through shared memory (a few microseconds a vote; the engine votes twice per token)
            self.vote = fleet_vote(self.gloo, self.rank, self.world, self.args.run_dir)
        self.check_bound_device()

    def check_bound_device(self, device_uuid=None) -> None:
        """With a topology binding, ``cuda:<local_rank>`` must be the GPU the binding gives this rank, and every rank must hold the
        same binding.  ``device_uuid`` is injectable for tests (default: what the CUDA runtime reports)."""
        binding = self.launch["binding"]
        digest = binding["binding_sha256"] if binding is not None else ""
        self.record["topology_binding_sha256"] = digest or None
        ok, why = True, ""
        if binding is not None and self.args.backend == "gpu":
            if binding["gpus"] != self.world:
                ok, why = False, f"the binding is for {binding['gpus']} GPUs, the fleet has {self.world} ranks"
            else:
                if device_uuid is None:
                    import torch

                    def device_uuid(index):
                        return "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                want, have = binding["ranks"][self.rank]["uuid"], device_uuid(self.local_rank)
                if have != want:
                    ok, why = False, f"rank {self.rank} sits on {have}, the binding says {want}"
        agreed = self.digest_consensus("binding:" + digest)
        if not self.vote.all(ok and agreed, "topology_binding"):
            raise SystemExit(why or "the ranks do not hold the same topology binding")
    def digest_consensus(self, digest: str) -> bool:
        if self.world == 1:
            return True
        import torch.distributed as dist

        gathered = [None] * self.world
        dist.all_gather_object(gathered, digest, group=self.gloo)
        return all(d == gathered[0] for d in gathered)

    def load(self):
        geometry, (kind, path) = resolve_model(self.args.model)
        capacity = self.args.context or (self.payload or {}).get("context_capacity") or request_schema.CAPACITY
        lanes = max(self.args.lanes, len(self.payload["requests"]) if self.payload and request_schema.is_concurrent(self.payload) else 1)
        if self.args.backend == "oracle":
            from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint
            from glm_tpu_b200.runner.oracle_runner import OracleRunner

            if kind != "random":
                from glm_tpu_b200.model_loader.sharded_state import loader

                checkpoint = loader.load_full_checkpoint(path)
            else:
                checkpoint = random_checkpoint(geometry, seed=self.args.seed)
            runner = OracleRunner(geometry, checkpoint, context_capacity=capacity, lanes=lanes)
        else:
            import torch

            from glm_tpu_b200.csrc.build import build
            from glm_tpu_b200.runner.gpu_runner import build_runner

            if self.rank == 0:
                build()
            self.vote.all(True, "library_built")
            device = torch.device("cuda", self.local_rank)
            checkpoint = None
            if kind == "checkpoint":
                from glm_tpu_b200.model_loader.sharded_state import loader

                # the site's pins travel with the load: another packed checkpoint than the pinned one is refused here
                checkpoint = loader.load_rank_checkpoint(path, self.rank, self.world, pins=self.launch["pins"], device=device)
                self.record["checkpoint_pins"] = {k: v for k, v in (self.launch["pins"] or {}).items() if v}
            elif geometry.num_layers <= 8 and geometry.hidden_size <= 1024:
                from glm_tpu_b200.models.glm_moe_dsa.weights import random_checkpoint

                checkpoint = random_checkpoint(geometry, seed=self.args.seed)  # fixtures: the same bits as the oracle
            stripe = 64 if capacity % (64 * self.world) == 0 else max(1, capacity // (8 * self.world))
            runner = build_runner(geometry, world=self.world, rank=self.rank, device=device, checkpoint=checkpoint, seed=self.args.seed,
                                  context_capacity=capacity, lanes=lanes, comm=self.args.comm, kv_layout=self.args.kv_layout,
                                  stripe=stripe, prefill_chunk=min(2048 if capacity <= 65536 else 1024, capacity))  # rows per prefill pass: weights are re-streamed per pass
        from glm_tpu_b200.tokenizer import load_tokenizer

        self.tokenizer = load_tokenizer(path if kind == "checkpoint" else None, vocab_size=geometry.vocab_size, eos_ids=geometry.eos_ids)
        self.profile = profile_for(geometry, capacity)
        self.engine = LLMEngine(runner, vote=self.vote, profile=self.profile, digest_consensus=self.digest_consensus)
        self.record["geometry_hash"] = geometry.geometry_hash
        from glm_tpu_b200.config.parallel import ParallelLayout

        model = getattr(runner, "model", None)  # which tensor is split how: must agree on every rank
        layout_hash = (model.layout if model is not None else ParallelLayout(geometry, self.world, self.rank)).layout_hash
        self.record["layout_hash"] = layout_hash
        self.vote.all(self.digest_consensus(layout_hash), "layout_agreed")
        self.record["context_capacity"] = capacity
        self.record["kv_layout"] = getattr(runner, "kv_layout", None)
        self.record["memory_admission"] = getattr(getattr(runner, "report", None), "memory", None)
        return runner

    def build_programs(self, runner):
        rec = runner.build_decode_program()
        self.record["programs"].append({"name": rec.name, "kind": rec.kind, "rows": rec.rows, "launches": rec.launches})

    def warmup(self):
        """Two tokens through the whole path with nothing delivered (first-use costs are paid here)."""
        ids = [1, 2, 3]
        req = request_schema.from_token_ids(ids, request_id="warmup", max_new_tokens=2,
                                            context_capacity=self.record["context_capacity"], profile=self.profile)
        self.engine.generate(req, None)

    # -------------------------------------------------------------------------------------------- requests
    def run_payload(self, payload: dict, out_dir: Path) -> list[dict]:
        out_dir.mkdir(parents=True, exist_ok=True)
        stream = (out_dir / proto.TOKENS_FILE).open("a", encoding="utf-8") if self.rank == 0 else None

        def sink(event):
            if stream is not None:
                stream.write(json.dumps(event.wire(), sort_keys=True, separators=(",", ":")) + "\n")
                stream.flush()

        try:
            reports = self.engine.run_payload(payload, sink)
        finally:
            if stream is not None:
                stream.close()
        if self.rank == 0:
            self.write_answers(payload, out_dir)
        self.record["requests"] += reports
        # the record of this sequence lists its own requests only; the cumulative one stays in the run directory
        persist_json(out_dir / proto.runner_file(self.rank), dict(self.record, requests=reports))
        return reports

    def write_answers(self, payload: dict, out_dir: Path) -> None:
        by_request: dict = {}
        for line in (out_dir / proto.TOKENS_FILE).read_text(encoding="utf-8").splitlines():
            ev = json.loads(line)
            by_request.setdefault(ev["request_id"], []).append(ev["token_id"])
        answers = {}
        for rid, ids in by_request.items():
            text = self.tokenizer.decode([t for t in ids if t not in self.profile.eos_ids])
            thinking, answer = final_channel("<think>" + text)
            answers[rid] = {"thinking": thinking, "answer": answer, "output_tokens": len(ids)}
        (out_dir / proto.ANSWER_FILE).write_text(json.dumps(answers, ensure_ascii=False, indent=1), encoding="utf-8")

    def persist(self):
        persist_json(self.run_dir / proto.runner_file(self.rank), self.record)

    def resident_loop(self, sequence: int) -> None:
        """Serve ``{"request": ..., "sequence": n}`` lines from stdin until ``{"stop":true}`` or EOF."""
        while True:
            if self.rank == 0:
                persist_json(self.run_dir / proto.READY_FILE, {"sequence": sequence})
            line = sys.stdin.readline()
            if not line:
                return
            command = json.loads(line)
            if command.get("stop"):
                return
            sequence = int(command["sequence"])
            request_schema.validate_payload(command["request"], self.profile)
            self.run_payload(command["request"], proto.result_dir(self.run_dir, sequence))


def main(argv=None) -> int:
    args = parse_args(argv)
    payload = preflight(args)
    if args.preflight_only:
        print(json.dumps({"preflight": "ok", "request_sha256": (payload or {}).get("request_sha256")}))
        return 0
    worker = Worker(args, payload)
    worker.init_runtime()
    (worker.run_dir / proto.worker_started_file(worker.rank)).write_text(json.dumps({"pid": os.getpid(), "rank": worker.rank}))
    runner = worker.phase("load", worker.load)
    if payload is not None:
        worker.phase("validate_request", lambda: request_schema.validate_payload(payload, worker.profile))
    worker.phase("programs", lambda: worker.build_programs(runner))
    if not args.no_warmup:
        worker.phase("warmup", worker.warmup)
    try:
        if payload is not None:
            worker.phase("requests", lambda: worker.run_payload(payload, worker.run_dir))
        worker.persist()
        if args.keep_loaded:
            worker.resident_loop(0)
    finally:
        worker.persist()
        if hasattr(runner, "close"):
            runner.close()
        if worker.world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
