"""The controller: stages a run, starts one worker per GPU, supervises them, serves a resident session and collects.

    python -m glm_tpu_b200.executor.multiproc_executor --request prepared.json --gpus 8 --model random:glm53 \
        [--keep-loaded] [--wall-seconds N] [--print-answers]

One-shot: stage the request, start the workers, wait for them (exit codes + wall deadline), summarize.  Resident
(``--keep-loaded``): after the first request the workers stay loaded; the controller polls the run directory --
``resident-ready.json`` says which sequence is done, ``inbox/NNNN.json`` is the next request (validated, then written
as one line to every worker's stdin), ``inbox/stop.json`` ends the session.  A run is good only if every rank's record
agrees on the request, the token digests and the program kinds.

There are no retries: a failed worker ends the run, the remaining workers are terminated (only process groups this
controller started), and ``controller_terminal.json`` records what happened.

Parity: reference ``glm_tpu/executor/multihost_executor.py:77-504`` (main, resident_controller, supervision, summarize).
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

from glm_tpu_b200.engine import request as request_schema
from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.executor import fleet as fleet_mod
from glm_tpu_b200.executor import jobs, staging
from glm_tpu_b200.utils.io_utils import persist_json, read_bounded

REPO = Path(__file__).resolve().parents[2]


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="glm_tpu_b200.executor.multiproc_executor")
    ap.add_argument("--request", help="prepared request or batch (JSON file)")
    ap.add_argument("--run-root", default=None)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--model", default="random:tiny")
    ap.add_argument("--backend", default="gpu", choices=["gpu", "oracle"])
    ap.add_argument("--context", type=int, default=0)
    ap.add_argument("--lanes", type=int, default=1)
    ap.add_argument("--comm", default=None, choices=["fused", "nccl"], help="default: GLM_B200_COMM, else fused")
    ap.add_argument("--kv-layout", default="auto")
    ap.add_argument("--keep-loaded", action="store_true")
    ap.add_argument("--wall-seconds", type=float, default=3600.0)
    ap.add_argument("--print-answers", action="store_true")
    ap.add_argument("--policy", default="record", choices=["record", "strict"])
    ap.add_argument("--master-port", type=int, default=29577)
    ap.add_argument("--poll-seconds", type=float, default=0.5)
    ap.add_argument("--site", default=None, help="site file whose pins (checkpoint manifest, topology binding, launch rules) bind this launch")
    ap.add_argument("--binding", default=None, help="topology binding file (default: <state_root>/topology_binding.json when the site pins one)")
    return ap.parse_args(argv)


def stage_site(run_dir: Path, site) -> list[str]:
    """Write the resolved site for the workers; returns the worker arguments that name it and its digest."""
    from glm_tpu_b200.utils.io_utils import create_private_exclusive

    path = run_dir / "site.json"
    create_private_exclusive(path, site.resolved_json())
    return ["--site-json", str(path), "--site-sha256", site.sha256]


def stage_source_manifest(run_dir: Path, repo: Path) -> list[str]:
    from glm_tpu_b200.executor import source_manifest
    from glm_tpu_b200.utils.io_utils import create_private_exclusive

    manifest = source_manifest.build(repo)
    path = run_dir / source_manifest.MANIFEST_FILE
    create_private_exclusive(path, source_manifest.to_bytes(manifest))
    return ["--source-manifest", str(path), "--source-manifest-sha256", source_manifest.digest(manifest)]


def stage_binding(run_dir: Path, site, binding_path: Path | None, gpus: int, nvml=None) -> tuple[list[str], dict]:
    """Authenticate the topology binding the site pins against the live box and hand it to the workers.

    Returns ``(worker arguments, extra environment)``: the environment makes ``cuda:<local_rank>`` the bound GPU in every worker
    (``CUDA_VISIBLE_DEVICES`` = the bound UUIDs in rank order).  Without a pin nothing is staged."""
    pin = site.topology_binding_sha256 if site is not None else ""
    if not pin and binding_path is None:
        return [], {}
    from glm_tpu_b200.exceptions import ConfigValidationError
    from glm_tpu_b200.parallel import topology as topo
    from glm_tpu_b200.utils.io_utils import create_private_exclusive
    from glm_tpu_b200.utils.json_utils import canonical_wire_bytes

    if binding_path is None:
        if site.paths.state_root is None:
            raise ConfigValidationError("[topology] binding_sha256 is set but neither --binding nor [paths] state_root says where the binding is")
        binding_path = site.paths.state_root / "topology_binding.json"
    binding = topo.load_topology_binding(binding_path, pin)
    if binding["gpus"] != gpus:
        raise ConfigValidationError(f"the topology binding is for {binding['gpus']} GPUs, the launch for {gpus}")
    try:
        live = topo.discover_topology(nvml)
    except ImportError as exc:
        raise ConfigValidationError("a pinned topology binding needs NVML (pynvml) to authenticate the live GPUs") from exc
    topo.validate_live(binding, live)
    staged = run_dir / "topology_binding.json"
    create_private_exclusive(staged, canonical_wire_bytes(binding) + b"\n")
    return ["--binding", str(staged), "--binding-sha256", binding["binding_sha256"]], {"CUDA_VISIBLE_DEVICES": topo.visible_devices(binding)}


def default_run_root() -> Path:
    from glm_tpu_b200 import envs

    return envs.GLM_B200_RUN_ROOT or Path.home() / ".cache" / "glm-b200" / "runs"


def summarize(run_dir: Path, world: int, sequence: int = 0) -> dict:
    """Do all ranks agree?  Same requests, same token digests, same program kinds."""
    out_dir = proto.result_dir(run_dir, sequence)
    records, missing = [], []
    for rank in range(world):
        path = out_dir / proto.runner_file(rank)
        if not path.exists():
            path = run_dir / proto.runner_file(rank)
        try:
            record = json.loads(path.read_text()) if path.exists() else None
        except (OSError, ValueError):
            record = None  # a record that cannot be read counts like one that was never written
        if isinstance(record, dict):
            records.append(record)
        else:
            missing.append(rank)
    digests = [[(r["request_id"], r["token_sha256"]) for r in rec.get("requests", [])] for rec in records]
    programs = [[(p["name"], p["kind"]) for p in rec.get("programs", [])] for rec in records]
    agree = not missing and bool(records) and all(d == digests[0] for d in digests) and all(p == programs[0] for p in programs)
    failures = [rec.get("failure_type") for rec in records if rec.get("failure_type")]
    reports = records[0].get("requests", []) if records else []
    return {
        "ranks": len(records),
        "missing_ranks": missing,
        "agree": bool(agree and not failures),
        "failures": failures,
        "requests": [
            {"request_id": r["request_id"], "emitted": r["emitted"], "finish_reason": r["finish_reason"],
             "decode_tokens_per_second": min((rec["requests"][i]["decode_tokens_per_second"] or 0.0) for rec in records) or None,
             "prefill_seconds": max(rec["requests"][i]["prefill_seconds"] for rec in records), "token_sha256": r["token_sha256"]}
            for i, r in enumerate(reports)
        ] if agree else [],
    }


def resident_controller(fl: fleet_mod.Fleet, run_dir: Path, world: int, profile_check, deadline: float | None, poll: float, *,
                        initial: bool = False, print_answers: bool = False, wall_seconds: float | None = None) -> dict:
    """Feed ``inbox/NNNN.json`` requests to the loaded workers until ``inbox/stop.json`` or a failure.

    ``initial``: the session was started with a request (sequence 0); its result is reported as soon as the workers are ready
    for the next one, not only when the session ends.

    ``deadline`` bounds the start-up together with the first request.  With ``wall_seconds`` a loaded, idle session has no
    deadline at all (it waits for its inbox as long as it lives) and every later request gets ``wall_seconds`` of its own from
    the moment it is handed to the workers; without it ``deadline`` bounds the whole loop."""
    inbox = run_dir / proto.INBOX_DIR
    served, sequence = [], 0
    reported_initial = not initial
    while deadline is None or time.monotonic() < deadline:
        codes = fl.poll()
        if any(c is not None for c in codes):
            return {"stopped": "worker_exit", "exit_codes": codes, "served": served}
        ready = run_dir / proto.READY_FILE
        ready_seq = json.loads(ready.read_text()).get("sequence", -1) if ready.exists() else -1
        if ready_seq == sequence:
            if wall_seconds is not None:
                deadline = None  # idle: nothing is running that could overrun
            if not reported_initial:
                reported_initial = True
                if print_answers and (run_dir / proto.ANSWER_FILE).exists():
                    print((run_dir / proto.ANSWER_FILE).read_text(), flush=True)
                print(proto.STDOUT_RESIDENT_RESULT + json.dumps({"sequence": 0, **summarize(run_dir, world)}), flush=True)
            if sequence > 0 and sequence not in served:
                summary = summarize(run_dir, world, sequence)
                persist_json(proto.result_dir(run_dir, sequence) / proto.MEASUREMENT_FILE, summary)
                print(proto.STDOUT_RESIDENT_RESULT + json.dumps({"sequence": sequence, **summary}), flush=True)
                served.append(sequence)
            if (inbox / proto.STOP_FILE).exists():
                _tell(fl, proto.STOP_COMMAND)
                return {"stopped": "stop_file", "served": served}
            nxt = inbox / proto.inbox_name(sequence + 1)
            if nxt.exists():
                # A request that cannot be read or does not pass the loaded profile's checks never reaches a GPU.  It ends the
                # session in order (the workers are told to stop) instead of being skipped: sequence numbers are claimed once, and
                # a producer that published something invalid cannot be trusted with the next number either.
                try:
                    payload = json.loads(read_bounded(nxt, request_schema.PAYLOAD_CAP))
                    profile_check(payload)
                except (OSError, ValueError) as exc:
                    _tell(fl, proto.STOP_COMMAND)
                    return {"stopped": "invalid_request", "sequence": sequence + 1, "error": f"{type(exc).__name__}: {exc}", "served": served}
                sequence += 1
                if wall_seconds is not None:
                    deadline = time.monotonic() + wall_seconds
                if not _tell(fl, proto.encode_command(sequence, payload)):
                    return {"stopped": "worker_exit", "exit_codes": fl.poll(), "served": served}
                continue
        time.sleep(poll)
    _tell(fl, proto.STOP_COMMAND)
    return {"stopped": "deadline", "served": served}


def _tell(fl: fleet_mod.Fleet, line: bytes) -> bool:
    """Write one line to every worker; False when a worker's pipe is gone (it exited between the poll and the write)."""
    try:
        fl.send_all(line)
    except OSError:
        return False
    return True


def main(argv=None) -> int:
    args = parse_args(argv)
    site = None
    if args.site:
        from glm_tpu_b200.config.site import SiteConfig

        site = SiteConfig.load(Path(args.site), required=True)
    run_root = Path(args.run_root) if args.run_root else (site.paths.run_root if site is not None else default_run_root())
    payload = json.loads(read_bounded(Path(args.request), request_schema.PAYLOAD_CAP)) if args.request else None
    if payload is None and not args.keep_loaded:
        raise SystemExit("--request is required unless --keep-loaded starts a resident session")
    rules = site.launch_rules if site is not None else args.policy
    with jobs.fleet_job(run_root, repo=REPO, policy=rules, require_idle=args.backend == "gpu") as job:
        run_dir = staging.new_run_dir(run_root)
        print(proto.STDOUT_RUN + str(run_dir), flush=True)
        staged = staging.stage_request(run_dir, payload)
        jobs.write_identity(run_dir, job, {"args": vars(args)})
        worker_args = ["--run-dir", str(run_dir), "--model", args.model, "--backend", args.backend, "--lanes", str(args.lanes),
                       "--kv-layout", args.kv_layout]
        if args.comm:  # left open, the workers read GLM_B200_COMM from the environment they inherit
            worker_args += ["--comm", args.comm]
        if args.context:
            worker_args += ["--context", str(args.context)]
        if staged is not None:
            worker_args += ["--request", str(staged), "--request-sha256", payload["request_sha256"]]
        if args.keep_loaded:
            worker_args.append("--keep-loaded")
        # what binds this launch: the resolved site (pins), a digest of every source file the workers import, the GPU binding
        extra_env: dict = {}
        if site is not None:
            worker_args += stage_site(run_dir, site)
        worker_args += stage_source_manifest(run_dir, REPO)
        if args.backend == "gpu":
            binding_args, extra_env = stage_binding(run_dir, site, Path(args.binding) if args.binding else None, args.gpus)
            worker_args += binding_args
        specs = fleet_mod.worker_specs(world=args.gpus, run_dir=run_dir, worker_args=worker_args, master_port=args.master_port,
                                       extra_env=extra_env)
        deadline = time.monotonic() + args.wall_seconds
        fl = job.start(specs, keep_stdin=args.keep_loaded)
        terminal: dict = {"run_dir": str(run_dir)}
        if args.keep_loaded:
            def check(p):
                pass  # the workers validate against the loaded profile; the controller only bounds and parses

            terminal["resident"] = resident_controller(fl, run_dir, args.gpus, check, deadline, args.poll_seconds,
                                                       initial=payload is not None, print_answers=args.print_answers,
                                                       wall_seconds=args.wall_seconds)
            codes = fl.wait(time.monotonic() + 30.0)
        else:
            codes = fl.wait(deadline)
        terminal["exit_codes"] = codes
        terminal["timed_out"] = any(c is None for c in codes)
        if any(c is None for c in codes) or any(c not in (None, 0) for c in codes):
            terminal["cleanup_exit_codes"] = fl.cleanup()
        summary = summarize(run_dir, args.gpus) if payload is not None else {"agree": all(c == 0 for c in codes), "requests": []}
        persist_json(run_dir / proto.SUMMARY_FILE, summary)
        terminal["ok"] = bool(summary["agree"]) and all(c == 0 for c in codes)
        persist_json(run_dir / proto.CONTROLLER_TERMINAL_FILE, terminal)
        if args.print_answers and (run_dir / proto.ANSWER_FILE).exists():
            print((run_dir / proto.ANSWER_FILE).read_text())
        print(json.dumps({"ok": terminal["ok"], "summary": summary}), flush=True)
        return 0 if terminal["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
