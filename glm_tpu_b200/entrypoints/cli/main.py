"""``glm-b200``: the command line of the engine (``python -m glm_tpu_b200``).

    info                         supported scope and limits
    ask [QUESTION | --questions FILE] [--context 8k|32k|128k|256k] [--concurrent] [--keep-loaded] ...
    prepare-request              messages or token ids -> prepared request (nothing is launched)
    collect-env | doctor         environment report checked against a profile
    checkpoint inventory|mark-source|pack|verify
    topology capture|bind
    serve                        loopback chat UI + OpenAI-compatible /v1 attached to a resident session

Subcommand modules are imported only when their command runs, so ``info`` and ``--help`` never import torch.

Parity: reference ``glm_tpu/entrypoints/cli/main.py:87-146``.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Sequence

CONTEXTS = ("8k", "32k", "128k", "256k")


def _info(args) -> int:
    print(json.dumps({
        "engine": "glm_tpu_b200",
        "model": "GlmMoeDsaForCausalLM (GLM-5.3), FP8 e4m3 routed experts with 128x128 block scales, bf16 elsewhere",
        "hardware": "one box of 1, 2, 4 or 8 NVIDIA B200 (sm_100a) with NVLink peer access",
        "modes": ["one-shot answer", "sequential queue (<= 10)", "four concurrent chats (32k)", "resident session",
                  "loopback chat UI", "OpenAI-compatible /v1 (chat completions, models, tools, SSE)"],
        "decoding": "greedy only; sampling parameters are accepted and ignored",
        "contexts": {"8k": 8192, "32k": 32768, "128k": 166912, "256k": 262144},
        "recovery": "none: a failed step poisons the engine; there are no retries",
        "not_loaded": "the checkpoint's multi-token-prediction layer",
    }, indent=2, sort_keys=True))
    return 0


def _ask(args) -> int:
    from glm_tpu_b200.entrypoints.cli.ask import main

    return main(args)


def _prepare(args) -> int:
    from glm_tpu_b200.entrypoints.cli.prepare import main

    return main(args)


def _collect_env(args) -> int:
    from glm_tpu_b200.entrypoints.cli.collect_env import main

    return main(args)


def _checkpoint(args) -> int:
    from glm_tpu_b200.entrypoints.cli.checkpoint import main

    return main(args)


def _topology(args) -> int:
    from glm_tpu_b200.entrypoints.cli.topology import main

    return main(args)


def serve_arguments(args) -> list[str]:
    """The server's own argument list: what the command line leaves open comes from the site file (``[serve] port``,
    ``[paths] state_root``), then from the built-in default."""
    from glm_tpu_b200.config.site import SiteConfig
    from glm_tpu_b200.exceptions import ConfigValidationError

    site = SiteConfig.load(args.site)
    state = args.state if args.state is not None else site.paths.state_root
    if state is None:
        raise ConfigValidationError("where the chat state lives is not set: give --state or [paths] state_root in the site file")
    port = args.port if args.port is not None else site.serve_port
    return ["--run", str(args.run), "--state", str(state), "--port", str(port)] + (["--no-api"] if args.no_api else [])


def _serve(args) -> int:
    from glm_tpu_b200.entrypoints.serve.server import main

    return main(serve_arguments(args))


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="glm-b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    sub.add_parser("info", help="show supported scope and limits").set_defaults(fn=_info)

    ask = sub.add_parser("ask", help="answer questions; optionally batch up to four concurrent chats")
    inputs = ask.add_mutually_exclusive_group(required=True)
    inputs.add_argument("question", nargs="?")
    inputs.add_argument("--questions", type=Path, help="private JSON array of one to ten question strings")
    ask.add_argument("--context", choices=CONTEXTS, default="32k")
    ask.add_argument("--capacity", type=int, help="explicit context slots (fixtures); overrides --context")
    ask.add_argument("--keep-loaded", action="store_true", help="keep the model loaded as a resident session")
    ask.add_argument("--concurrent", action="store_true", help="run up to four questions as concurrent chats (32k)")
    ask.add_argument("--max-new-tokens", type=int)
    ask.add_argument("--wall-seconds", type=int, default=86400)
    ask.add_argument("--prepare-only", action="store_true")
    ask.add_argument("--model", help="random:<tiny|small|glm53>[:layers] or a packed checkpoint (default: the site's)")
    ask.add_argument("--backend", choices=("gpu", "oracle"), default="gpu")
    ask.add_argument("--gpus", type=int)
    ask.add_argument("--site", type=Path)
    ask.set_defaults(fn=_ask)

    prep = sub.add_parser("prepare-request", help="prepare a request without launching the model")
    source = prep.add_mutually_exclusive_group(required=True)
    source.add_argument("--messages", type=Path, help="JSON array of chat messages")
    source.add_argument("--token-ids", type=Path, help="JSON array of prompt token ids")
    prep.add_argument("--output", type=Path, required=True)
    prep.add_argument("--request-id", default="request-01")
    prep.add_argument("--context", choices=CONTEXTS, default="32k")
    prep.add_argument("--capacity", type=int)
    prep.add_argument("--max-new-tokens", type=int)
    prep.add_argument("--reasoning-effort", choices=("low", "high", "max"), default="max")
    prep.add_argument("--model", default="random:glm53")
    prep.add_argument("--site", type=Path)
    prep.set_defaults(fn=_prepare)

    for name in ("collect-env", "doctor"):
        env = sub.add_parser(name, help="report the environment and check it against a profile")
        env.add_argument("--profile", choices=("dev", "serve"), default="dev")
        env.set_defaults(fn=_collect_env)

    ck = sub.add_parser("checkpoint", help="inventory, mark, pack and verify checkpoints")
    cks = ck.add_subparsers(dest="action", required=True)
    inv = cks.add_parser("inventory", help="read the safetensors headers of a source checkpoint")
    inv.add_argument("source", type=Path)
    inv.add_argument("--output", type=Path, help="also write the inventory (every tensor: dtype, shape, shard, byte range) to this file, create-once")
    mark = cks.add_parser("mark-source", help="write SOURCE_COMPLETE.json after checking the source against its index")
    mark.add_argument("source", type=Path)
    mark.add_argument("--hash-shards", action="store_true", help="record a SHA-256 of every shard (reads the whole source)")
    mark.add_argument("--upstream-marker", type=Path, help="compare this copy with the SOURCE_COMPLETE.json of another copy instead of marking it")
    mark.add_argument("--output", type=Path, help="with --upstream-marker: where the record computed here is written (the source is not written to)")
    pack = cks.add_parser("pack", help="pack a source checkpoint into per-GPU runtime shards")
    pack.add_argument("source", type=Path)
    pack.add_argument("target", type=Path)
    pack.add_argument("--gpus", type=int, default=8)
    pack.add_argument("--layers", type=int, default=0)
    pack.add_argument("--expert-split", default="auto", choices=["auto", "whole", "sliced"],
                      help="routed experts per GPU: whole experts, or a column slice of every expert (auto: sliced where the FP8 blocks allow)")
    pack.add_argument("--site", type=Path, help="site file (default: the configured one); its [checkpoint] source_marker_sha256 pins the source")
    pack.add_argument("--preflight-only", action="store_true", help="run every check a pack makes before it writes (marker, pin, tensor set, free space) and write nothing")
    ver = cks.add_parser("verify", help="re-hash a packed checkpoint against its manifest and seal")
    ver.add_argument("target", type=Path)
    ver.add_argument("--site", type=Path, help="site file (default: the configured one); its [checkpoint] manifest_sha256 pins the checkpoint")
    ver.add_argument("--files", nargs="+", metavar="NAME", help="check only these files of the checkpoint (default: all), e.g. the one a GPU loads")
    ver.add_argument("--headers-only", action="store_true", help="check seal, manifest, sizes and headers but do not re-hash the payloads")
    ck.set_defaults(fn=_checkpoint)

    topo = sub.add_parser("topology", help="capture and bind the GPU topology")
    tops = topo.add_subparsers(dest="action", required=True)
    cap = tops.add_parser("capture")
    cap.add_argument("--output", type=Path, required=True)
    bind = tops.add_parser("bind")
    bind.add_argument("capture", type=Path)
    bind.add_argument("--gpus", type=int, default=8)
    topo.set_defaults(fn=_topology)

    srv = sub.add_parser("serve", help="chat UI + /v1 API attached to a resident session")
    srv.add_argument("--run", type=Path, required=True)
    srv.add_argument("--state", type=Path, help="state directory (default: the site's [paths] state_root)")
    srv.add_argument("--port", type=int, help="loopback port (default: the site's [serve] port, 8011)")
    srv.add_argument("--no-api", action="store_true")
    srv.add_argument("--site", type=Path)
    srv.set_defaults(fn=_serve)
    return parser


def main(argv: Sequence[str] | None = None) -> int:
    """Exit status 0: done; 1: the command ran and reports a failure; 2: refused before anything ran (an invalid site file,
    checkpoint, request or argument), with one JSON line on stderr saying which check refused and why."""
    args = build_parser().parse_args(argv)
    try:
        return args.fn(args)
    except ValueError as exc:
        from glm_tpu_b200 import exceptions

        if not isinstance(exc, (exceptions.ConfigValidationError, exceptions.RequestValidationError, exceptions.ApiError)):
            raise  # not a refusal of ours: a defect, and it should look like one
        print(json.dumps({"ok": False, "refused": type(exc).__name__, "message": str(exc)}, sort_keys=True), file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
