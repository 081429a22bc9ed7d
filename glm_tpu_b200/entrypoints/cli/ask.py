"""``ask``: prepare one to ten questions and hand them to the controller.

Questions are rendered with the chat format, tokenized with the session's tokenizer and written as prepared requests
into a fresh owner-only directory under the run root (never inside the checkout); one batch (sequential, or up to four
concurrent chats at the 32K profile) is queued before the single launch.

Parity: reference ``glm_tpu/entrypoints/cli/ask.py:12-93``.
"""

from __future__ import annotations

import json
import os
import time
from pathlib import Path

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.utils.io_utils import create_private_exclusive, read_bounded
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes


def prepare_questions(questions, *, tokenizer, profile, output_root: Path, context_capacity: int, max_new_tokens, concurrent=False,
                      repo: Path | None = None) -> Path:
    if type(questions) is not list or not 1 <= len(questions) <= rq.QUEUE_LIMIT or any(type(q) is not str or not q.strip() for q in questions):
        raise ValueError("provide one to ten nonempty question strings")
    if repo is not None and Path(output_root).resolve().is_relative_to(Path(repo).resolve()):
        raise ValueError("private questions must stay outside the repository")
    if concurrent and (len(questions) > profile.concurrent_limit or context_capacity != profile.concurrent_capacity):
        raise ValueError("concurrent mode accepts up to four questions at the concurrent capacity profile")
    if max_new_tokens is not None and (type(max_new_tokens) is not int or max_new_tokens < 1):
        raise ValueError("output budget must be a positive integer")
    output_root = Path(output_root)
    output_root.mkdir(mode=0o700, parents=True)
    values = []
    for index, question in enumerate(questions):
        messages = [{"role": "user", "content": question}]
        create_private_exclusive(output_root / f"messages-{index:03d}.json", canonical_wire_bytes(messages) + b"\n")
        ids = tokenizer.apply_chat_template(messages, reasoning_effort="max")
        budget = max_new_tokens if max_new_tokens is not None else rq.default_max_new_tokens(len(ids), context_capacity, profile)
        if budget < 1:
            raise ValueError("the question leaves no room for an answer at this context capacity")
        prepared = rq.from_token_ids(ids, request_id=f"question-{index + 1:02d}", max_new_tokens=budget,
                                     context_capacity=context_capacity, profile=profile)
        create_private_exclusive(output_root / f"prepared-{index:03d}.json", canonical_wire_bytes(prepared) + b"\n")
        values.append(prepared)
    value = values[0] if len(values) == 1 and not concurrent else rq.batch(values, concurrent=concurrent, profile=profile)
    raw = canonical_wire_bytes(value) + b"\n"
    if len(raw) > rq.PAYLOAD_CAP:
        raise ValueError("combined request payload is too large")
    path = output_root / "request.json"
    create_private_exclusive(path, raw)
    return path


def main(args) -> int:
    from glm_tpu_b200.config.site import SiteConfig
    from glm_tpu_b200.executor import multiproc_executor as launch
    from glm_tpu_b200.tokenizer import load_tokenizer
    from glm_tpu_b200.worker.gpu_worker import profile_for, resolve_model

    site = SiteConfig.load(getattr(args, "site", None))
    questions = json.loads(read_bounded(args.questions, 10 * rq.MESSAGES_CAP)) if args.questions is not None else [args.question]
    model = args.model or (str(site.paths.packed_path) if site.paths.packed_path else "random:glm53")
    geometry, (kind, path) = resolve_model(model)
    capacity = args.capacity or rq.CONTEXT_ALIASES[args.context]
    profile = profile_for(geometry, capacity)
    tokenizer = load_tokenizer(path if kind == "checkpoint" else site.paths.model_path, vocab_size=geometry.vocab_size,
                               eos_ids=geometry.eos_ids)
    root = site.paths.run_root / ("inputs_" + time.strftime("%Y%m%dT%H%M%S") + f"_{os.getpid()}")
    request_path = prepare_questions(questions, tokenizer=tokenizer, profile=profile, output_root=root, context_capacity=capacity,
                                     max_new_tokens=args.max_new_tokens, concurrent=args.concurrent, repo=launch.REPO)
    print("PRIVATE_INPUT " + str(request_path), flush=True)
    if args.prepare_only:
        return 0
    argv = ["--request", str(request_path), "--run-root", str(site.paths.run_root), "--gpus", str(args.gpus or site.gpus), "--model", model,
            "--backend", args.backend, "--context", str(capacity), "--wall-seconds", str(args.wall_seconds), "--policy", site.policy,
            "--master-port", str(site.master_port), "--print-answers"]
    if args.concurrent:
        argv += ["--lanes", str(len(questions))]
    if args.keep_loaded:
        argv.append("--keep-loaded")
    return launch.main(argv)
