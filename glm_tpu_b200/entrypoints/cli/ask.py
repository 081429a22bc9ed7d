"""``ask``: turn one to ten questions into prepared requests and hand them to the controller.

The questions never touch the checkout: they are staged in a fresh owner-only directory under the run root, each as the chat messages
it was asked as (``messages-NNN.json``) and as the prepared request made from them (``prepared-NNN.json``: rendered with the chat
format, tokenized with the session's tokenizer, budgeted for the context profile), plus the one ``request.json`` the controller is
started with: the single request, or a batch (answered in order, or as up to four concurrent chats at the concurrent profile).

Parity: reference ``glm_tpu/entrypoints/cli/ask.py`` (same staging names, limits and refusals).
"""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass
from pathlib import Path

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.exceptions import RequestValidationError
from glm_tpu_b200.utils.io_utils import create_private_exclusive, read_bounded
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes


def _stage(directory: Path, name: str, value) -> bytes:
    """Write ``value`` as one canonical JSON line into a new private file; returns the bytes written."""
    line = canonical_wire_bytes(value) + b"\n"
    create_private_exclusive(directory / name, line)
    return line


@dataclass(frozen=True)
class QuestionSet:
    """What one ``ask`` invocation wants answered, checked against the profile before anything is written."""

    questions: list
    concurrent: bool
    context_capacity: int
    max_new_tokens: int | None

    def check(self, profile) -> None:
        texts = self.questions
        well_formed = isinstance(texts, list) and all(isinstance(t, str) and t.strip() for t in texts)
        if not well_formed or not 1 <= len(texts) <= rq.QUEUE_LIMIT:
            raise RequestValidationError("provide one to ten nonempty question strings")
        if self.concurrent and (len(texts) > profile.concurrent_limit or self.context_capacity != profile.concurrent_capacity):
            raise RequestValidationError("concurrent mode accepts up to four questions at the concurrent capacity profile")
        if self.max_new_tokens is not None and (type(self.max_new_tokens) is not int or self.max_new_tokens < 1):
            raise RequestValidationError("output budget must be a positive integer")

    def prepared(self, number: int, tokenizer, profile, directory: Path) -> dict:
        """Stage question ``number`` (0-based) and return its prepared request."""
        messages = [{"role": "user", "content": self.questions[number]}]
        _stage(directory, f"messages-{number:03d}.json", messages)
        prompt = tokenizer.apply_chat_template(messages, reasoning_effort="max")
        budget = self.max_new_tokens
        if budget is None:
            budget = rq.default_max_new_tokens(len(prompt), self.context_capacity, profile)
        if budget < 1:
            raise RequestValidationError("the question leaves no room for an answer at this context capacity")
        request = rq.from_token_ids(prompt, request_id=f"question-{number + 1:02d}", max_new_tokens=budget,
                                    context_capacity=self.context_capacity, profile=profile)
        _stage(directory, f"prepared-{number:03d}.json", request)
        return request


def prepare_questions(questions, *, tokenizer, profile, output_root: Path, context_capacity: int, max_new_tokens, concurrent=False,
                      repo: Path | None = None) -> Path:
    """Stage everything under ``output_root`` (which must not exist yet) and return the path of ``request.json``."""
    wanted = QuestionSet(questions, bool(concurrent), context_capacity, max_new_tokens)
    wanted.check(profile)
    directory = Path(output_root)
    if repo is not None and directory.resolve().is_relative_to(Path(repo).resolve()):
        raise RequestValidationError("private questions must stay outside the repository")
    directory.mkdir(mode=0o700, parents=True)
    try:
        requests = [wanted.prepared(number, tokenizer, profile, directory) for number in range(len(questions))]
        alone = len(requests) == 1 and not wanted.concurrent
        bundle = requests[0] if alone else rq.batch(requests, concurrent=wanted.concurrent, profile=profile)
        if len(canonical_wire_bytes(bundle)) + 1 > rq.PAYLOAD_CAP:
            raise RequestValidationError("combined request payload is too large")
        _stage(directory, "request.json", bundle)
    except BaseException:
        import shutil

        shutil.rmtree(directory, ignore_errors=True)  # a refused question set leaves no half-staged private input behind
        raise
    return directory / "request.json"


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
    stem = "inputs_" + time.strftime("%Y%m%dT%H%M%S") + f"_{os.getpid()}"
    root = next(candidate for candidate in (site.paths.run_root / (stem + (f".{n}" if n else "")) for n in range(1000)) if not candidate.exists())
    request_path = prepare_questions(questions, tokenizer=tokenizer, profile=profile, output_root=root, context_capacity=capacity,
                                     max_new_tokens=args.max_new_tokens, concurrent=args.concurrent, repo=launch.REPO)
    print("PRIVATE_INPUT " + str(request_path), flush=True)
    if args.prepare_only:
        return 0
    argv = ["--request", str(request_path), "--run-root", str(site.paths.run_root), "--gpus", str(args.gpus or site.gpus), "--model", model,
            "--backend", args.backend, "--context", str(capacity), "--wall-seconds", str(args.wall_seconds), "--policy", site.policy,
            "--master-port", str(site.master_port), "--print-answers"]
    if site.source != "<defaults>":
        argv += ["--site", site.source]  # its pins (checkpoint manifest, topology binding, launch rules) bind the workers
    if args.concurrent:
        argv += ["--lanes", str(len(questions))]
    if args.keep_loaded:
        argv.append("--keep-loaded")
    return launch.main(argv)
