"""``prepare-request``: turn a messages file (or raw token ids) into a prepared request without launching anything.

Parity: reference ``glm_tpu/entrypoints/cli/prepare.py:1-57``.
"""

from __future__ import annotations

import json
from pathlib import Path

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.utils.io_utils import create_private_exclusive, read_bounded
from glm_tpu_b200.utils.json_utils import canonical_wire_bytes


def main(args) -> int:
    from glm_tpu_b200.config.site import SiteConfig
    from glm_tpu_b200.tokenizer import load_tokenizer
    from glm_tpu_b200.worker.gpu_worker import profile_for, resolve_model

    site = SiteConfig.load(getattr(args, "site", None))
    geometry, (kind, path) = resolve_model(args.model)
    capacity = args.capacity or rq.CONTEXT_ALIASES[args.context]
    profile = profile_for(geometry, capacity)
    if args.token_ids is not None:
        ids = json.loads(read_bounded(args.token_ids, rq.PAYLOAD_CAP))
        budget = args.max_new_tokens or rq.default_max_new_tokens(len(ids), capacity, profile)
        prepared = rq.from_token_ids(ids, request_id=args.request_id, max_new_tokens=budget, context_capacity=capacity, profile=profile)
    else:
        tokenizer = load_tokenizer(path if kind == "checkpoint" else site.paths.model_path, vocab_size=geometry.vocab_size,
                                   eos_ids=geometry.eos_ids)
        messages = json.loads(read_bounded(args.messages, rq.MESSAGES_CAP))
        prepared = rq.from_messages(messages, tokenizer=tokenizer, request_id=args.request_id, max_new_tokens=args.max_new_tokens,
                                    context_capacity=capacity, profile=profile, reasoning_effort=args.reasoning_effort)
    ids, budget = prepared["prompt_ids"], prepared["max_new_tokens"]
    checkout = Path(__file__).resolve().parents[3]
    if Path(args.output).resolve().is_relative_to(checkout):
        from glm_tpu_b200.exceptions import ConfigValidationError

        raise ConfigValidationError("private requests must be written outside the source checkout")
    create_private_exclusive(Path(args.output), canonical_wire_bytes(prepared) + b"\n")
    print(json.dumps({"output": str(args.output), "prompt_tokens": len(ids), "max_new_tokens": budget,
                      "request_sha256": prepared["request_sha256"]}))
    return 0
