"""``Resident``: the client side of a resident session (used by the job queue, the UI and the /v1 server).

It talks to a running controller only through the run directory: it prepares requests with the session's tokenizer
and pins, claims the next sequence number, publishes a request into ``inbox/`` with a hard link (create-once: it can
never overwrite another producer's request) and observes progress by reading the rank-0 token stream incrementally.
A job is complete only when the controller's measurement says all ranks agreed on the request and the token digest.

Parity: reference ``glm_tpu/engine/resident_client.py:58-235``.
"""

from __future__ import annotations

import hashlib
import json
import os
import struct
from pathlib import Path

from glm_tpu_b200.engine import request as request_schema
from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.engine.outputs import final_channel
from glm_tpu_b200.exceptions import ApiError
from glm_tpu_b200.utils.io_utils import atomic_json


class ResidentUnavailable(ValueError):
    pass


class Resident:
    def __init__(self, run_dir: Path, tokenizer, profile: request_schema.RequestProfile, *, capacity: int, world: int = 1):
        self.run = Path(run_dir)
        self.tokenizer, self.profile = tokenizer, profile
        self.capacity, self.world = capacity, world

    # ------------------------------------------------------------------ liveness
    def check(self) -> None:
        """The session must look alive: run directory, ready file, a live controller, no terminal record."""
        ident = self.run / proto.CONTROLLER_IDENTITY_FILE
        if not (self.run / proto.INBOX_DIR).is_dir() or not ident.exists():
            raise ResidentUnavailable("The resident model is unavailable. No model was restarted.")
        if (self.run / proto.CONTROLLER_TERMINAL_FILE).exists():
            raise ResidentUnavailable("The resident session has ended. No model was restarted.")
        pid = json.loads(ident.read_text()).get("pid")
        if pid is not None:
            try:
                os.kill(int(pid), 0)
            except (OSError, ValueError) as exc:
                raise ResidentUnavailable("The resident controller is gone. No model was restarted.") from exc

    # ------------------------------------------------------------------ preparing
    def prepare(self, messages: list, key: str) -> dict:
        """A UI turn: the whole conversation so far, default output budget."""
        self.check()
        ids = self.tokenizer.apply_chat_template(messages, reasoning_effort="max")
        remaining = self.capacity - len(ids)
        if remaining <= 0:
            raise ApiError(f"this conversation fills the {self.capacity}-slot context; start a new one")
        budget = request_schema.default_max_new_tokens(len(ids), self.capacity, self.profile)
        return request_schema.from_token_ids(ids, request_id="ui-" + key, max_new_tokens=budget, context_capacity=self.capacity,
                                             profile=self.profile)

    def prepare_api(self, messages: list, key: str, *, tools, effort, max_new_tokens, context_capacity: int | None = None) -> dict:
        """A complete stateless chat (tools included) at the loaded profile."""
        self.check()
        capacity = context_capacity or self.capacity
        ids = self.tokenizer.apply_chat_template(messages, tools=tools, reasoning_effort=effort)
        remaining = capacity - len(ids)
        if remaining <= 0:
            raise ApiError(f"this conversation fills the {capacity}-slot context; send less history or smaller tool output")
        budget = remaining if max_new_tokens is None else min(max_new_tokens, remaining)
        budget = min(budget, self.profile.max_new)
        return request_schema.from_token_ids(ids, request_id="api-" + key, max_new_tokens=budget, context_capacity=capacity,
                                             profile=self.profile)

    # ------------------------------------------------------------------ publishing
    def next_sequence(self) -> int:
        self.check()
        ready_file = self.run / proto.READY_FILE
        if not ready_file.exists():
            raise ValueError("The resident model is still loading.")
        ready = json.loads(ready_file.read_text())["sequence"]
        if ready > 0 and not (proto.result_dir(self.run, ready) / proto.MEASUREMENT_FILE).exists():
            raise ValueError("The resident controller is still collecting its previous answer.")
        inbox = self.run / proto.INBOX_DIR
        if any(p.stem.isdigit() and int(p.stem) > ready for p in inbox.glob("*.json")):
            raise ValueError("The resident inbox has another request owner.")
        return ready + 1

    def publish(self, job: dict, state_dir: Path) -> None:
        self.check()
        request_schema.validate_payload(job["payload"], self.profile)
        source = Path(state_dir) / (job["id"] + ".request.json")
        if not source.exists():
            atomic_json(source, job["payload"])
        elif json.loads(source.read_text()) != job["payload"]:
            raise ValueError("Saved request identity differs; preserved for inspection.")
        target = self.run / proto.INBOX_DIR / proto.inbox_name(job["sequence"])
        try:
            os.link(source, target)  # publish once, never overwrite another producer
        except FileExistsError:
            if target.is_symlink() or json.loads(target.read_text()) != job["payload"]:
                raise ValueError("Resident sequence belongs to a different request.") from None

    # ------------------------------------------------------------------ observing
    def observe(self, job: dict) -> dict:
        root = proto.result_dir(self.run, job["sequence"])
        token_file = root / proto.TOKENS_FILE
        events = []
        if token_file.exists():
            for line in token_file.read_bytes().splitlines(keepends=True):
                if line.endswith(b"\n"):  # a partially written last line is not an event yet
                    events.append(json.loads(line))
        rid = job["payload"]["request_id"]
        if any(ev["request_id"] != rid or ev["index"] != i for i, ev in enumerate(events)):
            raise ValueError("Token stream identity differs.")
        ids = [ev["token_id"] for ev in events]
        text = self.tokenizer.decode([t for t in ids if t not in self.profile.eos_ids])
        thinking, answer = final_channel("<think>" + text)
        update = {"thinking": thinking, "answer": answer, "output_tokens": len(events), "status": "generating"}
        receipt = root / proto.MEASUREMENT_FILE
        if not receipt.exists():
            self.check()
            return update
        summary = json.loads(receipt.read_text())
        digest = hashlib.sha256(struct.pack(f"<{len(ids)}i", *ids)).hexdigest()
        reports = [r for r in summary.get("requests", []) if r["request_id"] == rid]
        if not (summary.get("agree") and summary.get("ranks") == self.world and len(reports) == 1):
            raise ValueError("Resident completion check failed.")
        report = reports[0]
        if report["token_sha256"] != digest or report["emitted"] != len(events):
            raise ValueError("All-rank request/token agreement failed.")
        complete = report["finish_reason"] == "eos" and bool(answer)
        update.update(status="complete" if complete else "incomplete", finish_reason=report["finish_reason"],
                      stop_cause=request_schema.stop_cause(job["payload"], report["finish_reason"]),
                      decode_tps=report.get("decode_tokens_per_second"), prefill_seconds=report.get("prefill_seconds"))
        return update
