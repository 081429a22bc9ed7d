"""The persistent queue of chat jobs, served one at a time by the resident session.

Jobs come from the browser workspace (a turn of a saved conversation) and from the ``/v1`` API (stateless).  The
queue owns a private state directory: ``chats.json`` holds conversations and jobs in one document, written
atomically under one lock.  ``step`` advances the oldest unfinished job: claim a sequence number (made durable before
anything is published), publish the request into the inbox, observe progress.  After an uncertain failure the queue
stops and keeps the job's identity, so a restart can reconcile the SAME request and never resubmits it under a fresh
sequence.  At most ``PENDING`` jobs wait at once; finished stateless jobs beyond ``API_HISTORY`` are retired.

Parity: reference ``glm_tpu/entrypoints/serve/job_queue.py:11-109``.
"""

from __future__ import annotations

import json
import threading
import time
from pathlib import Path

from glm_tpu_b200.exceptions import ApiError
from glm_tpu_b200.utils.io_utils import atomic_json

PENDING = 10
API_HISTORY = 50
ACTIVE = ("queued", "generating")
DONE = ("complete", "incomplete")


class JobQueue:
    def __init__(self, root: Path, backend):
        root = Path(root)
        root.mkdir(mode=0o700, parents=True, exist_ok=True)
        if root.is_symlink() or root.stat().st_mode & 0o077:
            raise ValueError("Chat directory must be private (mode 0700).")
        self.root, self.backend = root, backend
        self.mutex = threading.RLock()
        doc = root / "chats.json"
        self.db = json.loads(doc.read_text()) if doc.exists() else {"chats": [], "jobs": []}
        self.error: str | None = None
        self.stopping = threading.Event()
        self.conversations = None  # the ConversationStore built on this queue

    def save(self) -> None:
        atomic_json(self.root / "chats.json", self.db)

    def pending(self) -> int:
        return sum(1 for j in self.db["jobs"] if j["status"] in ACTIVE)

    def new_job(self, key: str, payload: dict, *, chat, label: str, user_text: str = "", api: bool = False) -> dict:
        return {"id": key, "chat": chat, "api": api, "label": label, "user_text": user_text, "status": "queued", "payload": payload,
                "sequence": None, "answer": "", "thinking": "", "output_tokens": 0, "prompt_tokens": len(payload["prompt_ids"]),
                "created": time.time()}

    def admit(self) -> None:
        if self.error:
            raise ApiError(self.error, status=503, kind="server_error")
        if self.pending() >= PENDING:
            raise ApiError("too many requests are already waiting for this one model", status=429, kind="rate_limit_error")

    def submit(self, payload: dict, key: str, *, label: str) -> dict:
        """Queue a stateless request (idempotent by ``key``)."""
        with self.mutex:
            existing = next((j for j in self.db["jobs"] if j["id"] == key), None)
            if existing is not None:
                return existing
            self.admit()
            job = self.new_job(key, payload, chat=None, label=label, api=True)
            self.db["jobs"].append(job)
            self.retire()
            self.save()
            return job

    def job(self, key: str):
        with self.mutex:
            found = next((j for j in self.db["jobs"] if j["id"] == key), None)
            return None if found is None else json.loads(json.dumps({k: v for k, v in found.items() if k != "payload"}))

    def retire(self) -> None:
        finished = [j for j in self.db["jobs"] if j.get("api") and j["status"] in DONE]
        for job in finished[:-API_HISTORY] if len(finished) > API_HISTORY else []:
            self.db["jobs"].remove(job)

    def step(self) -> None:
        with self.mutex:
            job = next((j for j in self.db["jobs"] if j["status"] in ACTIVE), None)
            if job is None or self.error:
                return
            try:
                if job["sequence"] is None:
                    job["sequence"] = self.backend.next_sequence()
                    self.save()  # durable identity before any inbox write
                self.backend.publish(job, self.root)
                job.update(self.backend.observe(job))
                if job.get("chat") and self.conversations is not None:
                    self.conversations.update_message(job)
                self.save()
            except Exception as exc:  # noqa: BLE001 - stop, keep the admission identity, never resubmit
                self.error = str(exc)
                job["error"] = self.error
                atomic_json(self.root / "error.json", {"error": self.error, "job": job["id"], "time": time.time()})

    def work(self) -> None:
        while not self.stopping.is_set():
            self.step()
            with self.mutex:
                active = any(j["status"] == "generating" for j in self.db["jobs"])
            self.stopping.wait(0.2 if active else 1.0)
