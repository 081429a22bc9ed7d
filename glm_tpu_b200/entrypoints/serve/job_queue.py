"""The persistent queue of chat jobs that the resident session serves one at a time.

Two producers feed it: the browser workspace (a turn of a saved conversation, ``api`` false) and the ``/v1`` endpoint (stateless,
``api`` true).  Conversations and jobs live in ONE document, ``chats.json`` in a directory only its owner may enter; every change is
made under ``mutex`` and written atomically.

``step`` moves the oldest unfinished job forward by one observation:

1. give it a sequence number from the backend and make that durable *before* anything reaches the session's inbox;
2. publish the request (idempotent: publishing the same sequence twice is a no-op on the other side);
3. fold what the session has produced so far into the job.

If any of this fails in a way that leaves the outcome unknown, the queue halts: the error is recorded, the job keeps its sequence, and
nothing is ever resubmitted under a new number, so a restart reconciles the same request.  No more than ``PENDING`` jobs wait at a time;
finished stateless jobs beyond the newest ``API_HISTORY`` are dropped.

Behaviour parity: reference ``glm_tpu/entrypoints/serve/job_queue.py`` (same states, limits and halt rule).
"""

from __future__ import annotations

import copy
import json
import stat
import threading
import time
from pathlib import Path

from glm_tpu_b200.exceptions import ApiError
from glm_tpu_b200.utils.io_utils import atomic_json

PENDING = 10
API_HISTORY = 50
ACTIVE = ("queued", "generating")
DONE = ("complete", "incomplete")
DOCUMENT, HALT_RECORD = "chats.json", "error.json"
BUSY_POLL_SECONDS, IDLE_POLL_SECONDS = 0.2, 1.0


def _private_directory(root: Path) -> Path:
    root.mkdir(mode=0o700, parents=True, exist_ok=True)
    facts = root.lstat()
    if not stat.S_ISDIR(facts.st_mode) or stat.S_IMODE(facts.st_mode) & 0o077:
        raise ValueError("Chat directory must be private (mode 0700).")
    return root


class JobQueue:
    def __init__(self, root: Path, backend):
        self.root = _private_directory(Path(root))
        self.backend = backend
        self.mutex = threading.RLock()
        self.stopping = threading.Event()
        self.error: str | None = None      # set when the queue has halted; every admission is refused from then on
        self.conversations = None          # the ConversationStore built on this queue registers itself here
        document = self.root / DOCUMENT
        self.db = json.loads(document.read_text()) if document.exists() else {"chats": [], "jobs": []}

    # ------------------------------------------------------------------------------------------------------------------ the document
    def save(self) -> None:
        atomic_json(self.root / DOCUMENT, self.db)

    def _find(self, key: str):
        for job in self.db["jobs"]:
            if job["id"] == key:
                return job
        return None

    def pending(self) -> int:
        return len([job for job in self.db["jobs"] if job["status"] in ACTIVE])

    def new_job(self, key: str, payload: dict, *, chat, label: str, user_text: str = "", api: bool = False) -> dict:
        return {
            "id": key, "chat": chat, "api": api, "label": label, "user_text": user_text,
            "status": "queued", "sequence": None, "payload": payload, "created": time.time(),
            "prompt_tokens": len(payload["prompt_ids"]), "output_tokens": 0, "thinking": "", "answer": "",
        }

    def retire(self) -> None:
        """Forget the oldest finished stateless jobs; conversation turns stay with their conversation."""
        spent = [job for job in self.db["jobs"] if job.get("api") and job["status"] in DONE]
        surplus = len(spent) - API_HISTORY
        for job in spent[:max(surplus, 0)]:
            self.db["jobs"].remove(job)

    # ------------------------------------------------------------------------------------------------------------------ producers
    def admit(self) -> None:
        if self.error:
            raise ApiError(self.error, status=503, kind="server_error")
        if self.pending() >= PENDING:
            raise ApiError("too many requests are already waiting for this one model", status=429, kind="rate_limit_error")

    def submit(self, payload: dict, key: str, *, label: str) -> dict:
        """Queue a stateless request.  Submitting a key twice returns the first job."""
        with self.mutex:
            known = self._find(key)
            if known is not None:
                return known
            self.admit()
            fresh = self.new_job(key, payload, chat=None, label=label, api=True)
            self.db["jobs"].append(fresh)
            self.retire()
            self.save()
            return fresh

    def job(self, key: str):
        """A detached copy of the job without its prepared request, or ``None``."""
        with self.mutex:
            found = self._find(key)
            if found is None:
                return None
            return copy.deepcopy({field: value for field, value in found.items() if field != "payload"})

    # ------------------------------------------------------------------------------------------------------------------ the consumer
    def _advance(self, job: dict) -> None:
        if job["sequence"] is None:
            job["sequence"] = self.backend.next_sequence()
            self.save()  # the identity is on disk before the session can see the request
        self.backend.publish(job, self.root)
        job.update(self.backend.observe(job))
        if job.get("chat") and self.conversations is not None:
            self.conversations.update_message(job)
        self.save()

    def _halt(self, job: dict, problem: Exception) -> None:
        self.error = job["error"] = str(problem)
        atomic_json(self.root / HALT_RECORD, {"error": self.error, "job": job["id"], "time": time.time()})

    def step(self) -> None:
        with self.mutex:
            if self.error:
                return
            oldest = next((job for job in self.db["jobs"] if job["status"] in ACTIVE), None)
            if oldest is None:
                return
            try:
                self._advance(oldest)
            except Exception as problem:  # noqa: BLE001 - whatever it was, the outcome is unknown: halt and keep the identity
                self._halt(oldest, problem)

    def work(self) -> None:
        """The consumer thread: step, then sleep briefly while something is generating and longer while idle."""
        while not self.stopping.is_set():
            self.step()
            with self.mutex:
                generating = any(job["status"] == "generating" for job in self.db["jobs"])
            self.stopping.wait(BUSY_POLL_SECONDS if generating else IDLE_POLL_SECONDS)
