"""Saved conversations of the loopback chat workspace, stored in the job queue's document.

A small action table (``ACTIONS``) maps each ``POST /api/chat`` action to its handler; the fields of a request go through
one validator each (``valid_title``, ``valid_message_id``, ``valid_text``).  Actions: ``create``, ``rename``, ``send`` (idempotent by a client-generated 32-hex message id; one
turn at a time per conversation; at most ten waiting jobs overall), ``delete`` (refused while a turn is running).
``snapshot`` is what ``GET /api/state`` returns: conversations, non-API jobs without their private payloads, the
session's availability, capacity and scheduling mode.

Parity: reference ``glm_tpu/entrypoints/ui/conversations.py:16-119``.
"""

from __future__ import annotations

import copy
import re
import uuid
from typing import Callable, NamedTuple

from glm_tpu_b200.entrypoints.serve.job_queue import ACTIVE, PENDING

MESSAGE_ID = re.compile("[a-f0-9]{32}")
MAX_MESSAGE_BYTES = 128000
MAX_TITLE_CHARS = 100
AUTO_TITLE_CHARS = 55
DEFAULT_TITLE = "New conversation"
PUBLIC_MESSAGE_EXTRAS = ("thinking", "output_tokens", "decode_tps")


class Refused(ValueError):
    """What the client did cannot be done; the sentence is shown to the user as it is."""


# ------------------------------------------------------------------------------------------------- field validators
def valid_title(value) -> str:
    title = value.strip() if isinstance(value, str) else ""
    if type(value) is not str or not 1 <= len(title) <= MAX_TITLE_CHARS:
        raise Refused("Use a title between 1 and 100 characters.")
    return title


def valid_message_id(value) -> str:
    if type(value) is not str or MESSAGE_ID.fullmatch(value) is None:
        raise Refused("Invalid message identity.")
    return value


def valid_text(value) -> str:
    if type(value) is not str or not value.strip() or len(value.encode()) > MAX_MESSAGE_BYTES:
        raise Refused("Enter a message of at most 128,000 bytes.")
    return value


class Action(NamedTuple):
    run: Callable  # (store, conversation or None, request) -> reply or None (None: persist and answer {"ok": True})
    on_conversation: bool


class ConversationStore:
    def __init__(self, queue, model_name: str = "GLM-5.3"):
        self.queue = queue
        self.model_name = model_name
        queue.conversations = self

    # --------------------------------------------------------------------------------------------- reads
    def snapshot(self) -> dict:
        q = self.queue
        with q.mutex:
            try:
                q.backend.check()
                availability = q.error
            except (ValueError, OSError) as exc:
                availability = str(exc)
            public_jobs = [{key: value for key, value in job.items() if key != "payload"} for job in q.db["jobs"] if not job.get("api")]
            state = {"chats": q.db["chats"], "jobs": public_jobs, "error": availability, "model": self.model_name,
                     "capacity": q.backend.capacity, "scheduling": "sequential"}
            return copy.deepcopy(state)  # the caller serialises it outside the lock

    def _find(self, conversation_id) -> dict:
        for conversation in self.queue.db["chats"]:
            if conversation["id"] == conversation_id:
                return conversation
        raise Refused("Conversation not found.")

    def _jobs_of(self, conversation: dict) -> list:
        return [job for job in self.queue.db["jobs"] if job["chat"] == conversation["id"]]

    # --------------------------------------------------------------------------------------------- writes
    def change(self, request: dict) -> dict:
        """One action of ``POST /api/chat``; every action runs under the queue's lock and is saved before it is answered."""
        q = self.queue
        with q.mutex:
            name = request.get("action")
            action = ACTIONS.get(name) if type(name) is str else None  # anything else (a list, a number) is an unknown action, not a crash
            if action is None:
                self._find(request.get("chat"))  # an unknown conversation is reported before an unknown action
                raise Refused("Unknown action.")
            conversation = self._find(request.get("chat")) if action.on_conversation else None
            reply = action.run(self, conversation, request)
            if reply is None or reply.pop("persist", False):
                q.save()
            return reply if reply is not None else {"ok": True}

    def _create(self, _conversation, _request) -> dict:
        conversation = {"id": uuid.uuid4().hex, "title": DEFAULT_TITLE, "messages": []}
        self.queue.db["chats"].append(conversation)
        return {"id": conversation["id"], "persist": True}

    def _rename(self, conversation: dict, request: dict) -> None:
        conversation["title"] = valid_title(request.get("title"))

    def _delete(self, conversation: dict, _request) -> None:
        q = self.queue
        if any(job["status"] in ACTIVE for job in self._jobs_of(conversation)):
            raise Refused("Wait for this conversation to finish before deleting it.")
        q.db["chats"].remove(conversation)
        q.db["jobs"] = [job for job in q.db["jobs"] if job["chat"] != conversation["id"]]

    def _send(self, conversation: dict, request: dict):
        q = self.queue
        key, text = valid_message_id(request.get("id")), request.get("text")
        earlier = next((job for job in q.db["jobs"] if job["id"] == key), None)
        if earlier is not None:  # the same send again (a retry after a lost reply): answer as before, change nothing
            if (earlier["chat"], earlier["user_text"]) != (conversation["id"], text):
                raise Refused("Message identity was already used.")
            return {"id": key}
        text = valid_text(text)
        self._require_room_for_a_turn(conversation)
        history = [{"role": m["role"], "content": m["content"]} for m in conversation["messages"]]
        turn = {"role": "user", "content": text}
        payload = q.backend.prepare(history + [turn], key)
        q.db["jobs"].append(q.new_job(key, payload, chat=conversation["id"], label="ui", user_text=text))
        first_turn = not conversation["messages"]
        conversation["messages"].extend([turn, {"role": "assistant", "content": "", "status": "queued", "job": key}])
        if first_turn and conversation["title"] == DEFAULT_TITLE:
            conversation["title"] = " ".join(text.split())[:AUTO_TITLE_CHARS]
        return None

    def _require_room_for_a_turn(self, conversation: dict) -> None:
        q = self.queue
        if q.error:
            raise Refused(q.error)
        if q.pending() >= PENDING:
            raise Refused("Ten messages are already waiting. Wait for an answer.")
        messages = conversation["messages"]
        if messages and messages[-1].get("status") != "complete":
            raise Refused("Wait for a completed answer, or start a new conversation.")

    # --------------------------------------------------------------------------------------------- called by the queue
    def update_message(self, job: dict) -> None:
        conversation = self._find(job["chat"])
        message = next(m for m in conversation["messages"] if m.get("job") == job["id"])
        message["content"], message["status"] = job["answer"], job["status"]
        message.update({key: job[key] for key in PUBLIC_MESSAGE_EXTRAS if key in job})


ACTIONS = {
    "create": Action(ConversationStore._create, on_conversation=False),
    "rename": Action(ConversationStore._rename, on_conversation=True),
    "send": Action(ConversationStore._send, on_conversation=True),
    "delete": Action(ConversationStore._delete, on_conversation=True),
}
