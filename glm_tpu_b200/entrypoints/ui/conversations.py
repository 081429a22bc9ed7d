"""Saved conversations of the loopback chat workspace, stored in the job queue's document.

Actions (``POST /api/chat``): ``create``, ``rename``, ``send`` (idempotent by a client-generated 32-hex message id; one
turn at a time per conversation; at most ten waiting jobs overall), ``delete`` (refused while a turn is running).
``snapshot`` is what ``GET /api/state`` returns: conversations, non-API jobs without their private payloads, the
session's availability, capacity and scheduling mode.

Parity: reference ``glm_tpu/entrypoints/ui/conversations.py:16-119``.
"""

from __future__ import annotations

import json
import re
import uuid

from glm_tpu_b200.entrypoints.serve.job_queue import ACTIVE, PENDING

_MESSAGE_ID = re.compile("[a-f0-9]{32}")
MAX_MESSAGE_BYTES = 128000
DEFAULT_TITLE = "New conversation"


class ConversationStore:
    def __init__(self, queue, model_name: str = "GLM-5.3"):
        self.queue = queue
        self.model_name = model_name
        queue.conversations = self

    def snapshot(self) -> dict:
        q = self.queue
        with q.mutex:
            availability = q.error
            try:
                q.backend.check()
            except (ValueError, OSError) as exc:
                availability = str(exc)
            jobs = [{k: v for k, v in j.items() if k != "payload"} for j in q.db["jobs"] if not j.get("api")]
            return json.loads(json.dumps({"chats": q.db["chats"], "jobs": jobs, "error": availability, "model": self.model_name,
                                          "capacity": q.backend.capacity, "scheduling": "sequential"}))

    def _chat(self, chat_id):
        chat = next((c for c in self.queue.db["chats"] if c["id"] == chat_id), None)
        if chat is None:
            raise ValueError("Conversation not found.")
        return chat

    def change(self, data: dict) -> dict:
        q = self.queue
        with q.mutex:
            action = data.get("action")
            if action == "create":
                chat = {"id": uuid.uuid4().hex, "title": DEFAULT_TITLE, "messages": []}
                q.db["chats"].append(chat)
                q.save()
                return {"id": chat["id"]}
            chat = self._chat(data.get("chat"))
            if action == "rename":
                title = data.get("title")
                if type(title) is not str or not 1 <= len(title.strip()) <= 100:
                    raise ValueError("Use a title between 1 and 100 characters.")
                chat["title"] = title.strip()
            elif action == "send":
                result = self._send(chat, data.get("id"), data.get("text"))
                if result is not None:
                    return result
            elif action == "delete":
                if any(j["chat"] == chat["id"] and j["status"] in ACTIVE for j in q.db["jobs"]):
                    raise ValueError("Wait for this conversation to finish before deleting it.")
                q.db["chats"].remove(chat)
                q.db["jobs"] = [j for j in q.db["jobs"] if j["chat"] != chat["id"]]
            else:
                raise ValueError("Unknown action.")
            q.save()
            return {"ok": True}

    def _send(self, chat: dict, key, text):
        q = self.queue
        if type(key) is not str or not _MESSAGE_ID.fullmatch(key):
            raise ValueError("Invalid message identity.")
        existing = next((j for j in q.db["jobs"] if j["id"] == key), None)
        if existing:
            if existing["chat"] != chat["id"] or existing["user_text"] != text:
                raise ValueError("Message identity was already used.")
            return {"id": key}
        if type(text) is not str or not text.strip() or len(text.encode()) > MAX_MESSAGE_BYTES:
            raise ValueError("Enter a message of at most 128,000 bytes.")
        if q.error:
            raise ValueError(q.error)
        if q.pending() >= PENDING:
            raise ValueError("Ten messages are already waiting. Wait for an answer.")
        if chat["messages"] and chat["messages"][-1].get("status") != "complete":
            raise ValueError("Wait for a completed answer, or start a new conversation.")
        messages = [{"role": m["role"], "content": m["content"]} for m in chat["messages"]]
        messages.append({"role": "user", "content": text})
        payload = q.backend.prepare(messages, key)
        q.db["jobs"].append(q.new_job(key, payload, chat=chat["id"], label="ui", user_text=text))
        chat["messages"] += [{"role": "user", "content": text}, {"role": "assistant", "content": "", "status": "queued", "job": key}]
        if len(chat["messages"]) == 2 and chat["title"] == DEFAULT_TITLE:
            chat["title"] = " ".join(text.split())[:55]
        return None

    def update_message(self, job: dict) -> None:
        chat = next(c for c in self.queue.db["chats"] if c["id"] == job["chat"])
        message = next(m for m in chat["messages"] if m.get("job") == job["id"])
        message.update(content=job["answer"], status=job["status"])
        for extra in ("thinking", "output_tokens", "decode_tps"):
            if extra in job:
                message[extra] = job[extra]
