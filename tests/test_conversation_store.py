"""Saved conversations: what a turn sends to the model (the whole history, answers without their reasoning), idempotent sends,
one turn at a time, the limits, what the browser may see, and requests of any shape answered with a sentence, never a crash.

Reference counterpart: ``tests/entrypoints/ui/test_conversations.py``."""

import pytest

from glm_tpu_b200.engine import request as rq
from glm_tpu_b200.entrypoints.serve.job_queue import PENDING, JobQueue
from glm_tpu_b200.entrypoints.ui.conversations import (AUTO_TITLE_CHARS, DEFAULT_TITLE, MAX_MESSAGE_BYTES, ConversationStore, Refused, valid_message_id,
                                                       valid_text, valid_title)
from glm_tpu_b200.exceptions import ApiError
from glm_tpu_b200.tokenizer import ByteTokenizer

PROFILE = rq.RequestProfile(vocab_size=1024, eos_ids=(1021, 1022, 1023), capacities=(4096,), prompt_limits={4096: 4096}, concurrent_capacity=4096)


class Backend:
    """Answers every turn at its second observation with "answer to: <last user text>" and some reasoning."""

    def __init__(self):
        self.capacity, self.tokenizer = 4096, ByteTokenizer(1024, PROFILE.eos_ids)
        self.prepared, self.sequence, self.polls, self.available = [], 0, {}, True

    def check(self):
        if not self.available:
            raise ValueError("The resident model is unavailable. No model was restarted.")

    def prepare(self, messages, key):
        self.prepared.append([dict(m) for m in messages])
        ids = self.tokenizer.apply_chat_template(messages)
        if len(ids) > 3000:
            raise ApiError("this conversation fills the 4096-slot context; start a new one")
        return rq.from_token_ids(ids, request_id="ui-" + key, max_new_tokens=64, context_capacity=4096, profile=PROFILE)

    def prepare_api(self, messages, key, **kw):
        ids = self.tokenizer.apply_chat_template(messages)
        return rq.from_token_ids(ids, request_id="api-" + key, max_new_tokens=8, context_capacity=4096, profile=PROFILE)

    def next_sequence(self):
        self.sequence += 1
        return self.sequence

    def publish(self, job, state):
        pass

    def observe(self, job):
        n = self.polls[job["id"]] = self.polls.get(job["id"], 0) + 1
        if n < 2:
            return {"thinking": "hm", "answer": "", "output_tokens": 1, "status": "generating"}
        return {"thinking": "hm, easy", "answer": "answer to: " + job["user_text"], "output_tokens": 9, "status": "complete", "stop_cause": "eos",
                "decode_tps": 140.0, "prefill_seconds": 0.02}


@pytest.fixture
def store(tmp_path):
    backend = Backend()
    queue = JobQueue(tmp_path / "state", backend)
    return ConversationStore(queue), queue, backend


def mid(n: int) -> str:
    return f"{n:032x}"


def finish(queue, rounds=3):
    for _ in range(rounds):
        queue.step()


def test_a_turn_sends_the_whole_history_without_the_reasoning(store):
    s, queue, backend = store
    chat = s.change({"action": "create"})["id"]
    assert s.change({"action": "send", "chat": chat, "id": mid(1), "text": "first question"}) == {"ok": True}
    finish(queue)
    assert s.change({"action": "send", "chat": chat, "id": mid(2), "text": "second question"}) == {"ok": True}
    assert backend.prepared[0] == [{"role": "user", "content": "first question"}]
    assert backend.prepared[1] == [{"role": "user", "content": "first question"}, {"role": "assistant", "content": "answer to: first question"},
                                   {"role": "user", "content": "second question"}]  # role and content only: no status, no job key, no reasoning
    finish(queue)
    conversation = s.snapshot()["chats"][0]
    assert [m["role"] for m in conversation["messages"]] == ["user", "assistant", "user", "assistant"]
    last = conversation["messages"][-1]
    assert last == {"role": "assistant", "content": "answer to: second question", "status": "complete", "job": mid(2), "thinking": "hm, easy",
                    "output_tokens": 9, "decode_tps": 140.0}
    assert conversation["title"] == "first question"  # named after its first message, once


def test_sends_are_idempotent_and_one_at_a_time(store):
    s, queue, backend = store
    chat, other = s.change({"action": "create"})["id"], s.change({"action": "create"})["id"]
    s.change({"action": "send", "chat": chat, "id": mid(1), "text": "q"})
    assert s.change({"action": "send", "chat": chat, "id": mid(1), "text": "q"}) == {"id": mid(1)} and len(backend.prepared) == 1
    for request, sentence in (({"chat": chat, "id": mid(1), "text": "another text"}, "Message identity was already used."),
                              ({"chat": other, "id": mid(1), "text": "q"}, "Message identity was already used."),
                              ({"chat": chat, "id": mid(2), "text": "too early"}, "Wait for a completed answer, or start a new conversation.")):
        with pytest.raises(Refused, match=sentence):
            s.change({"action": "send", **request})
    with pytest.raises(Refused, match="Wait for this conversation to finish"):
        s.change({"action": "delete", "chat": chat})
    assert s.change({"action": "send", "chat": other, "id": mid(3), "text": "elsewhere"}) == {"ok": True}  # another conversation may queue meanwhile
    assert queue.pending() == 2 and len(s.snapshot()["jobs"]) == 2
    finish(queue, 6)
    assert s.change({"action": "send", "chat": chat, "id": mid(1), "text": "q"}) == {"id": mid(1)}  # still the same answer after it finished
    s.change({"action": "delete", "chat": chat})
    snap = s.snapshot()
    assert [c["id"] for c in snap["chats"]] == [other] and [j["id"] for j in snap["jobs"]] == [mid(3)]  # its jobs went with it


def test_limits_and_a_halted_queue(store):
    s, queue, backend = store
    chats = [s.change({"action": "create"})["id"] for _ in range(PENDING + 1)]
    for i, chat in enumerate(chats[:PENDING]):
        s.change({"action": "send", "chat": chat, "id": mid(i), "text": f"q{i}"})
    with pytest.raises(Refused, match="Ten messages are already waiting"):
        s.change({"action": "send", "chat": chats[PENDING], "id": mid(99), "text": "one too many"})
    assert s.snapshot()["chats"][PENDING]["messages"] == []  # a refused send leaves no trace
    finish(queue, 3 * PENDING)
    long = s.change({"action": "create"})["id"]
    with pytest.raises(ApiError, match="fills the 4096-slot context"):
        s.change({"action": "send", "chat": long, "id": mid(100), "text": "x" * 3500})
    assert s.snapshot()["chats"][-1]["messages"] == [] and queue.job(mid(100)) is None
    queue.error = "Resident sequence belongs to a different request."
    with pytest.raises(Refused, match="belongs to a different request"):
        s.change({"action": "send", "chat": long, "id": mid(101), "text": "after the halt"})
    assert s.snapshot()["error"] == queue.error
    s.change({"action": "rename", "chat": long, "title": "still editable"})  # reading and tidying still work


def test_field_validators():
    assert valid_title("  A title ") == "A title" and valid_title("x" * 100) == "x" * 100
    for bad in ("", "   ", "x" * 101, None, 5, ["t"]):
        with pytest.raises(Refused, match="between 1 and 100 characters"):
            valid_title(bad)
    assert valid_message_id("0123456789abcdef" * 2) == "0123456789abcdef" * 2
    for bad in ("0123456789ABCDEF" * 2, "g" * 32, "a" * 31, "a" * 33, "", None, 7, "a" * 32 + "\n"):
        with pytest.raises(Refused, match="Invalid message identity"):
            valid_message_id(bad)
    assert valid_text(" keeps its spaces ") == " keeps its spaces " and valid_text("ü" * (MAX_MESSAGE_BYTES // 2)) is not None
    for bad in ("", " \n\t", None, 3, "ü" * (MAX_MESSAGE_BYTES // 2 + 1), "x" * (MAX_MESSAGE_BYTES + 1)):
        with pytest.raises(Refused, match="at most 128,000 bytes"):
            valid_text(bad)


def test_requests_of_any_shape_get_a_sentence(store):
    s, queue, _ = store
    chat = s.change({"action": "create"})["id"]
    for request, sentence in (({}, "Conversation not found."), ({"action": "explode"}, "Conversation not found."),
                              ({"action": "explode", "chat": chat}, "Unknown action."), ({"action": ["send"], "chat": chat}, "Unknown action."),
                              ({"action": {"a": 1}, "chat": chat}, "Unknown action."), ({"action": 5, "chat": chat}, "Unknown action."),
                              ({"action": None, "chat": chat}, "Unknown action."),
                              ({"action": "send", "chat": ["x"]}, "Conversation not found."), ({"action": "rename", "chat": None, "title": "t"}, "Conversation not found."),
                              ({"action": "send", "chat": chat, "id": "nope", "text": "t"}, "Invalid message identity."),
                              ({"action": "send", "chat": chat, "id": mid(1)}, "at most 128,000 bytes"),
                              ({"action": "send", "chat": chat, "id": mid(1), "text": ["t"]}, "at most 128,000 bytes"),
                              ({"action": "rename", "chat": chat}, "between 1 and 100"), ({"action": "rename", "chat": chat, "title": 5}, "between 1 and 100")):
        with pytest.raises(ValueError, match=sentence):  # the HTTP layer turns every ValueError into a 400 with this sentence
            s.change(request)
    snap = s.snapshot()
    assert snap["chats"] == [{"id": chat, "title": DEFAULT_TITLE, "messages": []}] and snap["jobs"] == []


def test_what_the_browser_sees(store):
    s, queue, backend = store
    chat = s.change({"action": "create"})["id"]
    s.change({"action": "send", "chat": chat, "id": mid(1), "text": "   a    question   with\n\nodd   spacing " + "and a long tail " * 10})
    queue.submit(backend.prepare_api([{"role": "user", "content": "from the api"}], "k"), "api-job", label="api")
    snap = s.snapshot()
    assert [j["id"] for j in snap["jobs"]] == [mid(1)] and all("payload" not in j for j in snap["jobs"])  # API traffic stays out of the workspace
    assert snap["model"] == "GLM-5.3" and snap["capacity"] == 4096 and snap["scheduling"] == "sequential" and snap["error"] is None
    title = snap["chats"][0]["title"]
    assert title == "a question with odd spacing and a long tail and a long "[:AUTO_TITLE_CHARS] and len(title) == AUTO_TITLE_CHARS
    snap["chats"][0]["title"] = "edited by the caller"
    assert s.snapshot()["chats"][0]["title"] == title  # a snapshot is detached from the store
    s.change({"action": "rename", "chat": chat, "title": "Named by hand"})
    finish(queue)
    assert s.snapshot()["chats"][0]["title"] == "Named by hand"
    backend.available = False
    assert s.snapshot()["error"] == "The resident model is unavailable. No model was restarted."
    reloaded = ConversationStore(JobQueue(queue.root, backend))  # the document on disk is the state: a restart shows the same
    assert reloaded.snapshot()["chats"][0]["title"] == "Named by hand" and reloaded.snapshot()["chats"][0]["messages"][1]["status"] == "complete"
