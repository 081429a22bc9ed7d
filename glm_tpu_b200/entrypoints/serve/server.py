"""Loopback chat UI and OpenAI-compatible API attached to an EXISTING resident session.

    python -m glm_tpu_b200.entrypoints.serve.server --run RUN_DIR --state STATE_DIR [--port 8011] [--no-api]

This process never touches a GPU, never starts workers and never sends a stop command: closing it leaves the model
loaded.  Chat history, prepared requests and the API key live in ``--state`` (owner-only, outside the checkout).

Parity: reference ``glm_tpu/entrypoints/serve/server.py:22-76``.
"""

from __future__ import annotations

import argparse
import json
import os
import threading
from http.server import ThreadingHTTPServer
from pathlib import Path

from glm_tpu_b200.engine import resident_protocol as proto
from glm_tpu_b200.engine.resident_client import Resident
from glm_tpu_b200.entrypoints.openai.serving_chat import OpenAIServingChat
from glm_tpu_b200.entrypoints.openai.serving_models import OpenAIServingModels
from glm_tpu_b200.entrypoints.serve.http_handler import handler
from glm_tpu_b200.entrypoints.serve.job_queue import JobQueue
from glm_tpu_b200.entrypoints.serve.security import api_token
from glm_tpu_b200.entrypoints.ui.conversations import ConversationStore

REPO = Path(__file__).resolve().parents[3]


def resident_for_run(run: Path) -> Resident:
    """Build the client from what the controller and rank 0 recorded in the run directory."""
    from glm_tpu_b200.tokenizer import load_tokenizer
    from glm_tpu_b200.worker.gpu_worker import profile_for, resolve_model

    ident = json.loads((run / proto.CONTROLLER_IDENTITY_FILE).read_text())
    args = ident.get("args", {})
    geometry, (kind, path) = resolve_model(args.get("model", "random:tiny"))
    record = run / proto.runner_file(0)
    capacity = json.loads(record.read_text())["context_capacity"] if record.exists() else (args.get("context") or 8192)
    tokenizer = load_tokenizer(path if kind == "checkpoint" else None, vocab_size=geometry.vocab_size, eos_ids=geometry.eos_ids)
    return Resident(run, tokenizer, profile_for(geometry, capacity), capacity=capacity, world=int(args.get("gpus", 1)))


class ProducerBusy(ValueError):
    pass


def hold_producer_lock(run: Path):
    """The one lock of a resident session's inbox (``inbox/producer.lock``, ``flock``, non-blocking).  Sequence numbers are claimed
    by reading the ready file and the inbox; two servers doing that at once could publish two requests under one number, so the
    second server is refused.  The returned descriptor holds the lock until it is closed or the process ends."""
    import fcntl

    inbox = run / proto.INBOX_DIR
    if not inbox.is_dir():
        raise ProducerBusy(f"{run} is not the run directory of a resident session (no inbox)")
    descriptor = os.open(inbox / proto.PRODUCER_LOCK, os.O_RDWR | os.O_CREAT | os.O_NOFOLLOW, 0o600)
    try:
        fcntl.flock(descriptor, fcntl.LOCK_EX | fcntl.LOCK_NB)
    except BlockingIOError:
        os.close(descriptor)
        raise ProducerBusy("another server already feeds this resident session; one producer per session") from None
    os.ftruncate(descriptor, 0)
    os.write(descriptor, f"{os.getpid()}\n".encode())
    return descriptor


def build(run: Path, state: Path, *, port: int, api: bool = True, api_key_file: Path | None = None, wait_seconds: float = 1800):
    backend = resident_for_run(run)
    queue = JobQueue(state, backend)
    store = ConversationStore(queue)
    chat = models = token = None
    if api:
        token = api_token(api_key_file or (state / "api-key"))
        chat = OpenAIServingChat(queue, backend, capacity=backend.capacity, wait_seconds=wait_seconds)
        models = OpenAIServingModels(capacity=backend.capacity, wait_seconds=wait_seconds, max_new=backend.profile.max_new)
    server = ThreadingHTTPServer(("127.0.0.1", port), handler(store, chat, models, token))
    return server, queue, token


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--run", type=Path, required=True)
    ap.add_argument("--state", type=Path, required=True)
    ap.add_argument("--port", type=int, default=8011)
    ap.add_argument("--api-key-file", type=Path)
    ap.add_argument("--no-api", action="store_true")
    args = ap.parse_args(argv)
    os.umask(0o077)
    if args.state.resolve().is_relative_to(REPO):
        ap.error("Private chat state must be outside the source checkout.")
    if args.api_key_file is None:  # command line > GLM_B200_API_KEY_FILE > <state>/api-key
        from glm_tpu_b200 import envs

        args.api_key_file = envs.GLM_B200_API_KEY_FILE
    try:
        producer = hold_producer_lock(args.run.resolve())
    except ProducerBusy as refusal:
        ap.error(str(refusal))
    server, queue, token = build(args.run.resolve(), args.state, port=args.port, api=not args.no_api, api_key_file=args.api_key_file)
    worker = threading.Thread(target=queue.work, daemon=True)
    worker.start()
    print(f"chat: http://127.0.0.1:{server.server_port} (existing model retained)", flush=True)
    if token is not None:
        print(f"OpenAI-compatible API: http://127.0.0.1:{server.server_port}/v1 (key in {args.api_key_file or args.state / 'api-key'})", flush=True)
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        queue.stopping.set()
        worker.join(timeout=5)
        server.server_close()
        os.close(producer)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
