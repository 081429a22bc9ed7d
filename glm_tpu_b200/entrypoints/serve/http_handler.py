"""The loopback HTTP surface: the browser workspace and the OpenAI-compatible ``/v1`` API.

``handler(store, chat, models, token)`` binds the four collaborators to a subclass of ``LoopbackSurface``.  A request passes three stages:

1. *gate*: the ``Host`` header must name this server on ``127.0.0.1`` or ``localhost`` and an ``Origin``, when present, must be that same
   host (with the loopback bind this stops DNS rebinding and cross-site requests); ``/v1`` additionally needs the bearer key, the
   workspace's ``POST`` the ``X-GLM-UI: 1`` header that a cross-site form cannot set;
2. *route*: two small tables, ``UI_PAGES`` for the static workspace and the methods ``_api_get`` / ``_api_post`` / ``_ui_get`` /
   ``_ui_post`` for everything else;
3. *reply*: JSON or a static asset with ``no-store``, ``nosniff`` and a strict content-security policy, or a server-sent-event stream.

Nothing is written to an access log: questions are private.  Bodies are size-capped before they are read.

Behaviour parity: reference ``glm_tpu/entrypoints/serve/http_handler.py`` (same routes, status codes and sentences).
"""

from __future__ import annotations

import json
import secrets
from http.server import BaseHTTPRequestHandler
from importlib import resources
from urllib.parse import urlsplit

from glm_tpu_b200.entrypoints.openai.protocol import BODY_CAP, ApiError

UI_PACKAGE = "glm_tpu_b200.entrypoints.ui"
UI_PAGES = {"/": ("index.html", "text/html"), "/app.js": ("app.js", "text/javascript"), "/style.css": ("style.css", "text/css")}
UI_BODY_CAP, UI_READ_SECONDS, API_READ_SECONDS = 256000, 10, 30
SECURITY_HEADERS = (
    ("Cache-Control", "no-store"),
    ("X-Content-Type-Options", "nosniff"),
    ("Content-Security-Policy", "default-src 'self'; script-src 'self'; style-src 'self'; img-src 'self' data:; connect-src 'self'; "
                                "frame-ancestors 'none'; base-uri 'none'; form-action 'self'"),
)
SSE_DONE = b"data: [DONE]\n\n"


def _api_problem(sentence: str) -> dict:
    return {"error": {"message": sentence, "type": "invalid_request_error", "param": None, "code": None}}


class LoopbackSurface(BaseHTTPRequestHandler):
    """One request; ``store``, ``chat``, ``models`` and ``token`` are class attributes set by :func:`handler`."""

    store = chat = models = token = None

    def log_message(self, *_):  # no access log
        return

    # ------------------------------------------------------------------------------------------------------------------ replies
    def _reply(self, status: int, payload: bytes, content_type: str) -> None:
        self.send_response(status)
        self.send_header("Content-Type", content_type + "; charset=utf-8")
        self.send_header("Content-Length", str(len(payload)))
        for name, value in SECURITY_HEADERS:
            self.send_header(name, value)
        self.end_headers()
        self.wfile.write(payload)

    def _reply_json(self, status: int, value) -> None:
        self._reply(status, json.dumps(value).encode(), "application/json")

    def _refuse_ui(self, status: int, sentence: str) -> None:
        self._reply_json(status, {"error": sentence})

    def _refuse_api(self, status: int, sentence: str) -> None:
        self._reply_json(status, _api_problem(sentence))

    def _reply_events(self, events) -> None:
        """A server-sent-event stream.  The first event is produced before the status line, so a refusal still gets its own status."""
        try:
            head = next(events)
        except ApiError as refusal:
            return self._reply_json(refusal.status, refusal.body())
        except StopIteration:
            return self._refuse_api(500, "empty stream")
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream; charset=utf-8")
        for name, value in SECURITY_HEADERS[:2]:
            self.send_header(name, value)
        self.end_headers()
        try:
            self._push(head)
            for event in events:
                self._push(event)
        except ApiError as refusal:  # the status line is out: the error travels in-band and the stream ends properly
            self._push(b"data: " + json.dumps(refusal.body()).encode() + b"\n\n" + SSE_DONE)
        except (BrokenPipeError, ConnectionResetError):
            return  # the client left; the admitted request still runs to its end

    def _push(self, chunk: bytes) -> None:
        self.wfile.write(chunk)
        self.wfile.flush()

    # ------------------------------------------------------------------------------------------------------------------ gates
    def _from_this_machine(self) -> bool:
        port = self.server.server_port
        host = self.headers.get("Host", "")
        if host not in (f"127.0.0.1:{port}", f"localhost:{port}"):
            return False
        origin = self.headers.get("Origin")
        return origin is None or origin == f"http://{host}"

    def _holds_key(self) -> bool:
        if self.token is None:
            return False
        scheme, _, offered = self.headers.get("Authorization", "").partition(" ")
        # compared as bytes: header text may carry any byte (http.server decodes it as latin-1), and the str form of the
        # constant-time comparison refuses non-ASCII text with an exception instead of an answer
        return scheme == "Bearer" and secrets.compare_digest(offered.encode("latin-1", "replace"), self.token.encode("utf-8"))

    def _json_body(self, cap: int, seconds: float):
        declared = int(self.headers.get("Content-Length", "0"))
        if declared <= 0 or declared > cap:
            raise ApiError("request body is empty or too large")
        self.connection.settimeout(seconds)
        return json.loads(self.rfile.read(declared))

    # ------------------------------------------------------------------------------------------------------------------ routes
    def do_GET(self):
        path = urlsplit(self.path).path
        if not self._from_this_machine():
            return self._refuse_ui(403, "Local origin required.")
        return self._api_get(path) if path.startswith("/v1/") else self._ui_get(path)

    def do_POST(self):
        path = urlsplit(self.path).path
        return self._api_post(path) if path.startswith("/v1/") else self._ui_post(path)

    def _ui_get(self, path: str):
        if path == "/api/state":
            return self._reply_json(200, self.store.snapshot())
        page = UI_PAGES.get(path)
        if page is None:
            return self._refuse_ui(404, "Not found.")
        file_name, content_type = page
        self._reply(200, resources.files(UI_PACKAGE).joinpath("static", file_name).read_bytes(), content_type)

    def _ui_post(self, path: str):
        if not self._from_this_machine() or self.headers.get("X-GLM-UI") != "1":
            return self._refuse_ui(403, "Local UI required.")
        if path != "/api/chat":
            return self._refuse_ui(404, "Not found.")
        try:
            change = self._json_body(UI_BODY_CAP, UI_READ_SECONDS)
            if not isinstance(change, dict):
                raise ValueError("Expected an object.")
            outcome = self.store.change(change)
        except (ValueError, OSError) as problem:  # ApiError is a ValueError: a bad size reads the same as bad JSON here
            return self._refuse_ui(400, str(problem))
        self._reply_json(200, outcome)

    def _api_get(self, path: str):
        if not self._holds_key():
            return self._refuse_api(401, "A local API key is required.")
        if path == "/v1/models" and self.models is not None:
            return self._reply_json(200, self.models.models())
        self._refuse_api(404, "Not found.")

    def _api_post(self, path: str):
        if not self._from_this_machine():
            return self._refuse_api(403, "Local origin required.")
        if not self._holds_key():
            return self._refuse_api(401, "A local API key is required.")
        if path != "/v1/chat/completions" or self.chat is None:
            return self._refuse_api(404, "Not found.")
        streaming = False
        try:
            request = self._json_body(BODY_CAP, API_READ_SECONDS)
            self.connection.settimeout(None)  # generation may take as long as its own deadline allows
            streaming = isinstance(request, dict) and bool(request.get("stream"))
            if not streaming:
                self._reply_json(200, self.chat.completion(request))
        except ApiError as refusal:
            return self._reply_json(refusal.status, refusal.body())
        except (ValueError, OSError) as problem:
            return self._refuse_api(400, str(problem))
        if streaming:  # outside the handlers above: once events flow, a refusal can only travel in-band
            self._reply_events(self.chat.stream(request))


def handler(store, chat=None, models=None, token: str | None = None):
    """The request-handler class for ``http.server``: ``LoopbackSurface`` bound to this workspace, API and key."""
    return type("BoundLoopbackSurface", (LoopbackSurface,), {"store": store, "chat": chat, "models": models, "token": token})
