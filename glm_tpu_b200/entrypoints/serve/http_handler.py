"""The loopback HTTP surface: the browser workspace and the OpenAI-compatible ``/v1`` API.

Routes: ``GET /`` ``/app.js`` ``/style.css`` (static UI), ``GET /api/state``, ``POST /api/chat`` (needs the
``X-GLM-UI: 1`` header), ``GET /v1/models`` and ``POST /v1/chat/completions`` (need the bearer key).  Every request must
carry a loopback ``Host`` (and, if present, a matching ``Origin``): together with the 127.0.0.1 bind this stops DNS
rebinding and cross-site requests.  Responses carry a strict content-security policy and ``no-store``.  Nothing is
written to an access log: questions are private.

Parity: reference ``glm_tpu/entrypoints/serve/http_handler.py:15-155``.
"""

from __future__ import annotations

import json
import secrets
from http.server import BaseHTTPRequestHandler
from importlib import resources
from urllib.parse import urlsplit

from glm_tpu_b200.entrypoints.openai.protocol import BODY_CAP, ApiError

UI_PACKAGE = "glm_tpu_b200.entrypoints.ui"
CSP = ("default-src 'self'; script-src 'self'; style-src 'self'; img-src 'self' data:; connect-src 'self'; "
       "frame-ancestors 'none'; base-uri 'none'; form-action 'self'")
ASSETS = {"/": ("index.html", "text/html"), "/app.js": ("app.js", "text/javascript"), "/style.css": ("style.css", "text/css")}


def _api_error(message: str) -> dict:
    return {"error": {"message": message, "type": "invalid_request_error", "param": None, "code": None}}


def handler(store, chat=None, models=None, token: str | None = None):
    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *_):
            pass

        def respond(self, code, value, kind="application/json"):
            raw = json.dumps(value).encode() if kind == "application/json" else value
            self.send_response(code)
            self.send_header("Content-Type", kind + "; charset=utf-8")
            self.send_header("Content-Length", str(len(raw)))
            self.send_header("Cache-Control", "no-store")
            self.send_header("X-Content-Type-Options", "nosniff")
            self.send_header("Content-Security-Policy", CSP)
            self.end_headers()
            self.wfile.write(raw)

        def bearer(self) -> bool:
            header = self.headers.get("Authorization", "")
            offered = header[7:] if header.startswith("Bearer ") else ""
            return token is not None and secrets.compare_digest(offered, token)

        def allowed(self) -> bool:
            host = self.headers.get("Host", "")
            port = self.server.server_port
            origin = self.headers.get("Origin")
            return host in {f"127.0.0.1:{port}", f"localhost:{port}"} and (origin is None or origin == "http://" + host)

        def body(self, cap: int, timeout: float):
            size = int(self.headers.get("Content-Length", "0"))
            if not 0 < size <= cap:
                raise ApiError("request body is empty or too large")
            self.connection.settimeout(timeout)
            return json.loads(self.rfile.read(size))

        def stream(self, source):
            try:
                first = next(source)
            except ApiError as exc:
                return self.respond(exc.status, exc.body())
            except StopIteration:
                return self.respond(500, _api_error("empty stream"))
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream; charset=utf-8")
            self.send_header("Cache-Control", "no-store")
            self.send_header("X-Content-Type-Options", "nosniff")
            self.end_headers()
            try:
                self.wfile.write(first)
                self.wfile.flush()
                for chunk in source:
                    self.wfile.write(chunk)
                    self.wfile.flush()
            except ApiError as exc:  # headers are out: report in-band and end the stream
                self.wfile.write(b"data: " + json.dumps(exc.body()).encode() + b"\n\n" + b"data: [DONE]\n\n")
                self.wfile.flush()
            except (BrokenPipeError, ConnectionResetError):
                pass  # the client left; the admitted request still finishes

        def do_GET(self):
            if not self.allowed():
                return self.respond(403, {"error": "Local origin required."})
            path = urlsplit(self.path).path
            if path.startswith("/v1/"):
                if not self.bearer():
                    return self.respond(401, _api_error("A local API key is required."))
                if path != "/v1/models" or models is None:
                    return self.respond(404, _api_error("Not found."))
                return self.respond(200, models.models())
            if path == "/api/state":
                return self.respond(200, store.snapshot())
            if path not in ASSETS:
                return self.respond(404, {"error": "Not found."})
            name, kind = ASSETS[path]
            self.respond(200, resources.files(UI_PACKAGE).joinpath("static", name).read_bytes(), kind)

        def do_POST(self):
            path = urlsplit(self.path).path
            if path.startswith("/v1/"):
                return self.completions(path)
            if not self.allowed() or self.headers.get("X-GLM-UI") != "1":
                return self.respond(403, {"error": "Local UI required."})
            if path != "/api/chat":
                return self.respond(404, {"error": "Not found."})
            try:
                data = self.body(256000, 10)
                if type(data) is not dict:
                    raise ValueError("Expected an object.")
                result = store.change(data)
            except (ValueError, OSError) as exc:
                return self.respond(400, {"error": str(exc)})
            self.respond(200, result)

        def completions(self, path):
            if not self.allowed():
                return self.respond(403, _api_error("Local origin required."))
            if not self.bearer():
                return self.respond(401, _api_error("A local API key is required."))
            if path != "/v1/chat/completions" or chat is None:
                return self.respond(404, _api_error("Not found."))
            try:
                data = self.body(BODY_CAP, 30)
            except ApiError as exc:
                return self.respond(exc.status, exc.body())
            except (ValueError, OSError) as exc:
                return self.respond(400, _api_error(str(exc)))
            self.connection.settimeout(None)
            if type(data) is dict and data.get("stream"):
                return self.stream(chat.stream(data))
            try:
                return self.respond(200, chat.completion(data))
            except ApiError as exc:
                return self.respond(exc.status, exc.body())
            except (ValueError, OSError) as exc:
                return self.respond(400, _api_error(str(exc)))

    return Handler
