"""The gates of the loopback surface with raw requests: headers a browser or ``urllib`` would never send (bytes above ASCII in the
key, a Content-Length that is not a number, a body larger than its cap), every route with and without its credentials, and what
every reply carries.

Reference counterpart: ``tests/entrypoints/serve/test_http_handler.py``."""

import http.client
import json
import threading
from http.server import ThreadingHTTPServer

import pytest

from glm_tpu_b200.entrypoints.openai.protocol import BODY_CAP, ApiError
from glm_tpu_b200.entrypoints.serve import http_handler
from glm_tpu_b200.entrypoints.serve.http_handler import UI_BODY_CAP, handler

TOKEN = "k" * 43


class Store:
    def __init__(self):
        self.changes = []

    def snapshot(self):
        return {"conversations": [], "queue": 0}

    def change(self, change):
        if change.get("action") == "boom":
            raise ValueError("Unknown action.")
        self.changes.append(change)
        return {"ok": True}


class Chat:
    def completion(self, request):
        if not isinstance(request, dict) or "messages" not in request:
            raise ApiError("messages must be a non-empty array")
        if request.get("model") == "other":
            raise ApiError("The model does not exist.", status=404, kind="not_found_error")
        return {"id": "chatcmpl-1", "choices": [{"message": {"role": "assistant", "content": "Four."}}]}

    def stream(self, request):
        if request.get("model") == "other":
            raise ApiError("The model does not exist.", status=404, kind="not_found_error")
        yield b'data: {"n": 1}\n\n'
        if request.get("fail_late"):
            raise ApiError("The resident model is unavailable.", status=503, kind="server_error")
        yield b'data: {"n": 2}\n\n'
        yield http_handler.SSE_DONE


class Models:
    def models(self):
        return {"object": "list", "data": [{"id": "glm-5.3"}]}


@pytest.fixture
def server():
    store = Store()
    srv = ThreadingHTTPServer(("127.0.0.1", 0), handler(store, Chat(), Models(), TOKEN))
    thread = threading.Thread(target=srv.serve_forever, daemon=True)
    thread.start()
    yield srv.server_port, store
    srv.shutdown()
    srv.server_close()


def request(port, method, path, *, headers=None, body=None, host=None):
    conn = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    try:
        conn.putrequest(method, path, skip_host=True, skip_accept_encoding=True)
        conn.putheader("Host", host if host is not None else f"127.0.0.1:{port}")
        for name, value in (headers or {}).items():
            conn.putheader(name, value)
        if body is not None and "Content-Length" not in (headers or {}):
            conn.putheader("Content-Length", str(len(body)))
        conn.endheaders(body)
        reply = conn.getresponse()
        return reply.status, reply.read(), {k.lower(): v for k, v in reply.getheaders()}
    finally:
        conn.close()


KEY = {"Authorization": "Bearer " + TOKEN}
UI = {"X-GLM-UI": "1"}


def test_every_reply_is_closed_to_caches_sniffing_and_framing(server):
    port, _ = server
    for method, path, headers, body in (("GET", "/", {}, None), ("GET", "/api/state", {}, None), ("GET", "/nothing", {}, None),
                                        ("GET", "/v1/models", KEY, None), ("GET", "/v1/models", {}, None),
                                        ("POST", "/api/chat", UI, b'{"action": "x"}'), ("POST", "/v1/chat/completions", KEY, b'{"messages": []}')):
        status, _, reply = request(port, method, path, headers=headers, body=body)
        assert reply["cache-control"] == "no-store" and reply["x-content-type-options"] == "nosniff", (path, status)
        assert "frame-ancestors 'none'" in reply["content-security-policy"] and "default-src 'self'" in reply["content-security-policy"]
        assert reply["content-type"].endswith("charset=utf-8")


def test_the_host_and_origin_gate(server):
    port, _ = server
    assert request(port, "GET", "/api/state")[0] == 200
    assert request(port, "GET", "/api/state", host=f"localhost:{port}")[0] == 200
    for host in ("evil.example", f"evil.example:{port}", "127.0.0.1", f"127.0.0.1:{port + 1}", f"127.0.0.1:{port}.evil.example", ""):
        status, body, _ = request(port, "GET", "/api/state", host=host)
        assert status == 403 and json.loads(body) == {"error": "Local origin required."}, host
    assert request(port, "GET", "/api/state", headers={"Origin": f"http://127.0.0.1:{port}"})[0] == 200
    for origin in ("http://evil.example", f"https://127.0.0.1:{port}", f"http://localhost:{port}", "null"):
        assert request(port, "GET", "/api/state", headers={"Origin": origin})[0] == 403, origin  # the origin must be the very host that was named
    assert request(port, "POST", "/api/chat", headers=UI, body=b"{}", host="evil.example")[0] == 403
    assert request(port, "POST", "/v1/chat/completions", headers=KEY, body=b"{}", host="evil.example")[0] == 403
    assert request(port, "GET", "/v1/models", headers=KEY, host="evil.example")[0] == 403


def test_the_workspace_needs_the_header_a_form_cannot_set(server):
    port, store = server
    assert request(port, "POST", "/api/chat", body=b'{"action": "new"}')[0] == 403
    assert request(port, "POST", "/api/chat", headers={"X-GLM-UI": "true"}, body=b'{"action": "new"}')[0] == 403
    status, body, _ = request(port, "POST", "/api/chat", headers=UI, body=b'{"action": "new"}')
    assert status == 200 and json.loads(body) == {"ok": True} and store.changes == [{"action": "new"}]
    assert request(port, "POST", "/api/other", headers=UI, body=b"{}")[0] == 404
    for body, sentence in ((b"[1]", "Expected an object."), (b"{broken", None), (b'{"action": "boom"}', "Unknown action.")):
        status, reply, _ = request(port, "POST", "/api/chat", headers=UI, body=body)
        assert status == 400 and (sentence is None or json.loads(reply) == {"error": sentence})
    assert len(store.changes) == 1


def test_the_api_needs_the_key(server):
    port, _ = server
    status, body, _ = request(port, "GET", "/v1/models")
    assert status == 401 and json.loads(body)["error"] == {"message": "A local API key is required.", "type": "invalid_request_error", "param": None, "code": None}
    for offered in ("Bearer", "Bearer ", "Bearer wrong", "bearer " + TOKEN, "Basic " + TOKEN, TOKEN, "Bearer " + TOKEN + "x", "Bearer " + TOKEN[:-1],
                    "Bearer  " + TOKEN):
        assert request(port, "GET", "/v1/models", headers={"Authorization": offered})[0] == 401, offered
    # bytes above ASCII in the offered key are an answer (401), not an exception in the comparison
    assert request(port, "GET", "/v1/models", headers={"Authorization": "Bearer sch\xfcssel"})[0] == 401
    assert request(port, "POST", "/v1/chat/completions", headers={"Authorization": "Bearer \xff\xfe"}, body=b"{}")[0] == 401
    status, body, _ = request(port, "GET", "/v1/models", headers=KEY)
    assert status == 200 and json.loads(body)["data"][0]["id"] == "glm-5.3"
    assert request(port, "GET", "/v1/other", headers=KEY)[0] == 404 and request(port, "POST", "/v1/other", headers=KEY, body=b"{}")[0] == 404
    # the UI header is no substitute for the key, and the key none for the UI header
    assert request(port, "POST", "/v1/chat/completions", headers=UI, body=b"{}")[0] == 401
    assert request(port, "POST", "/api/chat", headers=KEY, body=b"{}")[0] == 403


def test_a_server_without_api(server):
    store = Store()
    srv = ThreadingHTTPServer(("127.0.0.1", 0), handler(store))  # --no-api: no chat, no models, no key
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        port = srv.server_port
        assert request(port, "GET", "/api/state")[0] == 200
        assert request(port, "GET", "/v1/models", headers=KEY)[0] == 401  # there is no key that opens it
        assert request(port, "POST", "/v1/chat/completions", headers=KEY, body=b"{}")[0] == 401
    finally:
        srv.shutdown()
        srv.server_close()


def test_bodies_are_measured_before_they_are_read(server):
    port, store = server
    for length in ("0", "-5", "abc", str(UI_BODY_CAP + 1), ""):
        status, _, _ = request(port, "POST", "/api/chat", headers=dict(UI, **{"Content-Length": length}), body=b"")
        assert status == 400, length
    status, body, _ = request(port, "POST", "/v1/chat/completions", headers=dict(KEY, **{"Content-Length": str(BODY_CAP + 1)}), body=b"")
    assert status == 400 and "empty or too large" in json.loads(body)["error"]["message"]
    assert request(port, "POST", "/v1/chat/completions", headers=dict(KEY, **{"Content-Length": "nope"}), body=b"")[0] == 400
    assert request(port, "POST", "/v1/chat/completions", headers=KEY, body=b"{broken")[0] == 400
    assert store.changes == []
    big = json.dumps({"action": "new", "pad": "x" * (UI_BODY_CAP - 40)}).encode()
    assert len(big) <= UI_BODY_CAP and request(port, "POST", "/api/chat", headers=UI, body=big)[0] == 200  # right up to the cap is fine


def test_completions_and_their_refusals(server):
    port, _ = server
    status, body, _ = request(port, "POST", "/v1/chat/completions", headers=KEY, body=b'{"messages": [{"role": "user", "content": "2+2?"}]}')
    assert status == 200 and json.loads(body)["choices"][0]["message"]["content"] == "Four."
    status, body, _ = request(port, "POST", "/v1/chat/completions", headers=KEY, body=b'{"model": "other", "messages": []}')
    assert status == 404 and json.loads(body)["error"]["type"] == "not_found_error"
    status, body, _ = request(port, "POST", "/v1/chat/completions", headers=KEY, body=b"[]")
    assert status == 400 and json.loads(body)["error"]["message"] == "messages must be a non-empty array"


def test_streams(server):
    port, _ = server
    status, body, reply = request(port, "POST", "/v1/chat/completions", headers=KEY, body=b'{"stream": true, "messages": []}')
    assert status == 200 and reply["content-type"] == "text/event-stream; charset=utf-8" and reply["cache-control"] == "no-store"
    assert body == b'data: {"n": 1}\n\ndata: {"n": 2}\n\ndata: [DONE]\n\n'
    # a refusal before the first event still gets its own status; one after it travels in the stream, which then ends properly
    status, body, reply = request(port, "POST", "/v1/chat/completions", headers=KEY, body=b'{"stream": true, "model": "other", "messages": []}')
    assert status == 404 and reply["content-type"].startswith("application/json") and json.loads(body)["error"]["type"] == "not_found_error"
    status, body, _ = request(port, "POST", "/v1/chat/completions", headers=KEY, body=b'{"stream": true, "fail_late": true, "messages": []}')
    events = body.split(b"\n\n")
    assert status == 200 and events[0] == b'data: {"n": 1}' and json.loads(events[1][6:])["error"]["type"] == "server_error" and events[2] == b"data: [DONE]"


def test_other_methods_and_static_paths(server):
    port, _ = server
    for method in ("PUT", "DELETE", "PATCH", "OPTIONS"):
        assert request(port, method, "/api/chat", headers=UI, body=b"{}")[0] == 501  # not implemented, for anybody
    for path in ("/static/index.html", "/../etc/passwd", "/app.js/", "/index.html", "/%2e%2e/x"):
        assert request(port, "GET", path)[0] == 404, path  # the workspace is three named files, not a directory
    status, body, reply = request(port, "GET", "/?next=/v1/models")
    assert status == 200 and reply["content-type"].startswith("text/html")  # a query string does not change the route
