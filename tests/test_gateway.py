"""The C++ gateway against fake engines: hybrid proxying with SSE pass-through, the two-phase PD forward with
/pd/free, the finished-in-prefill shortcut, 502 on upstream failure, model aliases, and control-plane discovery."""
import json
import os
import socket
import subprocess
import threading
import time
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GATEWAY = os.environ.get("NE_GATEWAY_BIN") or os.path.join(ROOT, "nanoengine_b200", "_native", "ne-gateway")      # the variable lets the sanitizer run reuse these tests


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class FakeEngine:
    def __init__(self, role, finish_in_prefill=False):
        self.role, self.finish_in_prefill = role, finish_in_prefill
        self.requests, self.freed = [], []
        eng = self

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
                eng.requests.append((self.path, body))
                if self.path == "/pd/free":
                    eng.freed.append(body.get("seq_id"))
                    return self._json({"freed": 1})
                if self.path == "/list_entities":
                    return self._json({"entities": eng.entities})
                kv = body.get("kv_transfer_params") or {}
                if eng.role == "prefill" and kv.get("do_remote_decode"):
                    assert body.get("stream") is False
                    if eng.finish_in_prefill:
                        return self._json({"id": "x", "choices": [{"index": 0, "message": {"role": "assistant", "content": "done"}}]})
                    return self._json({"id": "x", "choices": [], "kv_transfer_params": {"migration": "beef", "seq_id": 41, "first_token": 7}})
                if body.get("stream"):
                    self.send_response(200)
                    self.send_header("Content-Type", "text/event-stream")
                    self.end_headers()
                    for i in range(3):
                        self.wfile.write(f"data: {json.dumps({'tok': i, 'role': eng.role, 'first': kv.get('first_token')})}\n\n".encode())
                        self.wfile.flush()
                    self.wfile.write(b"data: [DONE]\n\n")
                    return
                return self._json({"id": "y", "role": eng.role, "model": body.get("model"), "got_migration": kv.get("migration")})

            def _json(self, obj):
                b = json.dumps(obj).encode()
                self.send_response(200)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(b)))
                self.end_headers()
                self.wfile.write(b)

        self.entities = []
        self.port = _port()
        self.srv = ThreadingHTTPServer(("127.0.0.1", self.port), H)
        threading.Thread(target=self.srv.serve_forever, daemon=True).start()
        self.url = f"http://127.0.0.1:{self.port}"

    def stop(self):
        self.srv.shutdown()


def _gateway(*args):
    port = _port()
    p = subprocess.Popen([GATEWAY, "--port", str(port), "--host", "127.0.0.1", *args], stderr=subprocess.DEVNULL)
    for _ in range(100):
        try:
            socket.create_connection(("127.0.0.1", port), timeout=0.2).close()
            break
        except OSError:
            time.sleep(0.05)
    return p, f"http://127.0.0.1:{port}"


def _post(url, body, timeout=10):
    req = urllib.request.Request(url, json.dumps(body).encode(), {"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.status, r.read()
    except urllib.error.HTTPError as e:
        return e.code, e.read()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_hybrid_proxy_stream_and_alias():
    e = FakeEngine("hybrid")
    p, gw = _gateway("--hybrid", e.url, "--model-alias", "short=long-model-name")
    try:
        st, body = _post(gw + "/v1/chat/completions", {"model": "short", "messages": []})
        assert st == 200 and json.loads(body)["model"] == "long-model-name"
        st, body = _post(gw + "/v1/completions", {"prompt": "x", "stream": True})
        assert st == 200 and body.count(b"data: ") == 4 and body.rstrip().endswith(b"[DONE]")
        assert json.loads(urllib.request.urlopen(gw + "/health").read())["engines"] == 1
        assert _post(gw + "/nope", {})[0] == 404
    finally:
        p.terminate(); e.stop()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_pd_forward_frees_prefill_and_passes_first_token():
    pf, dc = FakeEngine("prefill"), FakeEngine("decode")
    p, gw = _gateway("--prefill", pf.url, "--decode", dc.url)
    try:
        st, body = _post(gw + "/v1/chat/completions", {"messages": [], "stream": True, "max_tokens": 5})
        assert st == 200 and b'"first": 7' in body and b'"role": "decode"' in body
        path, dbody = dc.requests[-1]
        assert dbody["kv_transfer_params"] == {"migration": "beef", "seq_id": 41, "first_token": 7} and dbody["stream"] is True
        for _ in range(50):
            if pf.freed:
                break
            time.sleep(0.05)
        assert pf.freed == [41]
        st, body = _post(gw + "/v1/completions", {"prompt": "x"})
        assert json.loads(body)["got_migration"] == "beef"
    finally:
        p.terminate(); pf.stop(); dc.stop()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_pd_request_finished_in_prefill_and_upstream_failure():
    pf, dc = FakeEngine("prefill", finish_in_prefill=True), FakeEngine("decode")
    p, gw = _gateway("--prefill", pf.url, "--decode", dc.url)
    try:
        st, body = _post(gw + "/v1/chat/completions", {"messages": [], "stream": True})
        assert st == 200 and body.startswith(b"data: ") and b"done" in body and not dc.requests
        st, body = _post(gw + "/v1/chat/completions", {"messages": []})
        assert json.loads(body)["choices"][0]["message"]["content"] == "done"
    finally:
        p.terminate(); pf.stop(); dc.stop()
    dead = f"http://127.0.0.1:{_port()}"
    p, gw = _gateway("--hybrid", dead)
    try:
        st, body = _post(gw + "/v1/completions", {"prompt": "x"})
        assert st == 502 and b"gateway_error" in body
    finally:
        p.terminate()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_discovery_adds_and_removes_engines():
    ctrl, e = FakeEngine("ctrl"), FakeEngine("hybrid")
    ctrl.entities = [{"id": "e0", "role": "hybrid", "host": "127.0.0.1", "port": e.port, "model": "m"}]
    p, gw = _gateway("--ctrl-address", ctrl.url)
    try:
        for _ in range(40):
            if json.loads(urllib.request.urlopen(gw + "/engines").read()):
                break
            time.sleep(0.1)
        assert _post(gw + "/v1/completions", {"prompt": "x"})[0] == 200
        ctrl.entities = []
        for _ in range(80):
            if not json.loads(urllib.request.urlopen(gw + "/engines").read()):
                break
            time.sleep(0.1)
        assert _post(gw + "/v1/completions", {"prompt": "x"})[0] == 503
    finally:
        p.terminate(); ctrl.stop(); e.stop()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_status_page_counts_engines_and_requests():
    pf, dc = FakeEngine("prefill"), FakeEngine("decode")
    p, gw = _gateway("--prefill", pf.url, "--decode", dc.url)
    try:
        st = json.loads(urllib.request.urlopen(gw + "/status").read())
        assert st["status"] == "ok" and st["engines"] == {"hybrid": 0, "prefill": 1, "decode": 1} and st["pd_routing"] is True
        assert st["requests"] == {"total": 0, "pd": 0, "failed": 0} and st["pid"] == p.pid
        assert _post(gw + "/v1/chat/completions", {"model": "m", "messages": []})[0] == 200
        st = json.loads(urllib.request.urlopen(gw + "/status").read())
        assert st["requests"]["total"] == 1 and st["requests"]["pd"] == 1 and st["uptime_s"] >= 0
    finally:
        p.terminate(); pf.stop(); dc.stop()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_ctrl_scope_filters_the_discovered_engines():
    a, b, ctrl = FakeEngine("hybrid"), FakeEngine("hybrid"), FakeEngine("ctrl")
    ctrl.entities = [{"id": "a", "role": "hybrid", "host": "127.0.0.1", "port": a.port, "model": "m", "scope": "blue"},
                     {"id": "b", "role": "hybrid", "host": "127.0.0.1", "port": b.port, "model": "m", "scope": "green"}]
    p, gw = _gateway("--ctrl-address", ctrl.url, "--ctrl-scope", "blue")
    try:
        for _ in range(100):
            if json.loads(urllib.request.urlopen(gw + "/status").read())["engines"]["hybrid"]:
                break
            time.sleep(0.1)
        st = json.loads(urllib.request.urlopen(gw + "/status").read())
        assert st["engines"]["hybrid"] == 1 and st["ctrl_scope"] == "blue"
        assert any(path == "/list_entities" and body.get("scope") == "blue" for path, body in ctrl.requests)
        for _ in range(3):
            assert _post(gw + "/v1/completions", {"prompt": "x"})[0] == 200
        assert len([r for r in a.requests if r[0] == "/v1/completions"]) == 3 and not b.requests
    finally:
        p.terminate(); a.stop(); b.stop(); ctrl.stop()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_start_status_stop_run_the_gateway_as_a_daemon(tmp_path):
    e = FakeEngine("hybrid")
    port = _port()
    env = dict(os.environ, NANOENGINE_ROUTER_RUNTIME_DIR=str(tmp_path / "rt"))
    common = ["--port", str(port), "--host", "127.0.0.1"]

    def run(*args):
        return subprocess.run([GATEWAY, *args], env=env, capture_output=True, text=True, timeout=20)

    try:
        assert "not running" in run("status", *common).stdout
        out = run("start", *common, "--hybrid", e.url)
        assert out.returncode == 0 and "started (pid=" in out.stdout
        pid = int(out.stdout.split("pid=")[1].split(")")[0])
        for _ in range(100):
            try:
                socket.create_connection(("127.0.0.1", port), timeout=0.2).close()
                break
            except OSError:
                time.sleep(0.05)
        assert _post(f"http://127.0.0.1:{port}/v1/completions", {"prompt": "x"})[0] == 200
        st = run("status", *common)
        assert f"running (pid={pid})" in st.stdout and '"hybrid":1' in st.stdout and '"total":1' in st.stdout
        assert "already running" in run("start", *common, "--hybrid", e.url).stdout
        assert f"stopped (pid={pid})" in run("stop", *common).stdout
        assert "not running" in run("status", *common).stdout
        assert not (tmp_path / "rt" / "ne-gateway.pid").exists()
    finally:
        run("stop", *common)
        e.stop()


@pytest.mark.skipif(not os.path.exists(GATEWAY), reason="gateway binary not built")
def test_malformed_requests_do_not_take_the_gateway_down():
    e = FakeEngine("hybrid")
    p, gw = _gateway("--hybrid", e.url)
    port = int(gw.rsplit(":", 1)[1])

    def raw(data: bytes):
        with socket.create_connection(("127.0.0.1", port), timeout=3) as s:
            s.sendall(data)
            s.settimeout(3)
            try:
                return s.recv(4096)
            except OSError:
                return b""

    try:
        raw(b"\x00\xff\xfe garbage\r\n\r\n")
        raw(b"POST /v1/completions HTTP/1.1\r\nContent-Length: 999999999999999999999\r\n\r\n{}")
        raw(b"POST /v1/completions HTTP/1.1\r\nContent-Length: 5\r\n\r\n{\"a\"")
        raw(b"GET /status HTTP/1.1\r\n" + b"X-Pad: " + b"a" * 70000 + b"\r\n\r\n")
        for body in (b"", b"not json", b'{"model": ', b'{"model": {"nested": [1, 2, {"x": "\\u12"}]}}', b"[" * 2000, b'{"kv_transfer_params": 7, "stream": "yes"}'):
            req = urllib.request.Request(gw + "/v1/chat/completions", body, {"Content-Type": "application/json"})
            try:
                urllib.request.urlopen(req, timeout=5).read()
            except urllib.error.HTTPError:
                pass
            except OSError:
                pass
        assert p.poll() is None                                                     # still running
        assert json.loads(urllib.request.urlopen(gw + "/health").read())["engines"] == 1
        assert _post(gw + "/v1/completions", {"prompt": "x"})[0] == 200
    finally:
        p.terminate(); e.stop()
