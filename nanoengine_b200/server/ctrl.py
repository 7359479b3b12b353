"""Control plane for dynamic discovery: engines announce their HTTP endpoint (role, model, scope) and keep it alive with a
heartbeat; the gateway polls the list and adds / drops engines as they come and go.

    nanoengine ctrl --port 4479                       # the registry (in memory, entries expire `ttl` seconds after their last heartbeat)
    nanoengine serve MODEL --ctrl_address http://host:4479 [--ctrl_scope blue]      # an engine that registers itself
    nanoengine-router --ctrl-address http://host:4479 [--ctrl-scope blue]           # a gateway that discovers engines

HTTP API (JSON bodies): POST /register {id, host, port, role, model, scope?, engine_id?}, POST /heartbeat {id} -> {found, unknown},
POST /unregister {id}, POST /list_entities {scope?} -> {entities: [...]}, GET /health.  Engines also publish their own description
(`LLMComponent`: block size, cache dtype, layer count, ... under the engine id) with POST /register_entity {id, ...}; a peer reads it
back with POST /get_entity {id} -> {entity} to check compatibility before it accepts migrated sequences.

Parity: the reference registers with an external control-plane service through its client library
(server/openai_server.py:1748-1810 `register_with_ctrl`: entity id, endpoint, role / model metadata, heartbeat with
re-registration when the entry is gone) and its router polls it (rust/src/router/engine_manager.rs:263-452); here the small
service itself is part of the package."""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Dict, List, Optional


class Registry:
    """Entities by id; an entity not heard from for `ttl` seconds is gone."""

    def __init__(self, ttl: float = 15.0, clock: Callable[[], float] = time.monotonic):
        self.ttl, self.clock = ttl, clock
        self._mu = threading.Lock()
        self._ents: Dict[str, dict] = {}
        self._engines: Dict[str, dict] = {}          # engine descriptions by engine id: {"info": {...}, "seen": t}

    def register(self, ent: dict) -> None:
        if not ent.get("id") or not ent.get("port"):
            raise ValueError("an entity needs an id and a port")
        e = {"id": str(ent["id"]), "host": str(ent.get("host") or "127.0.0.1"), "port": int(ent["port"]), "role": str(ent.get("role") or "hybrid"),
             "model": str(ent.get("model") or ""), "scope": str(ent.get("scope") or ""), "engine_id": str(ent.get("engine_id") or ""),
             "seen": self.clock()}
        if e["role"] not in ("hybrid", "prefill", "decode"):
            raise ValueError(f"unknown role {e['role']!r}")
        e["url"] = f"http://{e['host']}:{e['port']}"
        with self._mu:
            self._ents[e["id"]] = e

    def heartbeat(self, ent_id: str) -> bool:
        with self._mu:
            found = False
            for table in (self._ents, self._engines):
                e = table.get(ent_id)
                if e is None:
                    continue
                if self.clock() - e["seen"] > self.ttl:
                    del table[ent_id]
                else:
                    e["seen"] = self.clock()
                    found = True
            return found

    def register_engine(self, info: dict) -> None:
        if not info.get("id"):
            raise ValueError("an engine description needs an id")
        with self._mu:
            self._engines[str(info["id"])] = {"info": dict(info), "seen": self.clock()}

    def get_engine(self, engine_id: str) -> Optional[dict]:
        with self._mu:
            e = self._engines.get(engine_id)
            if e is None or self.clock() - e["seen"] > self.ttl:
                self._engines.pop(engine_id, None)
                return None
            return dict(e["info"])

    def unregister(self, ent_id: str) -> bool:
        with self._mu:
            a = self._ents.pop(ent_id, None) is not None
            b = self._engines.pop(ent_id, None) is not None
            return a or b

    def list(self, scope: Optional[str] = None) -> List[dict]:
        now = self.clock()
        with self._mu:
            for k in [k for k, e in self._ents.items() if now - e["seen"] > self.ttl]:
                del self._ents[k]
            return [{k: v for k, v in e.items() if k != "seen"} for e in self._ents.values() if not scope or e["scope"] == scope]


def make_server(host: str = "0.0.0.0", port: int = 4479, ttl: float = 15.0, registry: Optional[Registry] = None) -> ThreadingHTTPServer:
    reg = registry or Registry(ttl)

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _reply(self, code: int, obj) -> None:
            b = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(b)))
            self.end_headers()
            self.wfile.write(b)

        def do_GET(self):
            if self.path == "/health":
                return self._reply(200, {"status": "ok", "entities": len(reg.list())})
            self._reply(404, {"error": "unknown route"})

        def do_POST(self):
            try:
                body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
                if self.path == "/register":
                    reg.register(body)
                    return self._reply(200, {"ok": True})
                if self.path == "/heartbeat":
                    found = reg.heartbeat(str(body.get("id", "")))
                    return self._reply(200, {"found": found, "unknown": not found})
                if self.path == "/register_entity":
                    reg.register_engine(body)
                    return self._reply(200, {"ok": True})
                if self.path == "/get_entity":
                    return self._reply(200, {"entity": reg.get_engine(str(body.get("id", "")))})
                if self.path == "/unregister":
                    return self._reply(200, {"removed": reg.unregister(str(body.get("id", "")))})
                if self.path == "/list_entities":
                    return self._reply(200, {"entities": reg.list(body.get("scope") or None)})
            except (ValueError, KeyError, TypeError) as e:
                return self._reply(400, {"error": str(e)})
            self._reply(404, {"error": "unknown route"})

    srv = ThreadingHTTPServer((host, port), Handler)
    srv.registry = reg
    return srv


def run_ctrl(host: str = "0.0.0.0", port: int = 4479, ttl: float = 15.0) -> None:
    srv = make_server(host, port, ttl)
    try:
        srv.serve_forever()
    finally:
        srv.server_close()


class CtrlClient:
    """An engine's side: register, then a heartbeat thread that registers again when the control plane has forgotten the entry
    (it restarted, or the engine was silent for longer than the time to live)."""

    def __init__(self, address: str, scope: Optional[str] = None, timeout: float = 3.0):
        self.address, self.scope, self.timeout = address.rstrip("/"), scope or "", timeout
        self._ent: Optional[dict] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _post(self, path: str, obj: dict) -> dict:
        req = urllib.request.Request(self.address + path, json.dumps(obj).encode(), {"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
            return json.loads(r.read() or b"{}")

    def register(self, ent_id: str, host: str, port: int, role: str = "hybrid", model: str = "", engine_id: str = "") -> bool:
        self._ent = {"id": ent_id, "host": host, "port": port, "role": role, "model": model, "scope": self.scope, "engine_id": engine_id}
        try:
            return bool(self._post("/register", self._ent).get("ok"))
        except OSError:
            return False

    def list_entities(self) -> List[dict]:
        return self._post("/list_entities", {"scope": self.scope} if self.scope else {}).get("entities", [])

    def start_heartbeat(self, interval: float = 5.0) -> None:
        def loop():
            while not self._stop.wait(interval):
                try:
                    if not self._post("/heartbeat", {"id": self._ent["id"]}).get("found"):
                        self._post("/register", self._ent)
                except OSError:
                    pass                      # the control plane is away: keep trying, the engine keeps serving

        self._thread = threading.Thread(target=loop, name="ctrl-heartbeat", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self._ent is not None:
            try:
                self._post("/unregister", {"id": self._ent["id"]})
            except OSError:
                pass


def fetch_engine(address: str, engine_id: str, timeout: float = 3.0) -> Optional[dict]:
    """The description an engine published under its id (None: unknown, expired, or the control plane is away)."""
    req = urllib.request.Request(address.rstrip("/") + "/get_entity", json.dumps({"id": engine_id}).encode(), {"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return json.loads(r.read() or b"{}").get("entity")
    except OSError:
        return None


class EnginePublisher:
    """Keeps an engine's description (`LLMEngine.engine_info()`: layout facts a peer checks, the engine process's endpoint) alive in
    the control plane: publish, heartbeat, publish again when the registry has forgotten it."""

    def __init__(self, address: str, info_fn: Callable[[], dict], interval: float = 5.0):
        self.address, self.info_fn, self.interval = address.rstrip("/"), info_fn, interval
        self._stop = threading.Event()
        self.published = self._publish()
        self._thread = threading.Thread(target=self._loop, name="ctrl-engine-heartbeat", daemon=True)
        self._thread.start()

    def _post(self, path: str, obj: dict) -> Optional[dict]:
        req = urllib.request.Request(self.address + path, json.dumps(obj).encode(), {"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=3.0) as r:
                return json.loads(r.read() or b"{}")
        except OSError:
            return None

    def _publish(self) -> bool:
        return self._post("/register_entity", self.info_fn()) is not None

    def _loop(self):
        while not self._stop.wait(self.interval):
            r = self._post("/heartbeat", {"id": self.info_fn()["id"]})
            self.published = self._publish() if (r is None or r.get("unknown")) else True

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=2)
        self._post("/unregister", {"id": self.info_fn()["id"]})


def advertise_host(host: str) -> str:
    """The address other machines should use for a server bound to `host` (a wildcard bind is announced under this machine's own
    address)."""
    from ..utils.network import get_advertise_host
    return get_advertise_host(host)


def register_with_ctrl(config, host: str, port: int, served_model_name: str) -> Optional[CtrlClient]:
    """Announce this engine's HTTP endpoint and keep it alive; None when the control plane cannot be reached."""
    adv = advertise_host(host)
    cli = CtrlClient(config.ctrl_address, getattr(config, "ctrl_scope", None))
    ent_id = f"nanoengine-{served_model_name}-{adv}:{port}"
    if not cli.register(ent_id, adv, port, role=config.mode, model=served_model_name, engine_id=config.engine_id):
        return None
    cli.start_heartbeat()
    return cli
