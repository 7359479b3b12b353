"""Engine process and its client: the HTTP workers talk to one engine loop over a ZMQ ROUTER/DEALER pair.

Backend (`run_engine_backend`): owns the LLMEngine.  Each iteration drains the socket (ADD / FREE / ABORT / GET_INFO /
GET_METRICS / START_PROFILER / STOP_PROFILER), runs `engine.step()` when there is work, and pushes one STEPOUT_BATCH packet
per client with the tokens its sequences produced.  Frontend (`EngineClient`): assigns sequence ids, multiplexes any number
of concurrent requests over one DEALER socket and hands each request an asyncio queue of StepOut objects.  A watchdog
notices a dead backend within half a second and fails every pending request instead of letting callers hang.

One hop (ZMQ ipc) replaces the reference's two (ZMQ to a frontend process, then an mp.Queue to the backend process).
Parity: reference server/engine_server.py:212-415 (backend loop, action codes 1..8), :427-593 (frontend, watchdog
:547-591), server/zmq_engine_client.py:59-345, server/wire.py.
"""
from __future__ import annotations

import asyncio
import json
import multiprocessing as mp
import os
import struct
import tempfile
import threading
import time
from typing import Dict, List, Optional

from .._native import _core as C


def _pack_stepouts(outs) -> bytes:
    blobs = [o.to_bytes() for o in outs]
    return struct.pack("<I", len(blobs)) + b"".join(struct.pack("<I", len(b)) + b for b in blobs)


def _unpack_stepouts(buf: bytes):
    (n,), off, outs = struct.unpack_from("<I", buf, 0), 4, []
    for _ in range(n):
        (ln,) = struct.unpack_from("<I", buf, off)
        off += 4
        outs.append(C.StepOut.from_bytes(buf[off:off + ln]))
        off += ln
    return outs


def run_engine_backend(config_dict: dict, endpoint: str, ready=None, engine_factory=None):
    """Body of the engine process.  `engine_factory` lets tests substitute a fake engine."""
    import zmq
    from ..config import Config
    ctx = zmq.Context()
    sock = ctx.socket(zmq.ROUTER)
    sock.bind(endpoint)
    if engine_factory is not None:
        engine = engine_factory(config_dict)
    else:
        from ..engine.llm_engine import LLMEngine
        engine = LLMEngine(Config.from_dict(config_dict))
    owner: Dict[int, bytes] = {}       # seq_id -> client identity
    publisher = None
    if engine_factory is None:
        engine.endpoint = endpoint
        if config_dict.get("ctrl_address"):
            # peers find this engine process (a decode engine: the prefill engine that sent it a sequence) through the control plane
            from .ctrl import EnginePublisher
            publisher = EnginePublisher(config_dict["ctrl_address"], engine.engine_info)
    for peer_id, peer_ep in (config_dict.get("pd_peers") or {}).items():
        from ..parallel.kv_transfer import connect_remote
        connect_remote(engine, peer_id, peer_ep)      # decode role: prefill engines that will push KV into this engine's pools
    if ready is not None:
        ready.set()
    running = True
    while running:
        timeout = 0 if not engine.is_finished() else 50
        while sock.poll(timeout):
            timeout = 0
            ident, payload = sock.recv_multipart()
            try:
                pkt = C.WirePacket.from_bytes(payload)
            except ValueError as e:      # corrupted packet: tell the sender, keep serving
                sock.send_multipart([ident, C.WirePacket(-1, str(e).encode()).to_bytes()])
                continue
            a = pkt.action
            if a == C.ACT_ADD:
                try:
                    sid = engine.add_request_payload(pkt.payload)
                    owner[sid] = ident
                except Exception as e:
                    sock.send_multipart([ident, C.WirePacket(-1, f"add failed: {e}".encode()).to_bytes()])
            elif a == C.ACT_ABORT:
                (sid,) = struct.unpack("<Q", pkt.payload)
                engine.abort(sid)
                owner.pop(sid, None)
            elif a == C.ACT_FREE:
                ids = list(struct.unpack(f"<{len(pkt.payload) // 8}Q", pkt.payload))
                engine.free_to_be_migrated_ids(ids)
            elif a == C.ACT_GET_INFO:
                info = dict(engine.engine_info())
                if pkt.payload == b"export":
                    info["migrations"] = [m.to_bytes().hex() for m in engine.export_to_be_migrated()]
                sock.send_multipart([ident, C.WirePacket(C.ACT_GET_INFO, json.dumps(info).encode()).to_bytes()])
            elif a == C.ACT_GET_METRICS:
                sock.send_multipart([ident, C.WirePacket(C.ACT_GET_METRICS, engine.metrics_prometheus().encode()).to_bytes()])
            elif a == C.ACT_START_PROFILER:
                ok = False
                try:
                    ok = engine.start_profiler(pkt.payload.decode() or "trace")
                except Exception:
                    ok = False
                sock.send_multipart([ident, C.WirePacket(a, b"1" if ok else b"0").to_bytes()])
            elif a == C.ACT_STOP_PROFILER:
                paths = engine.stop_profiler()
                sock.send_multipart([ident, C.WirePacket(a, json.dumps(paths).encode()).to_bytes()])
            elif a in (C.ACT_PD_OPEN, C.ACT_PD_PUSH):
                # a decode engine on this machine asks this (prefill) engine to map its pools / push pages into them
                from ..parallel.kv_transfer import serve_pd_packet
                try:
                    reply = serve_pd_packet(engine, a, pkt.payload)
                    sock.send_multipart([ident, C.WirePacket(a, reply).to_bytes()])
                except Exception as e:
                    sock.send_multipart([ident, C.WirePacket(a, json.dumps({"error": str(e)}).encode()).to_bytes()])
            elif a == 99:   # shutdown
                running = False
        if not running:
            break
        if engine.is_finished():
            continue
        outs = engine.step()
        per_client: Dict[bytes, list] = {}
        for o in outs:
            ident = owner.get(o.seq_id)
            if ident is None:
                continue
            per_client.setdefault(ident, []).append(o)
            if o.status in (C.FINISHED, C.TO_BE_MIGRATED):
                owner.pop(o.seq_id, None)
        for ident, lst in per_client.items():
            sock.send_multipart([ident, C.WirePacket(C.ACT_STEPOUT_BATCH, _pack_stepouts(lst)).to_bytes()])
    if publisher is not None:
        publisher.stop()
    try:
        engine.shutdown()
    except Exception:
        pass
    sock.close(0)
    ctx.term()


class BackendDied(RuntimeError):
    pass


class EngineClient:
    """Asyncio client used by the HTTP server.  One instance per server process."""

    def __init__(self, endpoint: str, backend_proc: Optional[mp.Process] = None, id_base: int = 1):
        import zmq
        import zmq.asyncio
        self.endpoint = endpoint
        self.proc = backend_proc
        self.ctx = zmq.asyncio.Context()
        self.sock = self.ctx.socket(zmq.DEALER)
        self.sock.connect(endpoint)
        self.queues: Dict[int, asyncio.Queue] = {}
        self.replies: Dict[int, asyncio.Future] = {}
        self._next = id_base
        self._tasks: List[asyncio.Task] = []
        self.dead = False

    def start(self):
        loop = asyncio.get_running_loop()
        self._tasks = [loop.create_task(self._reader()), loop.create_task(self._watchdog())]

    async def close(self):
        for t in self._tasks:
            t.cancel()
        self.sock.close(0)

    def destroy(self):
        """Drop the socket and the ZMQ context without lingering (safe to call from any thread at shutdown)."""
        for t in self._tasks:
            try:
                t.cancel()
            except Exception:
                pass
        try:
            self.sock.close(0)
        except Exception:
            pass
        try:
            self.ctx.destroy(linger=0)
        except Exception:
            pass

    def next_seq_id(self) -> int:
        self._next += 1
        return self._next

    async def _reader(self):
        while True:
            payload = await self.sock.recv()
            pkt = C.WirePacket.from_bytes(payload)
            if pkt.action == C.ACT_STEPOUT_BATCH:
                for o in _unpack_stepouts(pkt.payload):
                    q = self.queues.get(o.seq_id)
                    if q is not None:
                        q.put_nowait(o)
            elif pkt.action in self.replies:
                fut = self.replies.pop(pkt.action)
                if not fut.done():
                    fut.set_result(pkt.payload)
            elif pkt.action == -1:
                for q in list(self.queues.values()):
                    q.put_nowait(RuntimeError(pkt.payload.decode(errors="replace")))

    async def _watchdog(self):
        while True:
            await asyncio.sleep(0.5)
            if self.proc is not None and not self.proc.is_alive():
                self.dead = True
                err = BackendDied(f"engine backend exited with code {self.proc.exitcode}")
                for q in list(self.queues.values()):
                    q.put_nowait(err)
                for f in list(self.replies.values()):
                    if not f.done():
                        f.set_exception(err)
                return

    async def submit(self, prompt_token_ids, sampling_params, affinity_key: int = 0, seq_id: Optional[int] = None) -> int:
        if self.dead:
            raise BackendDied("engine backend is not running")
        sid = seq_id if seq_id is not None else self.next_seq_id()
        self.queues[sid] = asyncio.Queue()
        req = C.RequestIn(sid, list(prompt_token_ids), sampling_params, affinity_key)
        await self.sock.send(C.WirePacket(C.ACT_ADD, req.to_bytes()).to_bytes())
        return sid

    async def submit_migrated(self, blob: bytes) -> int:
        m = C.RequestMigrate.from_bytes(blob)
        self.queues[m.seq_id] = asyncio.Queue()
        await self.sock.send(C.WirePacket(C.ACT_ADD, blob).to_bytes())
        return m.seq_id

    async def stream(self, sid: int):
        """Yield StepOut objects of one sequence until it finishes."""
        q = self.queues[sid]
        try:
            while True:
                o = await q.get()
                if isinstance(o, Exception):
                    raise o
                yield o
                if o.status in (C.FINISHED, C.TO_BE_MIGRATED):
                    return
        finally:
            self.queues.pop(sid, None)

    async def abort(self, sid: int):
        self.queues.pop(sid, None)
        await self.sock.send(C.WirePacket(C.ACT_ABORT, struct.pack("<Q", sid)).to_bytes())

    async def free(self, ids):
        await self.sock.send(C.WirePacket(C.ACT_FREE, struct.pack(f"<{len(ids)}Q", *ids)).to_bytes())

    async def _call(self, action: int, payload: bytes = b"", timeout: float = 30.0) -> bytes:
        fut = asyncio.get_running_loop().create_future()
        self.replies[action] = fut
        await self.sock.send(C.WirePacket(action, payload).to_bytes())
        return await asyncio.wait_for(fut, timeout)

    async def info(self, export: bool = False) -> dict:
        return json.loads(await self._call(C.ACT_GET_INFO, b"export" if export else b""))

    async def metrics(self) -> str:
        return (await self._call(C.ACT_GET_METRICS)).decode()

    async def start_profiler(self, name: str) -> bool:
        return (await self._call(C.ACT_START_PROFILER, name.encode())) == b"1"

    async def stop_profiler(self):
        return json.loads(await self._call(C.ACT_STOP_PROFILER, timeout=120.0))

    async def shutdown_backend(self):
        await self.sock.send(C.WirePacket(99, b"").to_bytes())


def spawn_backend(config, engine_factory=None, endpoint: Optional[str] = None):
    """Start the engine process; returns (process, endpoint) once it is serving."""
    endpoint = endpoint or f"ipc://{tempfile.gettempdir()}/ne-engine-{os.getpid()}-{int(time.time() * 1e6) & 0xffffff}.sock"
    ctx = mp.get_context("spawn")
    ready = ctx.Event()
    p = ctx.Process(target=run_engine_backend, args=(config.to_dict() if hasattr(config, "to_dict") else config, endpoint, ready, engine_factory), daemon=True)
    p.start()
    t0 = time.time()
    while not ready.wait(0.5):
        if not p.is_alive():
            raise BackendDied(f"engine backend failed to start (exit code {p.exitcode})")
        if time.time() - t0 > 1800:
            raise BackendDied("engine backend did not come up within 30 minutes")
    return p, endpoint
