"""Prefill -> decode KV migration.

The decode scheduler admits a migrated request by allocating local pages and emitting a ``MigrationIn`` (which remote
pages land in which local pages).  A ``KVMigrator`` turns that into data movement through a transport:

* ``LocalTransport``    both caches are reachable as tensors in this process and nothing needs a GPU kernel (CPU engines):
  indexed page copies.
* ``PeerPushTransport`` the north-star path: every PREFILL worker has the DECODE workers' pools mapped into its address space
  (the same process: the tensors themselves; another process: CUDA IPC handles opened once at connect time) and, asked by
  the decode engine, runs ``ne_kv_push`` - peer stores of every (plane, page) of every cache family into the decode pool's
  pages, then one completion flag per request in the decode GPU's memory.  The decode worker checks the flags with a
  bounded device wait; a request whose flag never comes is failed on its own, the engine keeps serving.

  The control path is one message per batch of requests from the decode engine to the prefill engine (``pusher``): a direct
  call when both engines live in one process, the engine server's ``ACT_PD_PUSH`` packet otherwise.

Before moving anything the two engines' layouts are checked for compatibility (architecture, page size, cache dtype,
layer count, MTP layers; then every cache family's plane count and page bytes): a mismatch fails at connect time instead
of corrupting the pool.  Page ids are validated against both pools before submission.

Parity: reference runtime/disagg/p2p/cache_transfer.py:1144-1756 (migrate_from_bytes: validation :1180-1200, per
(layer, block) ops, MTP hand-off restore), :81-108 (bounds validation before submission), :203-425 (memory registration),
cache_layout.py:14-240.  The reference's decode side READS from the prefill pool (RDMA / NVLink through dlslime); here the
prefill side WRITES, which posts stores over NVLink instead of waiting for load round trips.
"""
from __future__ import annotations

import pickle
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .._native import _core as C

_COMPAT_KEYS = ("architecture", "block_size", "kv_cache_dtype", "num_hidden_layers", "mtp_num_kv_layers")
PD_FLAGS_PER_SOURCE = 64           # completion-flag words a decode worker keeps per prefill rank
PD_MAX_SOURCES = 16


def check_compatible(local_info: Dict, remote_info: Dict) -> None:
    bad = [k for k in _COMPAT_KEYS if local_info.get(k) != remote_info.get(k)]
    if bad:
        raise ValueError("PD engines are not compatible: " + ", ".join(f"{k}: {local_info.get(k)} != {remote_info.get(k)}" for k in bad))
    if local_info.get("attention_sp", 1) != 1 or remote_info.get("attention_sp", 1) != 1:
        raise ValueError("PD migration requires attention_sp == 1 on both sides")
    if local_info.get("attention_tp", 1) != remote_info.get("attention_tp", 1):
        raise ValueError("PD migration requires the same attention_tp on both sides (KV heads are sharded by it)")


def validate_blocks(blocks: Sequence[int], num_blocks: int, what: str) -> None:
    for b in blocks:
        if not (0 <= b < num_blocks):
            raise ValueError(f"{what} page id {b} outside the pool of {num_blocks} pages")


# ---- pool descriptors: what a decode worker publishes and a prefill worker opens ----------------------------------------
_DT = {"uint8": torch.uint8, "int32": torch.int32, "int64": torch.int64}
_OPENED: Dict[bytes, int] = {}           # IPC handle -> base address of its mapping in this process (an allocation opens once)


class _Alias:
    """Lets torch wrap memory it did not allocate (a peer process' buffer mapped into this one)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


def export_tensor(t: torch.Tensor, direct: bool):
    """`direct`: the tensor itself (same process).  Otherwise a picklable / JSON-able description from which a worker process on
    this machine can map the same device memory: the CUDA IPC handle of the allocation the tensor lives in, the tensor's
    byte offset inside it, its element type and element count (the tensor must be contiguous)."""
    if direct or not t.is_cuda:
        return t
    import ctypes as _c
    from ..ops import sm100 as k
    assert t.is_contiguous() and str(t.dtype).replace("torch.", "") in _DT
    h = (_c.c_ubyte * 64)()
    off, size = _c.c_longlong(0), _c.c_longlong(0)
    with torch.cuda.device(t.device):
        rc = k.lib().ne_ipc_export(_c.c_void_p(t.data_ptr()), h, _c.byref(off), _c.byref(size))
    if rc != 0:
        raise RuntimeError(f"cannot export device memory for another process (code {rc})")
    return {"ipc": bytes(h).hex(), "offset": int(off.value), "numel": t.numel(), "dtype": str(t.dtype).replace("torch.", ""),
            "device": t.device.index}


def open_tensor(h) -> torch.Tensor:
    """The tensor behind an `export_tensor` result.  The mapping of a peer buffer is opened with THIS process' current device
    current (the device whose kernels will write to it), once per allocation; the tensor returned aliases it."""
    if isinstance(h, torch.Tensor):
        return h
    import ctypes as _c
    from ..ops import sm100 as k
    handle = bytes.fromhex(h["ipc"])
    base = _OPENED.get(handle)
    if base is None:
        out = _c.c_void_p(0)
        rc = k.lib().ne_ipc_open((_c.c_ubyte * 64).from_buffer_copy(handle), _c.byref(out))
        if rc != 0:
            raise RuntimeError(f"cannot map a peer process' device memory (code {rc}); both processes must see the exporting GPU")
        base = _OPENED[handle] = int(out.value)
    dt = _DT[h["dtype"]]
    typestr = {"uint8": "|u1", "int32": "<i4", "int64": "<i8"}[h["dtype"]]
    t = torch.as_tensor(_Alias(base + h["offset"], (h["numel"],), typestr))      # no `device=`: that could copy instead of aliasing
    assert t.data_ptr() == base + h["offset"] and t.dtype == dt
    return t


def check_families(mine: List[dict], theirs: List[dict]) -> None:
    a = [(f["name"], f["planes"], f["page_bytes"], f.get("by", "page")) for f in mine]
    b = [(f["name"], f["planes"], f["page_bytes"], f.get("by", "page")) for f in theirs]
    if a != b:
        raise ValueError(f"PD cache layouts differ: prefill {a} vs decode {b}")


class LocalTransport:
    """src_runners / dst_runners: ModelRunner objects of the prefill and the decode engine living in this process."""

    def __init__(self, src_runners, dst_runners):
        self.src, self.dst = src_runners, dst_runners

    def copy(self, src_dp: int, dst_dp: int, src_blocks: List[int], dst_blocks: List[int], src_slot: int, dst_slot: int,
             src_state: int = -1, dst_state: int = -1) -> int:
        s, d = self.src[src_dp], self.dst[dst_dp]
        sc, dc = s.cache, d.cache
        si = torch.as_tensor(src_blocks, dtype=torch.long, device=sc.kv.device)
        di = torch.as_tensor(dst_blocks, dtype=torch.long, device=dc.kv.device)
        bdim = 1 if sc.plan.mla else 2
        skv = sc.kv.view(torch.uint8) if sc.kv.dtype == torch.float8_e4m3fn else sc.kv
        dkv = dc.kv.view(torch.uint8) if dc.kv.dtype == torch.float8_e4m3fn else dc.kv
        dkv.index_copy_(bdim, di, skv.index_select(bdim, si).to(dkv.device))
        n = skv.index_select(bdim, si).numel() * skv.element_size()
        if sc.indexer is not None and dc.indexer is not None:
            # the indexer keys may sit on another device than the latent pages (hot / cold tier: pages in host memory)
            rows = sc.indexer.index_select(1, si.to(sc.indexer.device))
            dc.indexer.index_copy_(1, di.to(dc.indexer.device), rows.to(dc.indexer.device))
            n += rows.numel()
        for t, u in zip(sc.comp or [], dc.comp or []):                    # pooled-row pages (DeepSeek-V4)
            if t is not None:
                u.index_copy_(0, di, t.index_select(0, si).to(u.device))
                n += len(src_blocks) * t[0].numel() * t.element_size()
        sfam, dfam = sc.slot_families(), dc.slot_families()
        if sfam:
            # per-sequence state: recurrent state and convolution window, compressor carries
            if not (0 <= src_state < sc.plan.state_slots and 0 <= dst_state < dc.plan.state_slots):
                raise ValueError("kv transfer: a family with per-sequence state needs the state slots of both sides")
            for f, g in zip(sfam, dfam):
                g["tensor"].select(g["slot_dim"], dst_state).copy_(f["tensor"].select(f["slot_dim"], src_state))
                n += f["planes"] * f["slot_bytes"]
        if s.mtp_runner is not None and d.mtp_runner is not None and src_slot >= 0 and dst_slot >= 0:
            d.mtp_runner.restore_handoff(dst_slot, s.mtp_runner.publish_handoff(src_slot))
        return n

    # ticket interface used by KVMigrator: a local copy is complete when it returns
    def submit(self, src_dp, dst_dp, src_blocks, dst_blocks, src_slot, dst_slot, src_state=-1, dst_state=-1):
        return ("done", self.copy(src_dp, dst_dp, src_blocks, dst_blocks, src_slot, dst_slot, src_state, dst_state))

    def finish(self, tickets) -> List[bool]:
        return [True] * len(tickets)


class PeerPushTransport:
    """Decode-engine side of the push protocol.

    `pusher(requests)`  asks the prefill engine to push; `requests` is a list of dicts {src_dp, dst_dp, src_blocks,
                        dst_blocks, src_slot, dst_slot, flag, epoch}.  Returns the bytes each request will move (the pushes
                        are queued on the prefill GPUs' streams when it returns, not necessarily finished).
    `waiter(dst_dp, flags, epochs)`  bounded device wait on the decode worker `dst_dp`; returns one bool per flag.
    """

    def __init__(self, pusher: Callable[[List[dict]], List[int]], waiter: Callable[[int, List[int], List[int]], List[bool]]):
        self.pusher, self.waiter = pusher, waiter
        self.epoch = 0
        self._next_flag: Dict[int, int] = {}
        self._pending: List[dict] = []

    def submit(self, src_dp, dst_dp, src_blocks, dst_blocks, src_slot, dst_slot, src_state=-1, dst_state=-1):
        if not (0 <= src_dp < PD_MAX_SOURCES):
            raise ValueError(f"prefill rank {src_dp} outside the flag table")
        self.epoch += 1
        k = self._next_flag.get(src_dp, 0)
        self._next_flag[src_dp] = (k + 1) % PD_FLAGS_PER_SOURCE
        req = {"src_dp": int(src_dp), "dst_dp": int(dst_dp), "src_blocks": list(map(int, src_blocks)), "dst_blocks": list(map(int, dst_blocks)),
               "src_slot": int(src_slot), "dst_slot": int(dst_slot), "src_state": int(src_state), "dst_state": int(dst_state),
               "flag": src_dp * PD_FLAGS_PER_SOURCE + k, "epoch": self.epoch}
        self._pending.append(req)
        return req

    def finish(self, tickets) -> List[bool]:
        """Send every submitted request to the prefill engine in one message, then wait for the flags."""
        reqs, self._pending = self._pending, []
        try:
            sizes = self.pusher(reqs)
        except Exception:
            return [False] * len(tickets)
        for r, n in zip(reqs, sizes):
            r["nbytes"] = n
        ok = {}
        by_dst: Dict[int, List[dict]] = {}
        for r in reqs:
            by_dst.setdefault(r["dst_dp"], []).append(r)
        for dst, lst in by_dst.items():
            got = self.waiter(dst, [r["flag"] for r in lst], [r["epoch"] for r in lst])
            for r, g in zip(lst, got):
                ok[r["epoch"]] = bool(g)
        return [ok.get(t["epoch"], False) for t in tickets]


class KVMigrator:
    """Attached to a decode engine (``engine.migrator``).  `pull` is called with the serialized MigrationIn batches.
    One transport per prefill engine: `add_peer` registers further ones, requests are routed by the engine id they carry."""

    def __init__(self, transport, local_info: Dict, remote_info: Dict, remote_num_blocks: Optional[int] = None):
        check_compatible(local_info, remote_info)
        self.transport = transport
        self.local_info = local_info
        self.local_blocks = local_info["num_blocks"]
        self.remote_blocks = remote_num_blocks if remote_num_blocks is not None else remote_info["num_blocks"]
        self.peers: Dict[str, Tuple[object, int]] = {str(remote_info.get("id", "")): (transport, self.remote_blocks)}
        self.fail_next = False           # host-side fault injection for tests: pretend the peer vanished

    def add_peer(self, transport, remote_info: Dict) -> None:
        check_compatible(self.local_info, remote_info)
        self.peers[str(remote_info.get("id", ""))] = (transport, remote_info["num_blocks"])

    def _route(self, engine_id: str):
        return self.peers.get(str(engine_id), (self.transport, self.remote_blocks))

    def pull(self, blobs: Sequence[bytes]) -> Tuple[List[int], List[int], int]:
        ok, bad, nbytes = [], [], 0
        batches: Dict[int, Tuple[object, List[int], list]] = {}          # per transport: sequence ids and their tickets
        for blob in blobs:
            m = C.MigrationIn.from_bytes(blob)
            eids = list(getattr(m, "remote_engine_ids", []) or [])
            for i, sid in enumerate(m.seq_ids):
                lo, hi = m.block_offsets[i], m.block_offsets[i + 1]
                src, dst = list(m.remote_blocks[lo:hi]), list(m.local_blocks[lo:hi])
                try:
                    if self.fail_next:
                        self.fail_next = False
                        raise ConnectionError("prefill peer disappeared before the push")
                    tr, remote_blocks = self._route(eids[i] if i < len(eids) else "")
                    validate_blocks(src, remote_blocks, "remote")
                    validate_blocks(dst, self.local_blocks, "local")
                    rs, ls = list(m.remote_state_slots), list(m.local_state_slots)
                    t = tr.submit(m.remote_dp_idx[i], m.dp_idx, src, dst, m.remote_handoff_slots[i], m.local_handoff_slots[i],
                                  rs[i] if i < len(rs) else -1, ls[i] if i < len(ls) else -1)
                    b = batches.setdefault(id(tr), (tr, [], []))
                    b[1].append(sid); b[2].append(t)
                except Exception:
                    bad.append(sid)
        for tr, sids, tickets in batches.values():
            for sid, t, good in zip(sids, tickets, tr.finish(tickets)):
                if good:
                    ok.append(sid)
                    nbytes += t[1] if isinstance(t, tuple) else int(t.get("nbytes", 0))
                else:
                    bad.append(sid)
        return ok, bad, nbytes


# ---- wiring ----------------------------------------------------------------------------------------------------------------
def connect_inproc(prefill_engine, decode_engine) -> KVMigrator:
    """Both engines live in this process (their executors may still own worker processes): the decode workers publish their
    pools, the prefill workers open them, and the decode engine gets a migrator that pushes through direct calls."""
    direct = prefill_engine.executor.in_process and decode_engine.executor.in_process
    pools = decode_engine.executor.collective_rpc("pd_export_pool", direct)
    key = decode_engine.config.engine_id
    prefill_engine.executor.collective_rpc("pd_open_pool", key, pools)

    def pusher(reqs):
        # every prefill worker sees the batch and serves the requests of its own attention-DP rank (all TP ranks of it)
        per_worker = prefill_engine.executor.collective_rpc("pd_push", key, reqs)
        return [max(col) for col in zip(*per_worker)] if reqs else []

    def waiter(dst_dp, flags, epochs):
        per_worker = [r for r in decode_engine.executor.collective_rpc("pd_wait", dst_dp, flags, epochs) if r is not None]
        return [all(col) for col in zip(*per_worker)] if per_worker else [False] * len(flags)

    mig = KVMigrator(PeerPushTransport(pusher, waiter), decode_engine.engine_info(), prefill_engine.engine_info())
    decode_engine.migrator = mig
    return mig


# ---- the same protocol between two engine processes (ZMQ packets of the engine server) -------------------------------------
def _hexify(pools: List[dict]) -> List[dict]:
    def hx(v):
        return v.hex() if isinstance(v, (bytes, bytearray)) else v
    return [dict(p, families=[dict(f, tensor=hx(f["tensor"])) for f in p["families"]], flags=hx(p["flags"]), handoff=hx(p.get("handoff"))) for p in pools]


def _unhexify(pools: List[dict]) -> List[dict]:
    def ux(v):
        return bytes.fromhex(v) if isinstance(v, str) else v
    return [dict(p, families=[dict(f, tensor=ux(f["tensor"])) for f in p["families"]], flags=ux(p["flags"]), handoff=ux(p.get("handoff"))) for p in pools]


def serve_pd_packet(engine, action: int, payload: bytes) -> bytes:
    """Prefill engine process: answer one ACT_PD_OPEN / ACT_PD_PUSH packet (JSON both ways; the memory handles inside are the
    pickled CUDA IPC descriptors torch uses between its own processes, so this channel is for engines of one deployment on
    one machine - an `ipc://` endpoint - not for untrusted peers)."""
    import json
    msg = json.loads(payload)
    if action == C.ACT_PD_OPEN:
        n = sum(engine.executor.collective_rpc("pd_open_pool", msg["key"], _unhexify(msg["pools"])))
        return json.dumps({"mapped": n, "info": engine.engine_info()}).encode()
    per_worker = engine.executor.collective_rpc("pd_push", msg["key"], msg["reqs"])
    return json.dumps({"sizes": [max(col) for col in zip(*per_worker)] if msg["reqs"] else []}).encode()


class PdPeerClient:
    """Decode engine process: blocking client of one prefill engine's socket."""

    def __init__(self, endpoint: str, timeout_s: float = 30.0):
        import zmq
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.DEALER)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.connect(endpoint)
        self.timeout_ms = int(timeout_s * 1000)

    def call(self, action: int, obj: dict) -> dict:
        import json
        self.sock.send(C.WirePacket(action, json.dumps(obj).encode()).to_bytes())
        if not self.sock.poll(self.timeout_ms):
            raise TimeoutError("the prefill engine did not answer")
        pkt = C.WirePacket.from_bytes(self.sock.recv())
        out = json.loads(pkt.payload)
        if "error" in out:
            raise RuntimeError(f"prefill engine: {out['error']}")
        return out


def connect_remote(decode_engine, prefill_engine_id: str, endpoint: str) -> KVMigrator:
    """Decode engine process: publish the workers' pools to the prefill engine behind `endpoint` and attach (or extend) the
    migrator that asks it to push."""
    cli = PdPeerClient(endpoint)
    key = decode_engine.config.engine_id
    pools = decode_engine.executor.collective_rpc("pd_export_pool", False)
    rinfo = cli.call(C.ACT_PD_OPEN, {"key": key, "pools": _hexify(pools)})["info"]

    def pusher(reqs):
        return cli.call(C.ACT_PD_PUSH, {"key": key, "reqs": reqs})["sizes"]

    def waiter(dst_dp, flags, epochs):
        per_worker = [r for r in decode_engine.executor.collective_rpc("pd_wait", dst_dp, flags, epochs) if r is not None]
        return [all(col) for col in zip(*per_worker)] if per_worker else [False] * len(flags)

    tr = PeerPushTransport(pusher, waiter)
    if decode_engine.migrator is None:
        decode_engine.migrator = KVMigrator(tr, decode_engine.engine_info(), rinfo)
    else:
        decode_engine.migrator.add_peer(tr, rinfo)
    return decode_engine.migrator
