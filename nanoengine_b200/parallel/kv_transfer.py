"""Prefill -> decode KV migration.

The decode scheduler admits a migrated request by allocating local pages and emitting a ``MigrationIn`` (which remote
pages land in which local pages).  A ``KVMigrator`` turns that into data movement through a transport:

* ``LocalTransport``   both caches are reachable as tensors in this process (CPU tests, one-GPU PD): indexed page copies.
* ``PeerPushTransport`` the prefill GPU maps the decode GPU's pool (CUDA IPC) and runs ``ne_kv_push``: peer stores of every
  (layer, page) plus a completion flag per request, which the decode side checks with a bounded wait.

Before moving anything the two engines' layouts are checked for compatibility (architecture, page size, cache dtype,
layer count, MTP layers): a mismatch fails the request instead of corrupting the pool.

Parity: reference runtime/disagg/p2p/cache_transfer.py:1144-1756 (migrate_from_bytes: validation :1180-1200, per
(layer, block) ops, MTP hand-off restore), :81-108 (bounds validation before submission), cache_layout.py:14-240.
"""
from __future__ import annotations

import ctypes as _c
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .._native import _core as C

_COMPAT_KEYS = ("architecture", "block_size", "kv_cache_dtype", "num_hidden_layers", "mtp_num_kv_layers")


def check_compatible(local_info: Dict, remote_info: Dict) -> None:
    bad = [k for k in _COMPAT_KEYS if local_info.get(k) != remote_info.get(k)]
    if bad:
        raise ValueError("PD engines are not compatible: " + ", ".join(f"{k}: {local_info.get(k)} != {remote_info.get(k)}" for k in bad))
    if local_info.get("attention_sp", 1) != 1 or remote_info.get("attention_sp", 1) != 1:
        raise ValueError("PD migration requires attention_sp == 1 on both sides")


def validate_blocks(blocks: Sequence[int], num_blocks: int, what: str) -> None:
    for b in blocks:
        if not (0 <= b < num_blocks):
            raise ValueError(f"{what} page id {b} outside the pool of {num_blocks} pages")


class LocalTransport:
    """src_runners / dst_runners: ModelRunner objects of the prefill and the decode engine living in this process."""

    def __init__(self, src_runners, dst_runners):
        self.src, self.dst = src_runners, dst_runners

    def copy(self, src_dp: int, dst_dp: int, src_blocks: List[int], dst_blocks: List[int], src_slot: int, dst_slot: int) -> int:
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
            dc.indexer.index_copy_(1, di, sc.indexer.index_select(1, si).to(dc.indexer.device))
            n += sc.indexer.index_select(1, si).numel()
        if s.mtp_runner is not None and d.mtp_runner is not None and src_slot >= 0 and dst_slot >= 0:
            d.mtp_runner.restore_handoff(dst_slot, s.mtp_runner.publish_handoff(src_slot))
        return n


class PeerPushTransport:
    """One prefill GPU pushing into one decode GPU's pool through a peer mapping of that pool."""

    def __init__(self, src_cache, dst_kv_peer: torch.Tensor, dst_flags_peer: torch.Tensor):
        from ..ops import sm100
        self.k = sm100
        self.src_cache = src_cache
        self.dst_kv = dst_kv_peer            # tensor view of the remote pool (opened from a CUDA IPC handle)
        self.flags = dst_flags_peer          # int32 flag words in the remote GPU's memory
        self.counter = torch.zeros(1, dtype=torch.int32, device=src_cache.kv.device)
        self.epoch = 0

    def push(self, src_blocks: List[int], dst_blocks: List[int], flag_slots: List[int]) -> int:
        kv = self.src_cache.kv
        plan = self.src_cache.plan
        assert plan.mla, "the push kernel moves MLA latent pages"
        dev = kv.device
        layers = kv.shape[0]
        page_bytes = kv.shape[2] * kv.shape[3] * kv.element_size()
        sb = torch.tensor(src_blocks, dtype=torch.int32, device=dev)
        db = torch.tensor(dst_blocks, dtype=torch.int32, device=dev)
        fi = torch.tensor(flag_slots, dtype=torch.int32, device=dev)
        self.epoch += 1
        k = self.k
        k._ck(k.lib().ne_kv_push(k._p(kv), k._p(self.dst_kv), _c.c_longlong(kv.stride(0) * kv.element_size()),
                                 _c.c_longlong(self.dst_kv.stride(0) * self.dst_kv.element_size()), _c.c_int(page_bytes), k._p(sb), k._p(db),
                                 _c.c_int(len(src_blocks)), _c.c_int(layers), k._p(self.flags), k._p(fi), _c.c_int(len(flag_slots)),
                                 _c.c_int(self.epoch), k._p(self.counter), k._st()), "ne_kv_push")
        return len(src_blocks) * layers * page_bytes


class KVMigrator:
    """Attached to a decode engine (``engine.migrator``).  `pull` is called with the serialized MigrationIn batches."""

    def __init__(self, transport, local_info: Dict, remote_info: Dict, remote_num_blocks: Optional[int] = None):
        check_compatible(local_info, remote_info)
        self.transport = transport
        self.local_blocks = local_info["num_blocks"]
        self.remote_blocks = remote_num_blocks if remote_num_blocks is not None else remote_info["num_blocks"]
        self.fail_next = False           # host-side fault injection for tests: pretend the peer vanished

    def pull(self, blobs: Sequence[bytes]) -> Tuple[List[int], List[int], int]:
        ok, bad, nbytes = [], [], 0
        for blob in blobs:
            m = C.MigrationIn.from_bytes(blob)
            for i, sid in enumerate(m.seq_ids):
                lo, hi = m.block_offsets[i], m.block_offsets[i + 1]
                src, dst = list(m.remote_blocks[lo:hi]), list(m.local_blocks[lo:hi])
                try:
                    if self.fail_next:
                        self.fail_next = False
                        raise ConnectionError("prefill peer disappeared before the push")
                    validate_blocks(src, self.remote_blocks, "remote")
                    validate_blocks(dst, self.local_blocks, "local")
                    nbytes += self.transport.copy(m.remote_dp_idx[i], m.dp_idx, src, dst, m.remote_handoff_slots[i], m.local_handoff_slots[i])
                    ok.append(sid)
                except Exception:
                    bad.append(sid)
        return ok, bad, nbytes
