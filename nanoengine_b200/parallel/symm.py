"""Symmetric heap: one allocation per GPU, mapped into every peer of a process group, carved up by a bump
allocator that hands out the same offsets on every rank.

The fused compute+collective kernels receive the table of peer base addresses and plain offsets; a buffer "of
rank r" is ``peer_base[r] + offset``.  Flag words used for cross-GPU hand-shakes live in the same heap.  The
mapping and the handle exchange are PyTorch's symmetric-memory plumbing (CUDA IPC / fabric handles over the group's
store); every load, store and wait on that memory is done by this package's kernels.

Parity: reference runtime/context/peer.py:124-199 (fabric allocation through its transport library) and
kernel/jit/sgl/communicator.py:49-117 (PyTorch symmetric memory + multicast pointer for the NVLS kernels).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

MAX_PEERS = 16


@dataclass
class SymmBuffer:
    offset: int          # bytes from the heap base (identical on every rank)
    nbytes: int
    local: torch.Tensor  # uint8 view of this rank's copy

    def view(self, dtype, shape) -> torch.Tensor:
        return self.local.view(dtype).view(*shape)


class SymmetricHeap:
    """Collective constructor: every rank of `group` must create the heap with the same size, in the same order."""

    def __init__(self, nbytes: int, group=None, device=None):
        import os
        # By default the heap is not bound to an NVLink multicast object (the kernels then use plain peer loads / stores): a
        # rank that goes away while bound to one disturbs the GPUs of the ranks that stay.  NE_NVLS=1 opts in to the binding
        # for the in-switch (multimem) collectives; the choice is per process and must be the same on every rank.
        if os.environ.get("NE_NVLS", "0") != "1":
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        nbytes = (nbytes + 4095) // 4096 * 4096
        self.nbytes = nbytes
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.rank = self.handle.rank
        self.world_size = self.handle.world_size
        if self.world_size > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} peers per heap")
        self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        try:        # 0 when the fabric offers no NVLS multicast object for this group
            self.multicast_ptr: int = int(self.handle.multicast_ptr)
        except Exception:
            self.multicast_ptr = 0
        self.buf.zero_()
        self._cursor = 0
        self._named: Dict[str, SymmBuffer] = {}
        # device copy of the peer table for kernels that index it at run time
        self.peer_table = torch.tensor(self.peer_ptrs + [0] * (MAX_PEERS - self.world_size), dtype=torch.int64, device=self.device)
        self.barrier()

    def alloc(self, nbytes: int, name: Optional[str] = None, align: int = 1024) -> SymmBuffer:
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: want {nbytes} bytes at {off}, heap has {self.nbytes}")
        self._cursor = off + nbytes
        b = SymmBuffer(off, nbytes, self.buf[off: off + nbytes])
        if name:
            self._named[name] = b
        return b

    def get(self, name: str) -> SymmBuffer:
        return self._named[name]

    def peer_addr(self, rank: int, buf: SymmBuffer) -> int:
        return self.peer_ptrs[rank] + buf.offset

    def barrier(self) -> None:
        """Host-side rendezvous of the group (used at set-up and tear-down, never on the hot path)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)


_HEAPS: Dict[Tuple[int, int], SymmetricHeap] = {}


def get_heap(group, nbytes: int) -> SymmetricHeap:
    key = (id(group), nbytes)
    if key not in _HEAPS:
        _HEAPS[key] = SymmetricHeap(nbytes, group)
    return _HEAPS[key]


def peers_reachable(group=None) -> bool:
    """True when every rank of the group sits on this node with peer access to the others."""
    if not torch.cuda.is_available() or not dist.is_initialized():
        return False
    n = torch.cuda.device_count()
    me = torch.cuda.current_device()
    ok = all(me == d or torch.cuda.can_device_access_peer(me, d) for d in range(n))
    t = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return bool(t.item())
