"""Slots of vision embeddings on the encoder's GPU, read by the language-model workers.

One buffer [slots, max_tokens_per_slot, hidden]; a slot holds the merged embeddings of one request's images until the language
model has consumed them.  A worker in another process maps the buffer once (CUDA IPC, `parallel/kv_transfer.py::export_tensor
/ open_tensor`) and copies a slot's rows over NVLink; a worker in the same process reads the tensor directly.

Parity: reference runtime/context/cache/emb.py:24-120 (slot allocator, byte offsets, memory-region registration for one-sided
reads).
"""
from __future__ import annotations

import heapq
from typing import Dict, List

import torch


class EmbeddingPool:
    def __init__(self, num_slots: int, max_tokens_per_slot: int, hidden_size: int, device="cuda", dtype=torch.bfloat16):
        self.num_slots, self.max_tokens, self.hidden = num_slots, max_tokens_per_slot, hidden_size
        self.buffer = torch.zeros(num_slots, max_tokens_per_slot, hidden_size, dtype=dtype, device=device)
        self._free: List[int] = list(range(num_slots))
        self._tokens: Dict[int, int] = {}

    @property
    def available_slots(self) -> int:
        return len(self._free)

    def allocate(self, num_tokens: int) -> int:
        if num_tokens > self.max_tokens:
            raise RuntimeError(f"{num_tokens} embedding rows exceed the slot size {self.max_tokens}")
        if not self._free:
            raise RuntimeError("embedding pool: no free slot")
        s = heapq.heappop(self._free)
        self._tokens[s] = num_tokens
        return s

    def free(self, slots) -> int:
        n = 0
        for s in ([slots] if isinstance(slots, int) else slots):
            if s in self._tokens:
                del self._tokens[s]
                heapq.heappush(self._free, s)
                n += 1
        return n

    def write(self, slot: int, emb: torch.Tensor) -> None:
        n = emb.shape[0]
        if n > self.max_tokens:
            raise RuntimeError(f"{n} embedding rows exceed the slot size {self.max_tokens}")
        self.buffer[slot, :n].copy_(emb.to(self.buffer.dtype))
        self._tokens[slot] = n

    def read(self, slot: int) -> torch.Tensor:
        return self.buffer[slot, : self._tokens.get(slot, 0)]

    def num_tokens(self, slot: int) -> int:
        return self._tokens.get(slot, 0)

    def slot_byte_offset(self, slot: int) -> int:
        return slot * self.max_tokens * self.hidden * self.buffer.element_size()

    def export(self, direct: bool = False) -> dict:
        """What a reader needs to map the buffer: the tensor itself in this process, else its IPC descriptor."""
        from ..parallel.kv_transfer import export_tensor
        return {"tensor": export_tensor(self.buffer, direct), "slots": self.num_slots, "max_tokens": self.max_tokens,
                "hidden": self.hidden, "dtype": str(self.buffer.dtype).replace("torch.", "")}


class EmbeddingReader:
    """Language-model side: a mapped view of an encoder's pool."""

    def __init__(self, desc: dict, device):
        from ..parallel.kv_transfer import open_tensor
        self.device = torch.device(device)
        t = desc["tensor"]
        if isinstance(t, torch.Tensor):
            self.buffer = t
        else:
            with torch.cuda.device(self.device):          # the mapping is opened with the reading device current
                self.buffer = open_tensor(t)
        self.buffer = self.buffer.view(desc["slots"], desc["max_tokens"], desc["hidden"])

    def fetch(self, slot: int, num_tokens: int, dtype) -> torch.Tensor:
        return self.buffer[slot, :num_tokens].to(self.device, dtype, copy=True)
