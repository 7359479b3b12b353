"""Hot / cold tiering of the sparse-attention latent cache (HiSparse) for DSA decode engines.

The scheduler keeps addressing logical pages; those pages live in pinned host memory (the cold tier, `KVCache.kv` of a plan
with `hisparse=True`).  The device holds, per layer and per sequence slot, `hot_rows` latent rows plus the tables that map key
positions to hot rows and back.  Each decode step the indexer lists top-k key POSITIONS, `ops.hisparse_stage` makes them
resident (copying the missing rows from the cold tier) and returns hot row ids, the sparse attention kernel reads the hot
buffer, and the new token's row is written to the hot buffer and copied back to the cold tier.  The indexer's own key cache
(132 bytes per token and layer) stays on the device under the logical pages.

Capacity: a sequence costs `hot_rows * row_bytes * layers` of device memory whatever its length (4096 x 576 B x 61 = 144 MB
for DeepSeek-V3.2) plus 132 B per token and layer for the indexer keys, against 576 B per token and layer for a resident
cache: a 1M-token context needs 8 GB of device memory instead of 35 GB.

Parity: reference runtime/context/cache/hisparse.py:154-221 (context tensors), :294-316 (remap hooks), :352-391 (ring
buffers), capacity planner runtime/context/cache/__init__.py:44-150, docs/hisparse-design.md.
"""
from __future__ import annotations

from typing import Dict, List

import torch


class HiSparseTier:
    def __init__(self, num_layers: int, slots: int, hot_rows: int, max_ctx: int, row_bytes: int, cold_layers: List[torch.Tensor], device):
        """`cold_layers[l]`: the layer's logical pages [pages, page_rows, row] in (pinned) host memory.  One extra slot past
        `slots` is scratch for padded graph rows and dummy batches."""
        assert hot_rows % 64 == 0, "the hot buffer is read in 64-row tiles"
        self.L, self.slots, self.hot_rows, self.max_ctx, self.row_bytes = num_layers, slots, hot_rows, max_ctx, row_bytes
        self.device = torch.device(device)
        n = slots + 1
        self.scratch_slot = slots
        dev = self.device
        self.hot = torch.zeros(num_layers, n * hot_rows, row_bytes, dtype=torch.uint8, device=dev)
        self.pos_to_hot = torch.full((num_layers, n, max_ctx), -1, dtype=torch.int32, device=dev)
        self.hot_to_pos = torch.full((num_layers, n, hot_rows), -1, dtype=torch.int32, device=dev)
        self.stamp = torch.zeros(num_layers, n, hot_rows, dtype=torch.int32, device=dev)
        self.cursor = torch.zeros(num_layers, n, dtype=torch.int32, device=dev)
        self.step = torch.zeros(num_layers, 2, dtype=torch.int32, device=dev)
        self.cold = [c.view(torch.uint8) if c.dtype != torch.uint8 else c for c in cold_layers]
        self.page_rows = cold_layers[0].shape[1]
        self.owner: Dict[int, int] = {}
        self.loads = 0               # bookkeeping for tests and metrics: sequences whose slot was (re)initialised

    def device_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.hot, self.pos_to_hot, self.hot_to_pos, self.stamp, self.cursor, self.step))

    def layer(self, l: int) -> dict:
        return {"pos_to_hot": self.pos_to_hot[l], "hot_to_pos": self.hot_to_pos[l], "stamp": self.stamp[l], "cursor": self.cursor[l],
                "step": self.step[l], "cold": self.cold[l], "hot": self.hot[l], "page_rows": self.page_rows}

    def hot_pages(self, l: int, dtype) -> torch.Tensor:
        """The layer's hot rows as the [pages, 64, row] cache the attention kernels take."""
        t = self.hot[l].view(-1, 64, self.row_bytes)
        return t.view(dtype) if dtype != torch.uint8 else t

    def assign(self, slot: int, seq_id: int) -> None:
        """Called for every (slot, sequence) of a step before it runs: a slot that changes hands starts empty."""
        if slot < 0 or self.owner.get(slot) == seq_id:
            return
        self.owner[slot] = seq_id
        self.pos_to_hot[:, slot].fill_(-1)
        self.hot_to_pos[:, slot].fill_(-1)
        self.cursor[:, slot].zero_()
        self.loads += 1
