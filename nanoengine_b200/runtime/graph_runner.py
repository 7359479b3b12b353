"""CUDA-graph replay of the decode forward pass.

One graph per batch-size bucket (1, 2, 4, 8, then multiples of 16 up to ``cuda_graph_max_bs``), captured after an
eager warm-up of the same shape, all sharing one memory pool and one set of persistent input buffers.
Rows beyond the live batch point at the scratch page with context length 1, so a padded replay is valid work
that touches no live sequence.

When the forward pass contains collectives (expert- or tensor-parallel groups), every bucket is captured up front by
``capture_all`` - all ranks run it at start-up in the same order, so the warm-up passes and the captures, each of which
executes the collectives for real, stay matched across ranks.  A rank must never capture on its own later: its peers
would be replaying one round of collectives against its three.  Without collectives, buckets are captured on first use.

Parity: reference runtime/runner/graph_runner.py:55 (_make_bs_list), :65-540 (DecodeGraphRunner: persistent
buffers, shared pool, capture per size, run).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .context import ForwardContext


def make_bs_list(max_bs: int) -> List[int]:
    out = [b for b in (1, 2, 4, 8) if b <= max_bs]
    out += list(range(16, max_bs + 1, 16))
    if max_bs not in out:
        out.append(max_bs)
    return sorted(set(out))


class DecodeGraphRunner:
    def __init__(self, runner, q_len: int = 1):
        self.r = runner
        self.q_len = q_len
        cfg = runner.config
        self.max_bs = min(cfg.cuda_graph_max_bs, cfg.max_num_seqs)
        self.bs_list = make_bs_list(self.max_bs)
        bs = runner.plan.block_size
        self.max_blocks = (cfg.max_model_len + bs - 1) // bs + 1
        dev = runner.device
        n = self.max_bs * q_len
        self.input_ids = torch.zeros(n, dtype=torch.long, device=dev)
        self.positions = torch.zeros(n, dtype=torch.long, device=dev)
        self.slot_mapping = torch.zeros(n, dtype=torch.long, device=dev)
        self.context_lens = torch.ones(self.max_bs, dtype=torch.int32, device=dev)
        self.block_tables = torch.zeros(self.max_bs, self.max_blocks, dtype=torch.int32, device=dev)
        self.cu_seqlens_q = (torch.arange(self.max_bs + 1, dtype=torch.int32, device=dev) * q_len)
        # recurrent-state models: slot of every row (padding rows and capture warm-ups use the scratch slot)
        self.gdn = runner.plan.gdn
        self.state_slots = torch.full((self.max_bs,), runner.cache.scratch_slot, dtype=torch.int32, device=dev)
        self.seq_fresh = torch.zeros(self.max_bs, dtype=torch.int32, device=dev)
        # hot / cold tier: hot-buffer slot of every row (padding rows use the tier's scratch slot)
        self.hs = runner.cache.hisparse
        self.hs_slots = torch.full((self.max_bs,), self.hs.scratch_slot if self.hs is not None else 0, dtype=torch.int32, device=dev)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.outputs: Dict[int, torch.Tensor] = {}
        self.pool = None

    def bucket(self, n: int) -> int:
        for b in self.bs_list:
            if b >= n:
                return b
        return -1

    def can_run(self, ctx: ForwardContext) -> bool:
        return (ctx.q_len_uniform == self.q_len and ctx.num_seqs <= self.max_bs and ctx.block_tables.shape[1] <= self.max_blocks
                and self.bucket(ctx.num_seqs) > 0)

    def _static_ctx(self, b: int) -> ForwardContext:
        q = self.q_len
        return ForwardContext(
            is_prefill=False, num_seqs=b, num_tokens=b * q, cu_seqlens_q=self.cu_seqlens_q[: b + 1], context_lens=self.context_lens[:b],
            slot_mapping=self.slot_mapping[: b * q], block_tables=self.block_tables[:b], max_seqlen_q=q,
            max_seqlen_k=self.r.config.max_model_len, last_token_indices=None, q_len_uniform=q,
            kv_caches=self.r.cache.layers, indexer_caches=self.r.cache.indexer_layers,
            state_slots=self.state_slots[:b] if self.gdn else None, seq_fresh=self.seq_fresh[:b] if self.gdn else None,
            conv_states=self.r.cache.conv_states, rec_states=self.r.cache.rec_states,
            hisparse=self.hs, hs_slots=self.hs_slots[:b] if self.hs is not None else None)

    def _fill(self, ids, pos, ctx: ForwardContext, b: int):
        n, q = ctx.num_seqs, self.q_len
        sb = self.r.cache.scratch_block
        self.input_ids[: n * q].copy_(ids)
        self.positions[: n * q].copy_(pos)
        self.slot_mapping[: n * q].copy_(ctx.slot_mapping)
        self.context_lens[:n].copy_(ctx.context_lens)
        w = ctx.block_tables.shape[1]
        self.block_tables[:n, :w].copy_(ctx.block_tables)
        if self.gdn:
            self.state_slots[:n].copy_(ctx.state_slots)
            self.seq_fresh[:n].copy_(ctx.seq_fresh)
            self.state_slots[n:b].fill_(self.r.cache.scratch_slot)
        if self.hs is not None:
            self.hs_slots[:n].copy_(ctx.hs_slots)
            self.hs_slots[n:b].fill_(self.hs.scratch_slot)
        if n < b:
            # padding rows: q_len tokens of a one-page sequence on the scratch page
            self.input_ids[n * q: b * q].zero_()
            self.positions[n * q: b * q].copy_(torch.arange(q, device=ids.device).repeat(b - n))
            self.slot_mapping[n * q: b * q].copy_(sb * self.r.plan.block_size + torch.arange(q, device=ids.device).repeat(b - n))
            self.context_lens[n:b].fill_(q)
            self.block_tables[n:b].fill_(sb)

    def _capture(self, b: int):
        sctx = self._static_ctx(b)
        q = self.q_len
        ids, pos = self.input_ids[: b * q], self.positions[: b * q]
        if self.gdn:
            # the warm-up runs execute real steps: point every row at the scratch slot so no live sequence's state advances
            # (rows sharing one slot race on it, which is harmless for scratch data); run() refills the live slots afterwards
            self.state_slots[:b].fill_(self.r.cache.scratch_slot)
        if self.hs is not None:
            self.hs_slots[:b].fill_(self.hs.scratch_slot)      # same for the hot buffers: the warm-ups stage into the scratch slot
        # eager warm-up on the side stream: sets kernel attributes, fills caches of derived weights, sizes the allocator
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self.r.model(ids, pos, sctx)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=self.pool):
            out = self.r.model(ids, pos, sctx)
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[b], self.outputs[b] = g, out

    def _fill_padding_only(self, b: int):
        """Every row of bucket `b` becomes a padding row: q_len tokens of a one-page sequence on the scratch page."""
        q = self.q_len
        sb = self.r.cache.scratch_block
        dev = self.input_ids.device
        self.input_ids[: b * q].zero_()
        self.positions[: b * q].copy_(torch.arange(q, device=dev).repeat(b))
        self.slot_mapping[: b * q].copy_(sb * self.r.plan.block_size + torch.arange(q, device=dev).repeat(b))
        self.context_lens[:b].fill_(q)
        self.block_tables[:b].fill_(sb)
        if self.gdn:
            self.state_slots[:b].fill_(self.r.cache.scratch_slot)
            self.seq_fresh[:b].fill_(1)
        if self.hs is not None:
            self.hs_slots[:b].fill_(self.hs.scratch_slot)

    def capture_all(self) -> None:
        """Capture every bucket now, largest first (the pool is sized once), on dummy rows.  Collective: all ranks of the
        model's EP / TP groups must call this at the same point.
        Parity: reference runtime/runner/graph_runner.py:298-455 (capture loop with a barrier per size)."""
        for b in sorted(self.bs_list, reverse=True):
            if b in self.graphs:
                continue
            self._fill_padding_only(b)
            self._capture(b)

    def run(self, ids, pos, ctx: ForwardContext) -> torch.Tensor:
        b = self.bucket(ctx.num_seqs)
        # the padding rows must be in place before a capture too: the warm-up runs on them
        self._fill(ids, pos, ctx, b)
        if b not in self.graphs:
            if self.r.has_collectives():
                raise RuntimeError(f"decode graph for batch bucket {b} was not captured at start-up; a rank of a parallel group "
                                   "must not capture on its own (its peers would not run the matching collectives)")
            self._capture(b)
            self._fill(ids, pos, ctx, b)
        self.graphs[b].replay()
        return self.outputs[b][: ctx.num_seqs * self.q_len]
