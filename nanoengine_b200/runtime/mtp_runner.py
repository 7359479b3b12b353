"""MTP speculative decoding on the worker.

Every decode step verifies the N draft tokens of each sequence in one target forward ("lazy verify": rows
[last token, d1..dN] per sequence, sequence-major, q_len = N+1), accepts the longest matching prefix (greedy) or
runs one-coin-per-position rejection sampling (stochastic), emits the accepted drafts plus one more token, and then lets
the MTP predictor produce the next N drafts: first a "draft-extend" pass over the newly accepted tokens (which also fills
the predictor's own KV rows, kept in cache layers after the target's), then N-1 recurrent single-token passes.
Drafts live in a device hand-off table ``[slots + 1, N+1]`` indexed by the scheduler's hand-off slot (the extra row is
scratch for rows without a slot), so the controller never sees them; a PD hand-off publishes/restores one row.

A verify step is one fixed-shape device pipeline with no host synchronisation inside it: the target pass over B x (N+1)
rows, lm_head, the verify kernels (accepted count, next token, emitted bundle, predictor inputs), the predictor's
draft-extend pass over the same B x (N+1) rows (rows past the accepted prefix compute values nobody reads and write
predictor-KV rows that the next step overwrites), a gather of the row at the accepted count, and the N-1 chain passes
whose positions and cache slots are built on the device from the accepted counts.  The step ends with ONE device->host
copy (the emitted bundle).  Fixed shapes make the whole pipeline capturable: ``MTPGraphRunner`` replays it as one CUDA
graph per batch-size bucket.

Parity: reference runtime/runner/mtp_runner.py - linear_rejection_sample :111-187, linear_greedy_verify :190-208,
hand-off publish/restore :249-394, prepare_lazy_verify_decode :491-534, lazy_verify_sample :536-624,
generate_and_store :626-751, prefill drafts :834-987, collective padding for idle DP ranks :1374-1427.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch

from .._native import _core as C
from .context import ForwardContext


from ..ops.reference import mtp_greedy_verify as linear_greedy_verify          # noqa: E402  (the numerics live with the operators;
from ..ops.reference import mtp_rejection_sample as linear_rejection_sample   # noqa: E402   these names are the reference's)


class MTPRunner:
    def __init__(self, runner, force_accept: Optional[int] = None):
        self.r = runner
        self.N = runner.config.num_speculative_tokens
        self.force_accept = force_accept          # benchmarking aid: pretend exactly this many drafts match
        slots = max(1, runner.config.max_num_seqs)
        dev = runner.device
        # [:, 0] = valid flag, [:, 1:] = drafts; row `slots` is scratch (rows of a batch that have no hand-off slot write there)
        self.handoff = torch.zeros(slots + 1, self.N + 1, dtype=torch.int64, device=dev)
        self.scratch_row = slots
        self.mtp_layer0 = runner.mc.num_hidden_layers     # predictor KV rows live in cache layers after the target's
        self.accepted_total = 0
        self.verify_steps = 0
        self.seed_buf = torch.full((1,), 0x5eed + 7919 * runner.dist.attn_dp_rank, dtype=torch.int64, device=dev)
        self.graphs = None                        # MTPGraphRunner, set by the worker when CUDA graphs are on
        self.d2h_per_step = 0

    # ---- PD hand-off -----------------------------------------------------------------------------
    def publish_handoff(self, slot: int) -> List[int]:
        return self.handoff[slot].tolist()

    def restore_handoff(self, slot: int, row: List[int]) -> None:
        self.handoff[slot] = torch.tensor(row, dtype=torch.int64, device=self.handoff.device)

    def invalidate_handoff(self, slot: int) -> None:
        self.handoff[slot, 0] = 0

    # ---- helpers ---------------------------------------------------------------------------------
    def _ctx_rows(self, b, q_lens: List[int], seq_lens: List[int], positions: List[int]) -> ForwardContext:
        """A forward context for `q_lens[i]` rows per sequence ending at context length `seq_lens[i]`."""
        bb = C.RunnerIn()
        bb.is_prefill = True
        bb.seq_ids = list(b.seq_ids)
        bb.q_lens, bb.seq_lens, bb.positions = q_lens, seq_lens, positions
        bb.input_ids = [0] * len(positions)
        bb.block_tables, bb.block_offsets = list(b.block_tables), list(b.block_offsets)
        bb.temperatures = list(b.temperatures)
        bb.sample_mask = [1] * len(q_lens)
        bb.state_slots, bb.handoff_slots, bb.hisparse_slots = list(b.state_slots), list(b.handoff_slots), list(b.hisparse_slots)
        return self.r.prepare(bb)

    def _argmax(self, logits: torch.Tensor) -> torch.Tensor:
        from .. import ops
        z = torch.zeros(logits.shape[0], dtype=torch.float32, device=logits.device)
        return ops.sample(logits, z)[0]

    def _chain_ctx(self, ctx: ForwardContext, B: int, pos, slot, lens) -> ForwardContext:
        """One new row per sequence at the positions / cache slots the chain-metadata kernel wrote."""
        dev = self.r.device
        return ForwardContext(is_prefill=False, num_seqs=B, num_tokens=B, cu_seqlens_q=torch.arange(B + 1, dtype=torch.int32, device=dev),
                              context_lens=lens, slot_mapping=slot, block_tables=ctx.block_tables, max_seqlen_q=1,
                              max_seqlen_k=ctx.max_seqlen_k + self.N, last_token_indices=None, q_len_uniform=1,
                              kv_caches=self.r.cache.layers, indexer_caches=self.r.cache.indexer_layers)

    def _draft_chain(self, ctx: ForwardContext, B: int, h: torch.Tensor, tok: torch.Tensor, base_len: torch.Tensor, acc: torch.Tensor,
                     bufs=None) -> torch.Tensor:
        """Recurrent drafts 2..N: the predictor consumes its own output.  Draft k's input row sits at position
        base_len + acc + k - 1 (the row after the last one the predictor has seen); everything stays on the device."""
        from .. import ops
        dev = self.r.device
        bs = self.r.plan.block_size
        drafts = [tok]
        for k in range(1, self.N):
            if bufs is None:
                pos = torch.empty(B, dtype=torch.int64, device=dev)
                slot = torch.empty(B, dtype=torch.int64, device=dev)
                lens = torch.empty(B, dtype=torch.int32, device=dev)
            else:
                pos, slot, lens = bufs[k - 1]
            ops.mtp_chain_meta(base_len, acc, ctx.block_tables, bs, k, pos, slot, lens)
            cctx = self._chain_ctx(ctx, B, pos, slot, lens)
            h = self.r.mtp(tok, h, pos, cctx, step=0)
            tok = self._argmax(self.r.mtp.compute_logits(h))
            drafts.append(tok)
        return torch.stack(drafts, 1)              # [B, N]

    # ---- one step --------------------------------------------------------------------------------
    @torch.inference_mode()
    def run(self, b, ctx: ForwardContext):
        if b.is_prefill:
            return self._run_prefill(b, ctx)
        return self._run_verify(b)

    def run_dummy(self, ctx: ForwardContext):
        """Idle DP rank: mirror the predictor passes so expert-parallel collectives stay matched across ranks."""
        ids, pos = ctx.extras["input_ids"], ctx.extras["positions"]
        h = torch.zeros(ids.numel(), self.r.mc.hidden_size, dtype=self.r.dtype, device=self.r.device)
        for _ in range(self.N):
            h = self.r.mtp(ids, h, pos, ctx, step=0)

    def _run_prefill(self, b, ctx: ForwardContext):
        r = self.r
        ids, pos = ctx.extras["input_ids"], ctx.extras["positions"]
        hidden = r.model(ids, pos, ctx)
        mask = np.asarray(b.sample_mask, dtype=bool)
        temps = torch.tensor(list(b.temperatures), dtype=torch.float32, device=r.device)
        rows = ctx.last_token_indices.long()
        logits = r.model.compute_logits(hidden[rows])
        tok, lp = r.sampler(logits, temps, b.any_return_logprobs)
        # predictor over the chunk: token i pairs with the hidden state of position i-1, so inputs are the ids shifted left
        # with the freshly sampled token (or, for a non-final chunk, a placeholder that the next chunk overwrites) at the end
        shifted = torch.roll(ids, -1)
        shifted[rows] = tok
        h_mtp = r.mtp(shifted, hidden, pos, ctx, step=0)
        d1 = self._argmax(r.mtp.compute_logits(h_mtp[rows]))
        B = b.num_seqs
        base_len = torch.tensor([int(s) for s in b.seq_lens], dtype=torch.int32, device=r.device)
        zero = torch.zeros(B, dtype=torch.int32, device=r.device)
        drafts = self._draft_chain(ctx, B, h_mtp[rows], d1, base_len, zero) if self.N > 1 else d1.unsqueeze(1)
        slots = torch.tensor(list(b.handoff_slots), dtype=torch.long, device=r.device)
        done = torch.from_numpy(mask).to(r.device)
        srow = torch.where(done & (slots >= 0), slots, torch.full_like(slots, self.scratch_row))
        self.handoff.index_copy_(0, srow, torch.cat([torch.ones_like(drafts[:, :1]), drafts], 1))
        toks = tok.tolist()
        lps = lp.tolist() if lp is not None else None
        ids_out = [s for s, m in zip(b.seq_ids, mask) if m]
        return C.RunnerOut(ids_out, [[toks[i]] for i in range(len(toks)) if mask[i]],
                           None if lps is None else [[lps[i]] for i in range(len(lps)) if mask[i]])

    def device_step(self, ctx: ForwardContext, B: int, last: torch.Tensor, slots: torch.Tensor, temps: torch.Tensor, base_len: torch.Tensor,
                    want_logprob: bool = False, chain_bufs=None, target_forward=None):
        """The verify step on the device (see the module docstring).  `last` int64 [B] last token of every sequence, `slots`
        int64 [B] hand-off slots (-1 = none), `temps` fp32 [B], `base_len` int32 [B] context length including the last token.
        Returns (bundle int64 [B, N+1], num_accepted int32 [B], logprob fp32 [B] or None); nothing is read back here."""
        from .. import ops
        r, N = self.r, self.N
        srow = torch.where(slots >= 0, slots, torch.full_like(slots, self.scratch_row))
        row = self.handoff[srow]
        have = ((row[:, 0] == 1) & (slots >= 0)).to(torch.int32)
        drafts = row[:, 1:] * have.unsqueeze(1).to(torch.int64)                                # sequences without drafts verify zeros
        rows_ids = torch.cat([last.unsqueeze(1), drafts], 1).reshape(-1)                       # [B*(N+1)]
        pos = ctx.extras["positions"]
        hidden = (target_forward or r.model)(rows_ids, pos, ctx)                               # [B*(N+1), H]
        logits = r.model.compute_logits(hidden).view(B, N + 1, -1)
        self.seed_buf.add_(1)
        acc, nxt, bundle, ext, lp = ops.mtp_verify(logits, drafts, temps, have, None, r.sampler.gen, self.force_accept, want_logprob,
                                                   seed_buf=self.seed_buf if logits.is_cuda else None)
        # next drafts: the predictor runs over every verify row with the tokens the verify kernel laid out; the row at the
        # accepted count carries the hidden state the chain continues from
        h_mtp = r.mtp(ext.reshape(-1), hidden, pos, ctx, step=0)
        sel = torch.arange(B, device=hidden.device) * (N + 1) + acc.long()
        h_last = h_mtp.index_select(0, sel)
        d1 = self._argmax(r.mtp.compute_logits(h_last))
        nd = self._draft_chain(ctx, B, h_last, d1, base_len, acc, chain_bufs) if N > 1 else d1.unsqueeze(1)
        # one indexed row copy, every operand already on the device (a Python scalar here would be a host->device copy, which a
        # stream capture refuses); rows without a slot all land on the scratch row
        self.handoff.index_copy_(0, srow, torch.cat([torch.ones_like(nd[:, :1]), nd], 1))
        return bundle, acc, lp

    def _run_verify(self, b):
        r, N = self.r, self.N
        B = b.num_seqs
        n0 = list(b.seq_lens)                                                                   # context length incl. the last token
        positions = [p for n in n0 for p in range(n - 1, n + N)]
        ctx = self._ctx_rows(b, [N + 1] * B, [n + N for n in n0], positions)
        want_lp = bool(b.any_return_logprobs)
        h2d = np.asarray([list(b.input_ids), list(b.handoff_slots), n0], dtype=np.int64)      # one copy: last tokens, slots, lengths
        dev_i = r._to_dev(h2d)
        temps = r._to_dev(np.asarray(list(b.temperatures), dtype=np.float32))
        last, slots, base_len = dev_i[0], dev_i[1], dev_i[2].to(torch.int32)
        self._last = (ctx, B, last, slots, temps, base_len)
        if self.graphs is not None and not want_lp and self.graphs.can_run(ctx):
            bundle, acc = self.graphs.run(ctx, last, slots, temps, base_len)
            lp = None
        else:
            bundle, acc, lp = self.device_step(ctx, B, last, slots, temps, base_len, want_lp)
        # the single device->host copy of the step
        out = torch.cat([bundle, acc.to(torch.int64).unsqueeze(1)], 1).tolist()
        r.d2h_bytes += B * (N + 2) * 8
        lpl = lp.tolist() if lp is not None else None
        if lp is not None:
            r.d2h_bytes += B * 4
        acc_l = [row[-1] for row in out]
        self.accepted_total += sum(acc_l)
        self.verify_steps += B
        r._check_kernel_status()
        out_tokens = [row[: a + 1] for row, a in zip(out, acc_l)]
        lps = None
        if lpl is not None:
            lps = [[0.0] * a + [lpl[i]] for i, a in enumerate(acc_l)]
        return C.RunnerOut(list(b.seq_ids), out_tokens, lps)


    # ---- benchmark helpers ------------------------------------------------------------------------
    @torch.inference_mode()
    def make_resident_step(self):
        """A closure that repeats the most recent verify step on inputs already on the device (the same rows are verified and
        their KV rewritten every time, which costs what a fresh step costs)."""
        if getattr(self, "_last", None) is None:
            raise RuntimeError("run a verify step first")
        ctx, B, last, slots, temps, base_len = self._last

        @torch.inference_mode()
        def step():
            if self.graphs is not None and self.graphs.can_run(ctx):
                return self.graphs.run(ctx, last, slots, temps, base_len)[0]
            return self.device_step(ctx, B, last, slots, temps, base_len)[0]

        return step

    @torch.inference_mode()
    def count_step_launches(self) -> int:
        from ..ops import sm100
        ctx, B, last, slots, temps, base_len = self._last
        before = sm100.LAUNCHES[0]
        self.device_step(ctx, B, last, slots, temps, base_len)
        torch.cuda.synchronize()
        return sm100.LAUNCHES[0] - before


class MTPGraphRunner:
    """The verify step of `MTPRunner` as one CUDA graph per batch-size bucket: persistent input buffers (N+1 rows per
    sequence), the whole device pipeline captured once, replayed with fresh inputs.  Rows past the live batch are padding on
    the scratch page without a hand-off slot.  Covers what the reference splits over three runners - lazy verify, the cached
    draft chain and the predictor pass (runtime/runner/graph_runner.py:548-718, :726-953, :956-1054)."""

    def __init__(self, runner, mtp: "MTPRunner"):
        from .graph_runner import DecodeGraphRunner
        self.r, self.m = runner, mtp
        self.N = mtp.N
        self.base = DecodeGraphRunner(runner, q_len=self.N + 1)          # buffers, buckets and padding rules are those of decode
        dev = runner.device
        mb = self.base.max_bs
        self.last = torch.zeros(mb, dtype=torch.int64, device=dev)
        self.slots = torch.full((mb,), -1, dtype=torch.int64, device=dev)
        self.temps = torch.zeros(mb, dtype=torch.float32, device=dev)
        self.base_len = torch.ones(mb, dtype=torch.int32, device=dev)
        self.chain = [(torch.zeros(mb, dtype=torch.int64, device=dev), torch.zeros(mb, dtype=torch.int64, device=dev),
                       torch.ones(mb, dtype=torch.int32, device=dev)) for _ in range(max(0, self.N - 1))]
        self.graphs, self.outputs = {}, {}
        self.pool = None

    def can_run(self, ctx: ForwardContext) -> bool:
        return self.base.can_run(ctx)

    def _step(self, b: int):
        sctx = self.base._static_ctx(b)
        sctx.extras["positions"] = self.base.positions[: b * (self.N + 1)]
        bufs = [(p[:b], s[:b], l[:b]) for p, s, l in self.chain]
        bundle, acc, _ = self.m.device_step(sctx, b, self.last[:b], self.slots[:b], self.temps[:b], self.base_len[:b], False, bufs)
        return bundle, acc

    def _pad(self, n: int, b: int):
        if n < b:
            self.last[n:b].zero_()
            self.slots[n:b].fill_(-1)
            self.temps[n:b].zero_()
            self.base_len[n:b].fill_(1)

    def _capture(self, b: int):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._step(b)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=self.pool):
            out = self._step(b)
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[b], self.outputs[b] = g, out

    def capture_all(self) -> None:
        """Collective when the model has EP / TP groups: every rank captures every bucket, largest first, on padding rows."""
        for b in sorted(self.base.bs_list, reverse=True):
            if b not in self.graphs:
                self.base._fill_padding_only(b)
                self._pad(0, b)
                self._capture(b)

    def run(self, ctx: ForwardContext, last, slots, temps, base_len):
        n = ctx.num_seqs
        b = self.base.bucket(n)
        self.base._fill(torch.zeros(n * (self.N + 1), dtype=torch.long, device=last.device), ctx.extras["positions"], ctx, b)
        self.last[:n].copy_(last); self.slots[:n].copy_(slots); self.temps[:n].copy_(temps); self.base_len[:n].copy_(base_len)
        self._pad(n, b)
        if b not in self.graphs:
            if self.r.has_collectives():
                raise RuntimeError(f"verify graph for batch bucket {b} was not captured at start-up")
            # the warm-up passes are real steps on the live rows: keep the drafts they would consume and restore them afterwards
            saved = self.m.handoff.clone()
            seed = self.m.seed_buf.clone()
            self._capture(b)
            self.m.handoff.copy_(saved)
            self.m.seed_buf.copy_(seed)
        self.graphs[b].replay()
        bundle, acc = self.outputs[b]
        return bundle[:n], acc[:n]
