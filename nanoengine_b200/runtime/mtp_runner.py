"""MTP speculative decoding on the worker.

Every decode step verifies the N draft tokens of each sequence in one target forward ("lazy verify": rows
[last token, d1..dN] per sequence, sequence-major, q_len = N+1), accepts the longest matching prefix (greedy) or
runs one-coin-per-position rejection sampling (stochastic), emits the accepted drafts plus one more token, and then lets
the MTP predictor produce the next N drafts: first a "draft-extend" pass over the newly accepted tokens (which also fills
the predictor's own KV rows, kept in cache layers after the target's), then N-1 recurrent single-token passes.
Drafts live in a device hand-off table ``[slots, N+1]`` indexed by the scheduler's hand-off slot, so the controller never
sees them; a PD hand-off publishes/restores one row.

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


def linear_greedy_verify(logits: torch.Tensor, drafts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits [B, N+1, V], drafts [B, N].  Returns (num_accepted [B] in 0..N, next_token [B]): the longest prefix with
    argmax(row_i) == d_{i+1}; the next token is the argmax of the first mismatching row, or of the bonus row."""
    B, N1, _ = logits.shape
    am = logits.argmax(-1)                                   # [B, N+1]
    match = (am[:, :-1] == drafts).to(torch.int64)
    acc = match.cumprod(1).sum(1)                            # [B]
    nxt = am.gather(1, acc.unsqueeze(1)).squeeze(1)
    return acc, nxt


def linear_rejection_sample(logits: torch.Tensor, drafts: torch.Tensor, temperatures: torch.Tensor,
                            generator: Optional[torch.Generator] = None, uniforms: Optional[torch.Tensor] = None):
    """Speculative sampling for greedy (one-hot) drafts.

    Draft d_{i+1} is accepted with probability p_target(d_{i+1} | row i), one uniform coin per position; the accepted count
    is the length of the all-accepted prefix.  The next token is sampled from the target row at the first rejection with the
    rejected draft masked out (from the bonus row, unmasked, when everything was accepted) - which preserves the target
    distribution.  Rows with temperature < 1e-5 fall back to greedy verification.
    Returns (num_accepted [B], next_token [B], logprob_of_next [B] under the unmasked target row).
    """
    B, N1, V = logits.shape
    N = N1 - 1
    greedy = temperatures < 1e-5
    t = torch.where(greedy, torch.ones_like(temperatures), temperatures).view(B, 1, 1)
    logp = torch.log_softmax(logits.float() / t, -1)          # [B, N+1, V]
    p_draft = logp[:, :N].gather(2, drafts.long().unsqueeze(-1)).squeeze(-1).exp()    # [B, N]
    if uniforms is None:
        uniforms = torch.rand(B, N, generator=generator, device=logits.device, dtype=torch.float32)
    accept = (uniforms < p_draft).to(torch.int64)
    acc = accept.cumprod(1).sum(1)
    row = logp.gather(1, acc.view(B, 1, 1).expand(B, 1, V)).squeeze(1)               # target row at the stop position
    masked = row.clone()
    rejected = acc < N
    if N > 0:
        rej_tok = drafts.long().gather(1, acc.clamp_max(N - 1).unsqueeze(1)).squeeze(1)
        masked[rejected, rej_tok[rejected]] = float("-inf")
    u = torch.rand(B, V, generator=generator, device=logits.device, dtype=torch.float32).clamp_min(1e-20)
    nxt = (masked - torch.log(-torch.log(u))).argmax(-1)
    g_acc, g_nxt = linear_greedy_verify(logits, drafts)
    acc = torch.where(greedy, g_acc, acc)
    nxt = torch.where(greedy, g_nxt, nxt)
    row = logp.gather(1, acc.view(B, 1, 1).expand(B, 1, V)).squeeze(1)
    return acc, nxt, row.gather(1, nxt.unsqueeze(1)).squeeze(1)


class MTPRunner:
    def __init__(self, runner, force_accept: Optional[int] = None):
        self.r = runner
        self.N = runner.config.num_speculative_tokens
        self.force_accept = force_accept          # benchmarking aid: pretend exactly this many drafts match
        slots = max(1, runner.config.max_num_seqs)
        self.handoff = torch.zeros(slots, self.N + 1, dtype=torch.int64, device=runner.device)   # [:, 0] = valid flag, [:, 1:] = drafts
        self.mtp_layer0 = runner.mc.num_hidden_layers     # predictor KV rows live in cache layers after the target's
        self.accepted_total = 0
        self.verify_steps = 0

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

    def _draft_chain(self, b, hidden_last: torch.Tensor, first_tokens: torch.Tensor, base_lens: List[int]) -> torch.Tensor:
        """Recurrent drafts 2..N: the predictor consumes its own output.  `base_lens[i]` = context length after draft 1's row."""
        drafts = [first_tokens]
        h = hidden_last
        tok = first_tokens
        for k in range(1, self.N):
            lens = [n + k for n in base_lens]
            ctx = self._ctx_rows(b, [1] * len(lens), lens, [n - 1 for n in lens])
            ctx.kv_caches = self.r.cache.layers
            h = self.r.mtp(tok, h, ctx.extras["positions"], ctx, step=0)
            tok = self.r.mtp.compute_logits(h).argmax(-1)
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
        cu = ctx.cu_seqlens_q_host
        temps = torch.tensor(list(b.temperatures), dtype=torch.float32, device=r.device)
        rows = ctx.last_token_indices.long()
        logits = r.model.compute_logits(hidden[rows])
        tok, lp = r.sampler(logits, temps, b.any_return_logprobs)
        # predictor over the chunk: token i pairs with the hidden state of position i-1, so inputs are the ids shifted left
        # with the freshly sampled token (or, for a non-final chunk, a placeholder that the next chunk overwrites) at the end
        shifted = torch.roll(ids, -1)
        shifted[rows] = tok
        h_mtp = r.mtp(shifted, hidden, pos, ctx, step=0)
        d1 = r.mtp.compute_logits(h_mtp[rows]).argmax(-1)
        base_lens = [int(s) + 1 for s in b.seq_lens]
        drafts = self._draft_chain(b, h_mtp[rows], d1, base_lens) if self.N > 1 else d1.unsqueeze(1)
        slots = torch.tensor(list(b.handoff_slots), dtype=torch.long, device=r.device)
        done = torch.from_numpy(mask).to(r.device)
        valid = slots >= 0
        sel = done & valid
        if bool(sel.any()):
            self.handoff[slots[sel], 1:] = drafts[sel]
            self.handoff[slots[sel], 0] = 1
        toks = tok.tolist()
        lps = lp.tolist() if lp is not None else None
        ids_out = [s for s, m in zip(b.seq_ids, mask) if m]
        return C.RunnerOut(ids_out, [[toks[i]] for i in range(len(toks)) if mask[i]],
                           None if lps is None else [[lps[i]] for i in range(len(lps)) if mask[i]])

    def _run_verify(self, b):
        r, N = self.r, self.N
        B = b.num_seqs
        slots = torch.tensor(list(b.handoff_slots), dtype=torch.long, device=r.device)
        row = self.handoff[slots.clamp_min(0)]
        have = (row[:, 0] == 1) & (slots >= 0)
        drafts = torch.where(have.unsqueeze(1), row[:, 1:], torch.zeros_like(row[:, 1:]))     # sequences without drafts verify zeros
        last = torch.tensor(list(b.input_ids), dtype=torch.long, device=r.device)
        rows_ids = torch.cat([last.unsqueeze(1), drafts], 1).reshape(-1)                       # [B*(N+1)]
        n0 = list(b.seq_lens)                                                                   # context length incl. the last token
        q_lens = [N + 1] * B
        seq_lens = [n + N for n in n0]
        positions = [p for n in n0 for p in range(n - 1, n + N)]
        ctx = self._ctx_rows(b, q_lens, seq_lens, positions)
        pos = ctx.extras["positions"]
        hidden = r.model(rows_ids, pos, ctx)                                                   # [B*(N+1), H]
        logits = r.model.compute_logits(hidden).view(B, N + 1, -1)
        temps = torch.tensor(list(b.temperatures), dtype=torch.float32, device=r.device)
        if bool((temps < 1e-5).all()):
            acc, nxt = linear_greedy_verify(logits, drafts)
            lp = None
            if b.any_return_logprobs:
                lpr = torch.log_softmax(logits.float(), -1)
                lp = lpr.gather(1, acc.view(B, 1, 1).expand(B, 1, lpr.shape[-1])).squeeze(1).gather(1, nxt.unsqueeze(1)).squeeze(1)
        else:
            acc, nxt, lp = linear_rejection_sample(logits, drafts, temps, r.sampler.gen)
        acc = torch.where(have, acc, torch.zeros_like(acc))
        if self.force_accept is not None:
            acc = torch.full_like(acc, min(self.force_accept, N))
            nxt = logits.argmax(-1).gather(1, acc.unsqueeze(1)).squeeze(1)
        acc_l, nxt_l = acc.tolist(), nxt.tolist()
        dr_l = drafts.tolist()
        self.accepted_total += sum(acc_l)
        self.verify_steps += B
        # next drafts: draft-extend over the a+1 new tokens (their hidden states come from the verify pass), then the chain
        ext_q = [a + 1 for a in acc_l]
        ext_lens = [n + a for n, a in zip(n0, acc_l)]
        ext_pos = [p for n, a in zip(n0, acc_l) for p in range(n - 1, n + a)]
        ectx = self._ctx_rows(b, ext_q, ext_lens, ext_pos)
        sel_rows, new_tok = [], []
        for i, a in enumerate(acc_l):
            base = i * (N + 1)
            sel_rows.extend(range(base, base + a + 1))
            new_tok.extend(dr_l[i][:a] + [nxt_l[i]])
        sel = torch.tensor(sel_rows, dtype=torch.long, device=r.device)
        tok_in = torch.tensor(new_tok, dtype=torch.long, device=r.device)
        h_mtp = r.mtp(tok_in, hidden[sel], ectx.extras["positions"], ectx, step=0)
        last_rows = ectx.last_token_indices.long()
        d1 = r.mtp.compute_logits(h_mtp[last_rows]).argmax(-1)
        base_lens = [n + a + 1 for n, a in zip(n0, acc_l)]
        nd = self._draft_chain(b, h_mtp[last_rows], d1, base_lens) if N > 1 else d1.unsqueeze(1)
        ok = slots >= 0
        if bool(ok.any()):
            self.handoff[slots[ok], 1:] = nd[ok]
            self.handoff[slots[ok], 0] = 1
        out_tokens = [dr_l[i][:acc_l[i]] + [nxt_l[i]] for i in range(B)]
        lps = None
        if lp is not None:
            lpl = lp.tolist()
            lps = [[0.0] * acc_l[i] + [lpl[i]] for i in range(B)]
        return C.RunnerOut(list(b.seq_ids), out_tokens, lps)
