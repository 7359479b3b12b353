"""Pipeline-parallel helpers for the static, forward-only prefill pipeline: layer partition, stage boundary transfers and
micro-batch splitting.

Parity: reference models/pp_utils.py:24-73 (pp_layer_partition), :271-346 (pp_isend / pp_irecv of hidden states),
engine/llm_engine.py:224-330 (engine-side micro-batch pipeline), engine/scheduler.py:25-41 (token budget x depth).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from .._native import _core as C


def pp_layer_partition(num_layers: int, pp: int) -> List[Tuple[int, int]]:
    """Contiguous, balanced ranges; earlier stages take the remainder (the last stage also carries norm + lm_head)."""
    if pp < 1 or pp > num_layers:
        raise ValueError(f"cannot split {num_layers} layers over {pp} stages")
    base, rem = divmod(num_layers, pp)
    out, lo = [], 0
    for s in range(pp):
        n = base + (1 if s < rem else 0)
        out.append((lo, lo + n))
        lo += n
    return out


def pp_send(h: torch.Tensor, residual, dst: int, group=None) -> None:
    """Stage boundary: [h ; residual] in one message (residual is None only in front of the first layer)."""
    if residual is None:
        residual = torch.zeros_like(h)
    dist.send(torch.stack([h, residual]).contiguous(), dst, group=group)


def pp_recv(num_tokens: int, hidden: int, dtype, device, src: int, group=None):
    buf = torch.empty(2, num_tokens, hidden, dtype=dtype, device=device)
    dist.recv(buf, src, group=group)
    return buf[0], buf[1]


def split_batch(b, parts: int) -> List["C.RunnerIn"]:
    """Split a prefill batch into at most `parts` micro-batches along sequence boundaries, balancing token counts."""
    n = b.num_seqs
    if n == 0 or parts <= 1:
        return [b]
    parts = min(parts, n)
    total = sum(b.q_lens)
    target = total / parts
    groups, cur, acc = [], [], 0
    for i in range(n):
        cur.append(i)
        acc += b.q_lens[i]
        if acc >= target * (len(groups) + 1) and len(groups) < parts - 1:
            groups.append(cur)
            cur = []
    if cur:
        groups.append(cur)
    tok_off = [0]
    for q in b.q_lens:
        tok_off.append(tok_off[-1] + q)
    out = []
    for g in groups:
        m = C.RunnerIn()
        m.is_prefill, m.is_dummy, m.any_return_logprobs, m.dp_idx, m.step = b.is_prefill, b.is_dummy, b.any_return_logprobs, b.dp_idx, b.step
        m.seq_ids = [b.seq_ids[i] for i in g]
        m.q_lens = [b.q_lens[i] for i in g]
        m.seq_lens = [b.seq_lens[i] for i in g]
        m.input_ids = [t for i in g for t in b.input_ids[tok_off[i]:tok_off[i + 1]]]
        m.positions = [t for i in g for t in b.positions[tok_off[i]:tok_off[i + 1]]]
        bt, bo = [], [0]
        for i in g:
            bt.extend(b.block_tables[b.block_offsets[i]:b.block_offsets[i + 1]])
            bo.append(len(bt))
        m.block_tables, m.block_offsets = bt, bo
        m.temperatures = [b.temperatures[i] for i in g]
        m.sample_mask = [b.sample_mask[i] for i in g]
        m.state_slots = [b.state_slots[i] for i in g]
        m.handoff_slots = [b.handoff_slots[i] for i in g]
        m.hisparse_slots = [b.hisparse_slots[i] for i in g]
        out.append(m)
    if b.swap_in_src or b.swap_out_src:
        out[0].swap_in_src, out[0].swap_in_dst = list(b.swap_in_src), list(b.swap_in_dst)
        out[0].swap_out_src, out[0].swap_out_dst = list(b.swap_out_src), list(b.swap_out_dst)
    return out
