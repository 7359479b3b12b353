"""Context-parallel MLA decode: the KV pages of every sequence are dealt over the ranks of a group, each rank attends to its
own pages, and the partial results are merged by their log-sum-exp.

Page p of a sequence lives on rank ``p % cp`` (``shard_pages`` gives a rank's page list and token count), so a long context
is read by ``cp`` GPUs at once.  One decode step on every rank:

1. the tcgen05 fp8 MLA kernel runs over the local pages with ``local_splits`` key slices and leaves un-merged partial outputs
   (fp32, normalised per slice) and their log2-sum-exps;
2. both are pushed into every peer's gather buffer by the store kernels of the fused TP collectives (NVLink peer stores, a
   flag per source rank, bounded waits);
3. one merge kernel folds the ``cp * local_splits`` slices of every (token, head) row.

Every rank must pass the same queries (a data-parallel caller all-gathers them first) and ends with the full result.  The
steps are stream-ordered kernels, so the sequence can be captured in a CUDA graph.

Parity: the reference keeps this as an experiment outside the engine (bench/k3_partition/cp_merge.py:8-52: all-reduce(MAX)
of the log-sum-exps and an all-reduce(SUM) of the rescaled packed outputs; paged_cp.py:21-59 for the page split).
"""
from __future__ import annotations

import ctypes as _c
from typing import List, Tuple

import torch

from ..ops import sm100 as _k
from ..ops import sm100_attn as _attn
from .fused_tp import FusedTP


def shard_pages(block_table: List[int], context_len: int, block_size: int, cp: int, rank: int) -> Tuple[List[int], int]:
    """Pages of one sequence that `rank` holds under round-robin dealing, and how many of the sequence's tokens they contain."""
    n_pages = (context_len + block_size - 1) // block_size
    mine = [block_table[p] for p in range(rank, n_pages, cp)]
    tokens = 0
    for p in range(rank, n_pages, cp):
        tokens += min(block_size, context_len - p * block_size)
    return mine, tokens


class DecodeCP:
    def __init__(self, group, heads: int, kv_lora_rank: int = 512, max_tokens: int = 128, local_splits: int = 2,
                 spin_limit: int = 1 << 22):
        import torch.distributed as dist
        assert local_splits >= 2, "the attention kernel leaves partial results only when it slices the keys"
        self.world = dist.get_world_size(group)
        self.H, self.R, self.S, self.max_tokens = heads, kv_lora_rank, local_splits, max_tokens
        # fp32 payloads travel as pairs of bf16 columns through the bf16-typed gather buffers
        self.g_part = FusedTP(group, "cp_part", 2 * kv_lora_rank, self.world * local_splits * max_tokens * heads, spin_limit)
        self.g_lse = FusedTP(group, "cp_lse", 2 * heads, self.world * local_splits * max_tokens, spin_limit)

    def attention(self, q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, cu_seqlens_q: torch.Tensor,
                  context_lens: torch.Tensor, scale: float) -> torch.Tensor:
        """q [T, H, 576] (the same on every rank), cache / block_tables / context_lens describe this rank's pages.
        Returns [T, H, R] bf16, the attention over the union of all ranks' pages."""
        T, H, _ = q.shape
        S, R = self.S, self.R
        assert H == self.H and T <= self.max_tokens
        part, lse = _attn.mla_partials(q, cache, block_tables, cu_seqlens_q, context_lens, scale, R, S)
        allp = self.g_part.all_gather(part.view(torch.bfloat16).view(S * T * H, 2 * R))
        alll = self.g_lse.all_gather(lse.view(torch.bfloat16).view(S * T, 2 * H))
        out = torch.empty(T, H, R, dtype=torch.bfloat16, device=q.device)
        _k._ck(_k.lib().ne_attn_merge(_k._p(allp), _k._p(alll), _k._p(out), _c.c_int(self.world * S), _c.c_longlong(T * H), _c.c_int(R), _c.c_int(R),
                                      _k._st()), "ne_attn_merge")
        return out
