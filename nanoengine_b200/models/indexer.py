"""DSA / NSA lightning indexer (DeepSeek-V3.2): picks the top-k keys every query token attends to.

  q = wq_b(q_lora)            -> [T, Hi, D]      k = LayerNorm(wk(hidden)) -> [T, D]     head weights = weights_proj(hidden) -> [T, Hi]
  RoPE on the first rope_dim values of q and k, Hadamard transform of both, fp8 quantisation with one power-of-two scale per
  row; keys are stored in the indexer cache (per 64-token page: 64 x D e4m3 keys, then 64 fp32 scales) sharing the main
  page table.  score(i, j) = sum_h w[i,h] * relu(q[i,h] . k[j]) with the ReLU before the head sum; causal; top-k;
  logical -> physical slot through the block table; -1 marks unused entries.
When a sequence's context is not longer than top-k the selection is the identity, and the layer runs the dense kernel.

Parity: reference layers/backends/dsa/indexer/lightning.py:116-162 (scoring), :408-535 (IndexerCache), :538-1492
(Indexer: projections, store, prefill and decode top-k); kernels K3/K5/K9/T11/X5 of the survey are restated here as
operators (`ops.hadamard`, `ops.quant_fp8_per_token_pow2`, `ops.indexer_logits`, `ops.indexer_topk`).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .layers import QLinear

FP8 = torch.float8_e4m3fn


class LightningIndexer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.Hi, self.D, self.topk = cfg.index_n_heads, cfg.index_head_dim, cfg.index_topk
        self.rope_dim = cfg.qk_rope_head_dim
        q_in = cfg.q_lora_rank or cfg.hidden_size
        self.wq_b = QLinear(q_in, self.Hi * self.D, dtype, device, None)
        self.wk = QLinear(cfg.hidden_size, self.D, dtype, device, None)
        self.k_norm_weight = nn.Parameter(torch.ones(self.D, dtype=dtype, device=device), requires_grad=False)
        self.k_norm_bias = nn.Parameter(torch.zeros(self.D, dtype=dtype, device=device), requires_grad=False)
        self.weights_proj = QLinear(cfg.hidden_size, self.Hi, dtype, device, None)
        self.softmax_scale = self.D ** -0.5

    def load(self, leaf: str, w: torch.Tensor, s):
        if w.dtype == FP8:
            w = ref.dequant_fp8_block(w, s)
        if leaf == "wq_b":
            self.wq_b.set_weight(w)
        elif leaf == "wk":
            self.wk.set_weight(w)
        elif leaf == "weights_proj":
            self.weights_proj.set_weight(w)
        elif leaf == "k_norm":
            self.k_norm_weight.copy_(w.to(self.k_norm_weight.dtype))
        elif leaf == "k_norm.bias":
            self.k_norm_bias.copy_(w.to(self.k_norm_bias.dtype))

    # ---- cache -------------------------------------------------------------------------------
    def _store(self, cache: torch.Tensor, slots: torch.Tensor, k8: torch.Tensor, ks: torch.Tensor):
        """cache [blocks, bs*(D+4)] uint8.  Key row `off` of a page sits at off*D, its scale at bs*D + off*4."""
        bs = cache.shape[1] // (self.D + 4)
        blk, off = (slots // bs).long(), (slots % bs).long()
        flat = cache.view(-1)
        page = cache.shape[1]
        kidx = (blk * page + off * self.D).unsqueeze(1) + torch.arange(self.D, device=cache.device)
        flat[kidx.reshape(-1)] = k8.view(torch.uint8).reshape(-1)
        sidx = (blk * page + bs * self.D + off * 4).unsqueeze(1) + torch.arange(4, device=cache.device)
        flat[sidx.reshape(-1)] = ks.float().contiguous().view(torch.uint8).reshape(-1)

    def _gather(self, cache: torch.Tensor, block_table: torch.Tensor, n: int):
        bs = cache.shape[1] // (self.D + 4)
        nb = (n + bs - 1) // bs
        pages = cache[block_table[:nb].long()]                                      # [nb, bs*(D+4)]
        keys = pages[:, : bs * self.D].reshape(nb * bs, self.D).view(FP8)[:n]
        scales = pages[:, bs * self.D:].contiguous().view(torch.float32).reshape(nb * bs)[:n]
        return keys, scales

    # ---- forward -----------------------------------------------------------------------------
    def forward(self, hidden: torch.Tensor, q_in: torch.Tensor, positions: torch.Tensor, ctx: ForwardContext, rope_cache: torch.Tensor
                ) -> Optional[torch.Tensor]:
        T = hidden.shape[0]
        q = self.wq_b(q_in).view(T, self.Hi, self.D)
        k = ops.layernorm(self.wk(hidden), self.k_norm_weight, self.k_norm_bias, 1e-6)
        rd = self.rope_dim
        q = torch.cat([ref.apply_rope(q[..., :rd], positions, rope_cache, False), q[..., rd:]], -1)
        k = torch.cat([ref.apply_rope(k[..., :rd], positions, rope_cache, False), k[..., rd:]], -1)
        q, k = ops.hadamard(q), ops.hadamard(k)
        k8, ks = ops.quant_fp8_per_token_pow2(k)
        cache = ctx.indexer_caches[self.layer_idx]
        self._store(cache, ctx.slot_mapping, k8, ks)
        if max(ctx.context_lens_host or [ctx.max_seqlen_k]) <= self.topk:
            return None                                   # every key is selected anyway: dense attention
        q8, qs = ops.quant_fp8_per_token_pow2(q.reshape(T * self.Hi, self.D))
        q8, qs = q8.view(T, self.Hi, self.D), qs.view(T, self.Hi)
        w = self.weights_proj(hidden).float() * (self.Hi ** -0.5) * self.softmax_scale
        out = torch.full((T, self.topk), -1, dtype=torch.int32, device=hidden.device)
        cu, cl = ctx.cu_seqlens_q_host, ctx.context_lens_host
        bs = cache.shape[1] // (self.D + 4)
        for i in range(ctx.num_seqs):
            lo, hi = cu[i], cu[i + 1]
            if hi == lo:
                continue
            n = cl[i]
            keys, kscale = self._gather(cache, ctx.block_tables[i], n)
            logits = ops.indexer_logits(q8[lo:hi], qs[lo:hi], w[lo:hi], keys, kscale)          # [q, n]
            valid = torch.arange(n - (hi - lo) + 1, n + 1, device=hidden.device)               # causal: keys visible to each row
            idx = ops.indexer_topk(logits, valid, self.topk)
            out[lo:hi] = ops.logical_to_physical(idx, ctx.block_tables[i:i + 1].expand(hi - lo, -1), bs)
        return out
