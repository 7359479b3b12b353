"""DSA / NSA lightning indexer (DeepSeek-V3.2): picks the top-k keys every query token attends to.

  q = wq_b(q_lora)            -> [T, Hi, D]      k = LayerNorm(wk(hidden)) -> [T, D]     head weights = weights_proj(hidden) -> [T, Hi]
  RoPE on the first rope_dim values of q and k, Hadamard transform of both, fp8 quantisation with one power-of-two scale per
  row; keys are stored in the indexer cache (per 64-token page: 64 x D e4m3 keys, then 64 fp32 scales) sharing the main
  page table.  score(i, j) = sum_h w[i,h] * relu(q[i,h] . k[j]) with the ReLU before the head sum; causal; top-k;
  logical -> physical slot through the block table; -1 marks unused entries.
When a sequence's context is not longer than top-k the selection is the identity, and the layer runs the dense kernel.

Parity: reference layers/backends/dsa/indexer/lightning.py:116-162 (scoring), :408-535 (IndexerCache), :538-1492
(Indexer: projections, store, prefill and decode top-k).  The work is three operators: `ops.indexer_k_store` (key path
into the cache), `ops.indexer_q_prep` (query path) and `ops.indexer_select` (fp8 logits + top-k + page translation).
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

    # ---- forward -----------------------------------------------------------------------------
    def forward(self, hidden: torch.Tensor, q_in: torch.Tensor, positions: torch.Tensor, ctx: ForwardContext, rope_cache: torch.Tensor,
                logical: bool = False) -> Optional[torch.Tensor]:
        """Physical cache rows of the selected keys of every token ([T, topk], -1 padded), or None when every context fits the
        list (dense attention).  `logical`: always select, and list key positions (the hot / cold tier maps them itself)."""
        T = hidden.shape[0]
        rd = self.rope_dim
        q = self.wq_b(q_in).view(T, self.Hi, self.D)
        cache = ctx.indexer_caches[self.layer_idx]
        ops.indexer_k_store(self.wk(hidden), self.k_norm_weight, self.k_norm_bias, 1e-6, positions, rope_cache, rd, cache, ctx.slot_mapping)
        if not logical and max(ctx.context_lens_host or [ctx.max_seqlen_k]) <= self.topk:
            return None                                   # every key is selected anyway: dense attention
        q8, qs = ops.indexer_q_prep(q, positions, rope_cache, rd)
        w = self.weights_proj(hidden).float() * (self.Hi ** -0.5) * self.softmax_scale
        cu = ctx.cu_seqlens_q_host if ctx.cu_seqlens_q_host is not None else ctx.cu_seqlens_q
        cl = ctx.context_lens_host if ctx.context_lens_host is not None else ctx.context_lens
        if hidden.is_cuda:
            cu, cl = ctx.cu_seqlens_q, ctx.context_lens       # device tables: no host round trip inside a captured graph
        return ops.indexer_select(q8, qs, w, cache, ctx.block_tables, cu, cl, self.topk, logical)
