"""CUDA bodies of attention and sampling."""
from __future__ import annotations

import torch

from . import reference as ref


def mla_attention_paged(q, cache, block_tables, cu_seqlens_q, context_lens, scale, kv_lora_rank, sparse_indices=None):
    return ref.mla_attention_paged(q, cache, block_tables, cu_seqlens_q, context_lens, scale, kv_lora_rank, sparse_indices)


def gqa_attention_paged(q, k_cache, v_cache, block_tables, cu_seqlens_q, context_lens, scale):
    return ref.gqa_attention_paged(q, k_cache, v_cache, block_tables, cu_seqlens_q, context_lens, scale)


def sample(logits, temperatures, generator=None, return_logprobs=False):
    return ref.sample(logits, temperatures, generator, return_logprobs)
