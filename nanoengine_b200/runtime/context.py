"""Per-step attention metadata handed to every layer of a forward pass.

Parity: reference runtime/context/batch.py:11-43 (BatchContext fields: cu_seqlens_q/k,
slot_mapping, context_lens, block_tables, sampling indices).  Here it is an explicit argument of
``model.forward`` instead of a process-global singleton, which keeps CUDA-graph capture and
multi-engine processes (prefill + decode engines in one test) free of hidden state.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch


@dataclass
class ForwardContext:
    is_prefill: bool
    num_seqs: int
    num_tokens: int
    cu_seqlens_q: torch.Tensor            # int32 [B+1]
    context_lens: torch.Tensor            # int32 [B]  context length of each sequence after this step
    slot_mapping: torch.Tensor            # int64 [T]  cache row of every new token
    block_tables: torch.Tensor            # int32 [B, max_blocks]
    max_seqlen_q: int = 1
    max_seqlen_k: int = 1
    last_token_indices: Optional[torch.Tensor] = None   # int32 [B] row of each sequence's last new token
    q_len_uniform: int = 0                # > 0 when every sequence contributes exactly this many rows (decode / verify)
    is_dummy: bool = False
    kv_caches: Optional[List[Any]] = None  # per-layer cache tensors (MLA: [blocks, bs, D]; GQA: (k, v))
    indexer_caches: Optional[List[Any]] = None
    # recurrent-state layers: slot of each sequence in the state pools, whether the sequence starts in this step, the pools
    state_slots: Optional[torch.Tensor] = None      # int32 [B]
    seq_fresh: Optional[torch.Tensor] = None        # int32 [B], 1 = no state carried in (first chunk of the prompt)
    conv_states: Optional[List[Any]] = None         # per linear layer [slots, K-1, conv_dim]
    rec_states: Optional[List[Any]] = None          # per linear layer [slots, Hv, Dv, Dk] fp32
    # DeepSeek-V4 compressors: per layer (None for a window-only layer) the pooled-row pages and the two carry pools
    comp_caches: Optional[List[Any]] = None         # [blocks, entries_per_page, head_dim]
    comp_kv_states: Optional[List[Any]] = None      # [slots, c * ratio, c * head_dim] fp32
    comp_score_states: Optional[List[Any]] = None
    # hot / cold tier of the sparse-attention cache: the tier object and the hot-buffer slot of each sequence
    hisparse: Optional[Any] = None
    hs_slots: Optional[torch.Tensor] = None         # int32 [B]
    extras: Dict[str, Any] = field(default_factory=dict)   # per-forward scratch shared by layers (e.g. DSA top-k reuse)
    # host copies for the CPU reference path and for planning
    cu_seqlens_q_host: Optional[List[int]] = None
    context_lens_host: Optional[List[int]] = None
