"""Qwen3 dense and Qwen3-MoE: GQA attention with per-head q/k RMSNorm and RoPE (theta 1e6), softmax top-k routed experts.

Parallel layout (config "TP attention + EP experts"): the residual stream stays token-sliced between blocks - rank r of
the attention-TP group holds rows [r*T/tp, (r+1)*T/tp).  An attention block all-gathers its normalised slice in front
of the head-sharded qkv GEMM and reduce-scatters the row-parallel o_proj output back to slices (the two TP boundaries
that are fused with their GEMMs on GPUs); the MoE block runs expert-parallel directly on each rank's slice, so no
extra transition pass exists between the two.

Parity: reference runtime/models/qwen3_moe/qwen3_moe.py - attention :58-146, sparse block :225-324 (softmax top-k
:283-297), layer :327-436 (TP<->EP transitions :388-397); qwen3_moe_loader.py:27-130; models/qwen3/.
"""
from __future__ import annotations

import re
from typing import Iterable, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..parallel.dist import get_dist_context
from ..parallel.ep import ep_moe_forward
from ..parallel.tp import tp_all_gather, tp_all_gather_linear, tp_linear_reduce_scatter, tp_reduce_scatter
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .layers import ParallelLMHead, QLinear, RMSNorm, RoutedExperts, SwiGLUMLP, TPSwiGLUMLP, VocabParallelEmbedding


VOCAB_PARALLEL = True     # split embed_tokens / lm_head by vocabulary rows whenever attention is tensor-parallel


class Qwen3Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        d = get_dist_context()
        self.cfg, self.layer_idx = cfg, layer_idx
        tp, r = d.attn_tp_size, d.attn_tp_rank
        self.tp, self.tp_rank = tp, r
        self.hd = cfg.head_dim
        assert cfg.num_attention_heads % tp == 0
        self.hq = cfg.num_attention_heads // tp
        self.hkv = max(1, cfg.num_key_value_heads // tp)
        # kv head owned by this rank when there are fewer kv heads than TP ranks
        self.kv_first = (r * cfg.num_key_value_heads) // tp
        self.qkv_proj = QLinear(cfg.hidden_size, (self.hq + 2 * self.hkv) * self.hd, dtype, device, cfg.quant, bias=cfg.attention_bias)
        self.o_proj = QLinear(self.hq * self.hd, cfg.hidden_size, dtype, device, cfg.quant)
        self.q_norm = RMSNorm(self.hd, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.k_norm = RMSNorm(self.hd, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.scale = self.hd ** -0.5

    def forward(self, x_slice, positions, ctx: ForwardContext, rope_cache, total_rows: int):
        qkv = tp_all_gather_linear(ops.dense(x_slice), total_rows, self.qkv_proj) if self.tp > 1 else self.qkv_proj(x_slice)
        T = qkv.shape[0]
        kc, vc = ctx.kv_caches[self.layer_idx]
        # head split, q / k RMSNorm, rotary embedding and the paged K / V store in one pass over the projection output
        q = ops.gqa_qkv_prepare(qkv, self.hq, self.hkv, self.hd, self.q_norm.weight if self.q_norm is not None else None,
                                self.k_norm.weight if self.k_norm is not None else None, self.cfg.rms_norm_eps, False, positions, rope_cache,
                                kc, vc, ctx.slot_mapping)
        o = ops.gqa_attention_paged(q, kc, vc, ctx.block_tables, ctx.cu_seqlens_q, ctx.context_lens, self.scale)
        o = o.reshape(T, self.hq * self.hd)
        return tp_linear_reduce_scatter(o, self.o_proj) if self.tp > 1 else self.o_proj(o)


class Qwen3MoE(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, layer_idx: Optional[int] = None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.gate_weight = nn.Parameter(torch.empty(cfg.n_routed_experts, cfg.hidden_size, dtype=torch.float32, device=device), requires_grad=False)
        self.experts = RoutedExperts(cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size, dtype, device, cfg.quant, layer_idx)

    def forward(self, x, ctx, total_rows: Optional[int] = None):
        c = self.cfg
        x = ops.dense(x)
        ffn_tp = self.experts.ffn_tp > 1
        if ffn_tp:
            # experts split by intermediate columns over the TP group: every rank works on all tokens with its share of each
            # expert and the partial outputs are reduce-scattered back to the token slices
            from ..parallel.tp import tp_all_gather, tp_reduce_scatter
            x = tp_all_gather(x, total_rows)
        logits = ops.router_logits(x, self.gate_weight)
        from ..parallel.ep import routing_options
        idx, w = ops.moe_route(logits, None, c.num_experts_per_tok, 1, 1, c.norm_topk_prob, 1.0, "softmax", **routing_options(self.layer_idx, x.device))
        out = ep_moe_forward(self.experts, x, idx, w, ctx)
        return tp_reduce_scatter(out) if ffn_tp else out


class Qwen3DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        fp8 = cfg.quant == "fp8"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8)
        self.self_attn = Qwen3Attention(cfg, layer_idx, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8)
        self.is_moe = cfg.is_moe_layer(layer_idx)
        self.ffn_tp = get_dist_context().ffn_tp_size > 1
        if self.is_moe:
            self.mlp = Qwen3MoE(cfg, dtype, device, layer_idx)
        elif self.ffn_tp:
            self.mlp = TPSwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quant)
        else:
            self.mlp = SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quant)

    def forward(self, h, residual, positions, ctx, rope_cache, total_rows):
        x, residual = self.input_layernorm(h, residual) if residual is not None else (self.input_layernorm(h), h)
        a = self.self_attn(x, positions, ctx, rope_cache, total_rows)
        x, residual = self.post_attention_layernorm(a, residual)
        if self.is_moe:
            m = self.mlp(x, ctx, total_rows)
        else:
            m = self.mlp(x, total_rows) if self.ffn_tp else self.mlp(x)
        return m, residual


class Qwen3MoeForCausalLM(nn.Module):
    """Serves both Qwen3MoeForCausalLM and dense Qwen3ForCausalLM (n_routed_experts = 0)."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", layer_range=None):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        d = get_dist_context()
        self.tp, self.tp_rank = d.attn_tp_size, d.attn_tp_rank
        # with tensor-parallel attention the embedding table and the output projection are split by vocabulary rows
        self.vocab_parallel = self.tp > 1 and VOCAB_PARALLEL
        if self.vocab_parallel:
            self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
            self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device)
        else:
            self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
            self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        self.layers = nn.ModuleList([Qwen3DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        rc = ref.rope_cos_sin_cache(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_scaling)
        self.register_buffer("rope_cache", rc.to(device), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def num_cache_layers(self) -> int:
        return self.cfg.num_hidden_layers

    def forward(self, input_ids, positions, ctx: ForwardContext, inputs_embeds=None):
        if self.vocab_parallel and inputs_embeds is None:
            T = input_ids.shape[0]
            h = self.embed_tokens.forward_scatter(input_ids)          # partial rows summed straight into the token slices
        else:
            h = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
            T = h.shape[0]
        if self.tp > 1 and not (self.vocab_parallel and inputs_embeds is None):
            per = -(-T // self.tp)
            pad = per * self.tp - T
            if pad:
                h = torch.cat([h, h.new_zeros(pad, h.shape[1])], 0)
            h = h[self.tp_rank * per: (self.tp_rank + 1) * per].contiguous()
        residual = None
        for layer in self.layers:
            h, residual = layer(h, residual, positions, ctx, self.rope_cache, T)
        h, _ = self.norm(h, residual)
        return tp_all_gather(h, T) if self.tp > 1 else h

    def compute_logits(self, hidden):
        if self.vocab_parallel:
            return self.lm_head(hidden)
        return ops.lm_head(hidden, self.lm_head.weight)

    # ---- weights ---------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        cfg = self.cfg
        hd = cfg.head_dim
        n = 0
        pending = {}
        scales = {}
        fp8 = torch.float8_e4m3fn

        def deq(w, s):
            return ref.dequant_fp8_block(w, s) if w.dtype == fp8 else w.float()

        def place(base, w, s):
            nonlocal n
            n += 1
            if base == "model.embed_tokens":
                (self.embed_tokens.load_full(w) if self.vocab_parallel else self.embed_tokens.weight.copy_(w.to(self.dtype))); return
            if base == "lm_head":
                (self.lm_head.load_full(w) if self.vocab_parallel else self.lm_head.weight.copy_(w.to(self.dtype))); return
            if base == "model.norm":
                self.norm.weight.copy_(w.to(self.dtype)); return
            m = re.match(r"model\.layers\.(\d+)\.(.*)", base)
            if not m:
                return
            L = self.layers[int(m.group(1))]
            rest = m.group(2)
            if rest in ("input_layernorm", "post_attention_layernorm"):
                getattr(L, rest).weight.copy_(w.to(self.dtype)); return
            A = L.self_attn
            if rest in ("self_attn.q_norm", "self_attn.k_norm"):
                mod = getattr(A, rest.split(".")[1])
                if mod is not None:
                    mod.weight.copy_(w.to(self.dtype))
                return
            if rest in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                key = f"{m.group(1)}.qkv"
                g = pending.setdefault(key, {})
                wf = deq(w, s)
                leaf = rest.split(".")[1]
                if leaf == "q_proj":
                    g[leaf] = wf[A.tp_rank * A.hq * hd: (A.tp_rank + 1) * A.hq * hd]
                else:
                    g[leaf] = wf[A.kv_first * hd: (A.kv_first + A.hkv) * hd]
                if len(g) == 3:
                    A.qkv_proj.set_weight(torch.cat([g["q_proj"], g["k_proj"], g["v_proj"]], 0)); pending.pop(key)
                return
            if rest == "self_attn.o_proj":
                wf = deq(w, s)
                A.o_proj.set_weight(wf[:, A.tp_rank * A.hq * hd: (A.tp_rank + 1) * A.hq * hd].contiguous()); return
            if rest == "mlp.gate":
                L.mlp.gate_weight.copy_(w.float()); return
            e = re.match(r"mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)$", rest)
            if e:
                eid, which = int(e.group(1)), e.group(2)[:-5]
                ex = L.mlp.experts
                if not ex.load_expert(eid, which, w, s):
                    n -= 1
                return
            if rest in ("mlp.gate_proj", "mlp.up_proj"):
                key = f"{m.group(1)}.gate_up"
                g = pending.setdefault(key, {})
                wf = deq(w, s)
                if L.ffn_tp:
                    lo, hi = L.mlp.shard_rows()
                    wf = wf[lo:hi]
                g[rest.split(".")[1]] = wf
                if len(g) == 2:
                    L.mlp.gate_up_proj.set_weight(torch.cat([g["gate_proj"], g["up_proj"]], 0)); pending.pop(key)
                return
            if rest == "mlp.down_proj":
                if L.ffn_tp:
                    lo, hi = L.mlp.shard_rows()
                    L.mlp.down_proj.set_weight(deq(w, s)[:, lo:hi].contiguous()); return
                L.mlp.down_proj.set_weight(w, s); return

        wbuf = {}
        with torch.no_grad():
            for name, t in weights:
                if name.endswith(".weight_scale_inv"):
                    base = name[: -len(".weight_scale_inv")]
                    if base in wbuf:
                        place(base, wbuf.pop(base), t)
                    else:
                        scales[base] = t
                    continue
                if not name.endswith(".weight"):
                    continue
                base = name[: -len(".weight")]
                if t.dtype == fp8:
                    if base in scales:
                        place(base, t, scales.pop(base))
                    else:
                        wbuf[base] = t
                else:
                    place(base, t, None)
        if pending or wbuf:
            raise ValueError(f"incomplete checkpoint: {list(pending)[:3]} {list(wbuf)[:3]}")
        return n
