"""DeepSeek-V2 / V3 / V3.2 family: MLA attention over a paged latent KV cache, sigmoid-routed MoE with a
shared expert, optional DSA lightning indexer, and the MTP (next-n) head.

Parity: reference runtime/models/deepseek_v2/deepseek_v2.py - MoE :404-594, dense MLP :597-655, decoder
layer :658-740, absorbed kc/vc BMMs :926-941, attention :944-2043 (YaRN softmax scale :1075-1082, absorbed
decode :1825-2043); deepseek_v2_mtp.py:56-189; loader deepseek_v2_loader.py:36-270 (kv_b_proj -> kc/vc).

B200-first differences: q_a_proj and kv_a_proj_with_mqa are one GEMM (their input is shared), the absorbed
form is used for prefill and decode alike so a single paged-latent attention kernel serves both (a
chunked-prefix or prefix-cache hit needs no gather/expand/merge pass), and the KV row layout is the raw
576-value row the Blackwell decode kernel reads.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..parallel.dist import get_dist_context
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .layers import QLinear, RMSNorm, RoutedExperts, SwiGLUMLP


class MLAAttention(nn.Module):
    """`cache_idx`: which page family entry the layer uses (its rank among the full-attention layers in the hybrid families;
    the layer index otherwise).  With `cfg.mla_output_gate` the heads' output is multiplied by sigmoid(g_proj(x)) before
    o_proj (reference models/kimi_k3/kimi_k3.py:73-100)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device, cache_idx: Optional[int] = None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.cache_idx = layer_idx if cache_idx is None else cache_idx
        H, R, rope, nope, v = cfg.num_attention_heads, cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.qk_nope_head_dim, cfg.v_head_dim
        self.H, self.R, self.rope, self.nope, self.v = H, R, rope, nope, v
        self.q_lora = cfg.q_lora_rank
        q = cfg.quant
        if self.q_lora:
            # fused [q_a_proj ; kv_a_proj_with_mqa]
            self.qkv_a_proj = QLinear(cfg.hidden_size, self.q_lora + R + rope, dtype, device, q)
            self.q_a_layernorm = RMSNorm(self.q_lora, cfg.rms_norm_eps, dtype, device, quant_out=(q == "fp8"))
            self.q_b_proj = QLinear(self.q_lora, H * (nope + rope), dtype, device, q)
        else:
            self.q_proj = QLinear(cfg.hidden_size, H * (nope + rope), dtype, device, q)
            self.kv_a_proj_with_mqa = QLinear(cfg.hidden_size, R + rope, dtype, device, q)
        self.kv_a_layernorm = RMSNorm(R, cfg.rms_norm_eps, dtype, device)
        # absorbed halves of kv_b_proj
        self.kc = nn.Parameter(torch.empty(H, nope, R, dtype=dtype, device=device), requires_grad=False)   # W_UK
        self.vc = nn.Parameter(torch.empty(H, R, v, dtype=dtype, device=device), requires_grad=False)      # W_UV^T
        # K-major bf16 copies of kc / vc for the per-head tensor-core GEMMs: built by `refresh_absorbed` whenever the weights are set
        self.kc_t: Optional[torch.Tensor] = None
        self.vc_t: Optional[torch.Tensor] = None
        self.o_proj = QLinear(H * v, cfg.hidden_size, dtype, device, q)
        self.scale = (nope + rope) ** -0.5
        sc = cfg.rope_scaling
        if sc and sc.get("type", sc.get("rope_type")) == "yarn" and sc.get("mscale_all_dim"):
            m = ref.yarn_mscale(float(sc["factor"]), float(sc["mscale_all_dim"]))
            self.scale *= m * m
        self.indexer = None
        if cfg.has_indexer:
            from .indexer import LightningIndexer
            self.indexer = LightningIndexer(cfg, self.cache_idx, dtype, device)
        self.g_proj = QLinear(cfg.hidden_size, H * v, dtype, device, None) if cfg.mla_output_gate else None

    def set_kv_b(self, w: torch.Tensor, scale_inv: Optional[torch.Tensor] = None):
        """kv_b_proj.weight [H*(nope+v), R] -> kc [H, nope, R], vc [H, R, v]."""
        if w.dtype == torch.float8_e4m3fn:
            w = ref.dequant_fp8_block(w, scale_inv)
        w = w.view(self.H, self.nope + self.v, self.R)
        self.kc.copy_(w[:, : self.nope].to(self.kc.dtype))
        self.vc.copy_(w[:, self.nope:].transpose(1, 2).to(self.vc.dtype))
        self.refresh_absorbed()

    def refresh_absorbed(self):
        """Rebuild the operand copies derived from kc / vc.  Called by `set_kv_b`; call it again after writing kc / vc directly.
        Parity: reference models/deepseek_v2/deepseek_v2_loader.py:36-121 transforms kv_b_proj once at load."""
        if self.kc.is_cuda:
            if self.kc_t is not None and self.kc_t.device == self.kc.device:
                # same storage: CUDA graphs that captured these addresses stay valid
                self.kc_t.copy_(ops.kmajor(self.kc))
                self.vc_t.copy_(ops.kmajor(self.vc))
            else:
                self.kc_t, self.vc_t = ops.kmajor(self.kc), ops.kmajor(self.vc)
        else:
            self.kc_t = self.vc_t = None

    def forward(self, x: torch.Tensor, positions: torch.Tensor, ctx: ForwardContext, rope_cache: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        H, R, rope, nope = self.H, self.R, self.rope, self.nope
        if self.q_lora:
            a = self.qkv_a_proj(x)
            q_c = self.q_a_layernorm(a[:, : self.q_lora])
            kv_a = a[:, self.q_lora:]
            q = self.q_b_proj(q_c)
        else:
            q_c = None
            q = self.q_proj(x)
            kv_a = self.kv_a_proj_with_mqa(x)
        q = q.view(T, H, nope + rope)
        if ctx.hisparse is not None and not ctx.is_prefill and self.indexer is not None:
            return self._forward_hot_cold(x, q, q_c, kv_a, positions, ctx, rope_cache)
        cache = ctx.kv_caches[self.cache_idx]
        ops.mla_kv_prepare(kv_a, self.kv_a_layernorm.weight, self.kv_a_layernorm.eps, positions, rope_cache, cache, ctx.slot_mapping, R)
        sparse = None
        if self.indexer is not None:
            xd = ops.dense(x)
            sparse = self.indexer(xd, ops.dense(q_c) if q_c is not None else xd, positions, ctx, rope_cache)
        if (NONABSORBED_PREFILL and ctx.is_prefill and sparse is None and x.is_cuda and ctx.extras.get("no_prefix") and nope == 128
                and rope == 64 and self.v == 128 and x.dtype == torch.bfloat16):
            return self._prefill_nonabsorbed(x, q, kv_a, positions, ctx, rope_cache)
        q_full = ops.mla_query(q, self.kc, positions, rope_cache, nope, cache, sparse is None, kc_t=self.kc_t)   # [T, H, R + rope]
        o_lat = ops.mla_attention_paged(q_full, cache, ctx.block_tables, ctx.cu_seqlens_q, ctx.context_lens, self.scale, R,
                                        sparse_indices=sparse)
        o = ops.bmm_absorb(o_lat, self.vc, wt=self.vc_t).reshape(T, H * self.v)           # [T, H * v]
        if self.g_proj is not None:
            o = ops.sigmoid_mul(o, self.g_proj(ops.dense(x)))
        return self.o_proj(o)


    def _prefill_nonabsorbed(self, x, q, kv_a, positions, ctx: ForwardContext, rope_cache):
        """Prompts without a cached prefix: keys and values are expanded from the latent rows of the same tokens (two GEMMs against
        W_UK / W_UV) and attended in their own 192 / 128-wide geometry, 128 query tokens per tile - about a third of the
        multiply-adds of the absorbed 576 / 512-wide form and no re-read of the pages per query token.  The latent cache was
        written just before (decode and later chunks read it).
        Parity: reference models/deepseek_v2/deepseek_v2.py:1792-1816 (non-absorbed ragged prefill)."""
        T, H, R, nope = x.shape[0], self.H, self.R, self.nope
        ckv = ops.rmsnorm(kv_a[:, :R], self.kv_a_layernorm.weight, self.kv_a_layernorm.eps)
        ckv = ops.dense(ckv)
        k_pe = ops.apply_rope(kv_a[:, R:].contiguous().view(T, 1, self.rope), positions, rope_cache, True).view(T, self.rope)
        ops.apply_rope(q[..., nope:], positions, rope_cache, True, q[..., nope:])           # in place on the strided view
        k_nope = ops.linear(ckv, self.kc.view(H * nope, R)).view(T, H, nope)
        v = ops.linear(ckv, self.vc_t.view(H * self.v, R)).view(T, H, self.v)
        o = ops.mla_prefill_ragged(q, k_nope, k_pe, v, ctx.cu_seqlens_q, self.scale).reshape(T, H * self.v)
        if self.g_proj is not None:
            o = ops.sigmoid_mul(o, self.g_proj(ops.dense(x)))
        return self.o_proj(o)

    def _forward_hot_cold(self, x, q, q_c, kv_a, positions, ctx: ForwardContext, rope_cache):
        """Decode step under the hot / cold tier: the indexer lists key positions, the tier makes them resident in the
        sequence's hot buffer (the new token's row included), the key path writes the new row there and copies it back to
        the cold pages, and the sparse attention reads the hot buffer.
        Parity: reference docs/hisparse-design.md "Model forward", runtime/context/cache/hisparse.py:294-316."""
        T, H, R, nope = x.shape[0], self.H, self.R, self.nope
        assert ctx.q_len_uniform == 1, "the hot / cold tier serves plain decode steps (one new token per sequence)"
        tier = ctx.hisparse
        L = tier.layer(self.cache_idx)
        xd = ops.dense(x)
        sel = self.indexer(xd, ops.dense(q_c) if q_c is not None else xd, positions, ctx, rope_cache, logical=True)
        hot_ids, new_slot = ops.hisparse_stage(L, sel, ctx.hs_slots, ctx.context_lens, ctx.block_tables)
        dt = ctx.kv_caches[self.cache_idx].dtype
        hot = tier.hot_pages(self.cache_idx, dt)
        ops.mla_kv_prepare(kv_a, self.kv_a_layernorm.weight, self.kv_a_layernorm.eps, positions, rope_cache, hot, new_slot, R)
        ops.hisparse_writeback(L["hot"], L["cold"], new_slot, ctx.slot_mapping)
        q_full = ops.mla_query(q, self.kc, positions, rope_cache, nope, hot, False, kc_t=self.kc_t)
        o_lat = ops.mla_attention_paged(q_full, hot, ctx.block_tables, ctx.cu_seqlens_q, ctx.context_lens, self.scale, R, sparse_indices=hot_ids)
        o = ops.bmm_absorb(o_lat, self.vc, wt=self.vc_t).reshape(T, H * self.v)
        if self.g_proj is not None:
            o = ops.sigmoid_mul(o, self.g_proj(xd))
        return self.o_proj(o)


NONABSORBED_PREFILL = True        # prompts without a cached prefix attend in the 192 / 128-wide geometry on the GPU
OVERLAP_SHARED_EXPERTS = True


def _side_stream(device):
    from ..runtime.stream_pool import get_cuda_stream
    return get_cuda_stream("shared_expert", device)


class MoEGate(nn.Module):
    def __init__(self, cfg: ModelConfig, device, layer_idx: Optional[int] = None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.weight = nn.Parameter(torch.empty(cfg.n_routed_experts, cfg.hidden_size, dtype=torch.float32, device=device), requires_grad=False)
        self.e_score_correction_bias = None
        if cfg.topk_method == "noaux_tc" and cfg.scoring_func == "sigmoid":
            self.e_score_correction_bias = nn.Parameter(torch.zeros(cfg.n_routed_experts, dtype=torch.float32, device=device), requires_grad=False)

    def forward(self, x):
        c = self.cfg
        from ..parallel.ep import routing_options
        logits = ops.router_logits(x, self.weight)
        return ops.moe_route(logits, self.e_score_correction_bias, c.num_experts_per_tok, c.n_group, c.topk_group,
                             c.norm_topk_prob, c.routed_scaling_factor, c.scoring_func, **routing_options(self.layer_idx, x.device))


class DeepseekMoE(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, layer_idx: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.gate = MoEGate(cfg, device, layer_idx)
        self.experts = RoutedExperts(cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size, dtype, device, cfg.quant, layer_idx,
                                     act=cfg.glu_act)
        self.shared_experts = None
        if cfg.n_shared_experts > 0:
            self.shared_experts = SwiGLUMLP(cfg.hidden_size, cfg.moe_intermediate_size * cfg.n_shared_experts, dtype, device, cfg.quant,
                                            act=cfg.glu_act)

    def forward(self, xq, ctx: ForwardContext):
        """`xq`: the normalised hidden states, possibly with their block-quantised copy (ops.QAct) for the shared expert."""
        from ..parallel.ep import ep_moe_forward
        x = ops.dense(xq)
        if self.shared_experts is None:
            idx, w = self.gate(x)
            return ep_moe_forward(self.experts, x, idx, w, ctx, add_in=None)
        if not (x.is_cuda and OVERLAP_SHARED_EXPERTS):
            idx, w = self.gate(x)
            return ep_moe_forward(self.experts, x, idx, w, ctx, add_in=self.shared_experts(xq))
        # The shared expert runs on a side stream next to routing, dispatch and the routed GEMMs (its two small GEMMs leave
        # most SMs idle, and so do the routing kernels); the main stream joins it right before the combine adds its output.
        # Works the same eagerly and under CUDA-graph capture (the fork / join become graph edges).
        # Parity: reference models/deepseek_v2/deepseek_v2.py:560-591 (shared-expert overlap on a side stream).
        main = torch.cuda.current_stream(x.device)
        side = _side_stream(x.device)
        fork = torch.cuda.Event()
        fork.record(main)
        side.wait_event(fork)
        with torch.cuda.stream(side):
            shared = self.shared_experts(xq)
            done = torch.cuda.Event()
            done.record(side)

        def join():
            main.wait_event(done)
            return shared

        idx, w = self.gate(x)
        return ep_moe_forward(self.experts, x, idx, w, ctx, add_in=join)


class DeepseekDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device, force_dense: bool = False):
        super().__init__()
        self.layer_idx = layer_idx
        fp8 = cfg.quant == "fp8"             # the norms feed fp8 linears: they also emit the block-quantised copy
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8)
        self.self_attn = MLAAttention(cfg, layer_idx, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8)
        self.is_moe = cfg.is_moe_layer(layer_idx) and not force_dense
        self.mlp = DeepseekMoE(cfg, dtype, device, layer_idx) if self.is_moe else SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quant, act=cfg.glu_act)

    def forward(self, h, residual, positions, ctx, rope_cache):
        x, residual = self.input_layernorm(h, residual) if residual is not None else (self.input_layernorm(h), h)
        a = self.self_attn(x, positions, ctx, rope_cache)
        x, residual = self.post_attention_layernorm(a, residual)
        m = self.mlp(x, ctx) if self.is_moe else self.mlp(x)
        return m, residual


class DeepseekModel(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, layer_range: Optional[Tuple[int, int]] = None):
        super().__init__()
        self.cfg = cfg
        lo, hi = layer_range or (0, cfg.num_hidden_layers)
        self.layer_range = (lo, hi)
        d = get_dist_context()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device) if d.is_first_pp else None
        self.layers = nn.ModuleDict({str(i): DeepseekDecoderLayer(cfg, i, dtype, device) for i in range(lo, hi)})
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device) if d.is_last_pp else None
        rc = ref.rope_cos_sin_cache(cfg.qk_rope_head_dim, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_scaling)
        self.register_buffer("rope_cache", rc.to(device), persistent=False)

    def forward(self, input_ids, positions, ctx, inputs_embeds=None, residual=None):
        h = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        for i in range(*self.layer_range):
            h, residual = self.layers[str(i)](h, residual, positions, ctx, self.rope_cache)
        if self.norm is None:
            return h, residual           # pipeline boundary: the next stage continues with (h, residual)
        h, _ = self.norm(h, residual)
        return h


class DeepseekV3ForCausalLM(nn.Module):
    """Causal LM over the paged cache: ``forward`` returns final hidden states, ``compute_logits`` applies lm_head."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", layer_range=None):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        self.model = DeepseekModel(cfg, dtype, device, layer_range)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def num_cache_layers(self) -> int:
        return self.cfg.num_hidden_layers

    def forward(self, input_ids, positions, ctx: ForwardContext, inputs_embeds=None):
        return self.model(input_ids, positions, ctx, inputs_embeds)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.lm_head(hidden, self.lm_head.weight)

    # ---- weights ---------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        from .weights import load_deepseek_weights
        return load_deepseek_weights(self, weights)


class DeepseekMTP(nn.Module):
    """Next-n predictor: h' = block(eh_proj([enorm(embed(next_token)) ; hnorm(h_prev)])), logits via the shared head.
    Its KV rows live in cache layers placed after the target model's layers."""

    def __init__(self, cfg: ModelConfig, dtype, device, embed: nn.Embedding, lm_head: nn.Linear):
        super().__init__()
        self.cfg = cfg
        n = max(1, cfg.num_nextn_predict_layers)
        self.embed_tokens, self.shared_head = embed, lm_head
        self.enorm = nn.ModuleList([RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device) for _ in range(n)])
        self.hnorm = nn.ModuleList([RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device) for _ in range(n)])
        self.eh_proj = nn.ModuleList([QLinear(2 * cfg.hidden_size, cfg.hidden_size, dtype, device, None) for _ in range(n)])
        self.blocks = nn.ModuleList([DeepseekDecoderLayer(cfg, cfg.num_hidden_layers + i, dtype, device) for i in range(n)])
        self.final_norm = nn.ModuleList([RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device) for _ in range(n)])
        rc = ref.rope_cos_sin_cache(cfg.qk_rope_head_dim, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_scaling)
        self.register_buffer("rope_cache", rc.to(device), persistent=False)

    def forward(self, input_ids, prev_hidden, positions, ctx, step: int = 0):
        k = step % len(self.blocks)
        e = self.enorm[k](self.embed_tokens(input_ids))
        h = self.hnorm[k](prev_hidden)
        x = self.eh_proj[k](torch.cat([e, h], -1))
        m, residual = self.blocks[k](x, None, positions, ctx, self.rope_cache)
        out, _ = self.final_norm[k](m, residual)
        return out

    def compute_logits(self, hidden):
        return ops.lm_head(hidden, self.shared_head.weight)
