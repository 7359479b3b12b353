"""Kimi-K3 family (text stack): Kimi-delta-attention layers between NoPE MLA layers with a sigmoid output gate, block
attention residuals instead of a plain residual stream, SiTU-GLU MLPs, and routed experts that work in a latent space
(down-projection, experts, norm, up-projection) next to a replicated shared expert.

Parity: reference runtime/models/kimi_k3/kimi_k3.py - MLP :34-70, gated NoPE MLA :73-100, attention residual :103-161,
latent MoE :164-280, decoder layer :283-380, model :383-440; loader kimi_k3_loader.py:30-138 (w1 / w2 / w3 experts, packed
MXFP4 expert tensors, split convolution weights).

B200-first differences: the residual mixture (scores, softmax, combination, output norm and the optional bank write) is one
CUDA kernel with one CTA per token; packed MXFP4 expert tensors are expanded at load time into the block-scaled fp8 (or
bf16) form the grouped tcgen05 GEMM of this package reads; attention runs with attention_tp = 1 (sequences are spread by
attention-DP), so the reduce-scatter placement of the reference's TP8 path has no counterpart here.
"""
from __future__ import annotations

import math
import re
from typing import Iterable, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..parallel.dist import get_dist_context
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .deepseek import MLAAttention, MoEGate
from .kda import KimiDeltaAttention
from .layers import QLinear, RMSNorm, RoutedExperts, SwiGLUMLP


class KimiMoE(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, layer_idx: int):
        super().__init__()
        H, Z = cfg.hidden_size, cfg.routed_expert_hidden_size or cfg.hidden_size
        self.latent = Z if cfg.routed_expert_hidden_size else 0
        self.gate = MoEGate(cfg, device, layer_idx)
        if self.latent:
            self.routed_expert_down_proj = QLinear(H, Z, dtype, device, None)
            self.routed_expert_norm = RMSNorm(Z, cfg.rms_norm_eps, dtype, device)
            self.routed_expert_up_proj = QLinear(Z, H, dtype, device, None)
        self.experts = RoutedExperts(cfg.n_routed_experts, Z, cfg.moe_intermediate_size, dtype, device, cfg.quant, layer_idx, act=cfg.glu_act)
        self.shared_experts = None
        if cfg.n_shared_experts > 0:
            self.shared_experts = SwiGLUMLP(H, cfg.moe_intermediate_size * cfg.n_shared_experts, dtype, device, None, act=cfg.glu_act)

    def forward(self, x, ctx: ForwardContext, prefix: Optional[torch.Tensor] = None):
        from ..parallel.ep import ep_moe_forward
        x = ops.dense(x)
        idx, w = self.gate(x)
        z = self.routed_expert_down_proj(x) if self.latent else x
        out = ep_moe_forward(self.experts, z, idx, w, ctx, add_in=None)
        if self.latent:
            out = self.routed_expert_up_proj(self.routed_expert_norm(out))
        if self.shared_experts is not None:
            out = out + self.shared_experts(x)
        return out if prefix is None else out + prefix


class ResidualBank:
    """Frozen block sums of one forward pass: bank [T, blocks, D], of which the first `valid` rows count."""

    def __init__(self, hidden: torch.Tensor, blocks: int):
        self.bank = hidden.new_empty(hidden.shape[0], max(1, blocks), hidden.shape[1])
        self.valid = 0

    def aggregate(self, prefix, delta, score_w: torch.Tensor, out_norm: RMSNorm, write: bool = False):
        """Layer input = out_norm(mixture of the frozen blocks and the running sum `prefix + delta`).  `write`: this layer
        starts a new block, so the running sum is frozen into the bank.  Returns (input, running sum)."""
        prefix = delta if prefix is None else prefix + delta
        if self.valid:
            out = ops.attn_res_mix(prefix, self.bank, self.valid, score_w, out_norm.weight, out_norm.eps, self.valid if write else -1)
        else:
            out = out_norm(prefix)
            if write:
                self.bank[:, 0].copy_(prefix)
        if write:
            self.valid += 1
        return out, prefix


class KimiDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.kind = cfg.layer_type(layer_idx)
        H = cfg.hidden_size
        if self.kind == "linear_attention":
            self.linear_attn = KimiDeltaAttention(cfg, cfg.num_layers_of("linear_attention", layer_idx), dtype, device)
        else:
            self.self_attn = MLAAttention(cfg, layer_idx, dtype, device, cache_idx=cfg.num_layers_of("full_attention", layer_idx))
        self.is_moe = cfg.is_moe_layer(layer_idx)
        self.mlp = KimiMoE(cfg, dtype, device, layer_idx) if self.is_moe else SwiGLUMLP(H, cfg.intermediate_size, dtype, device, None, act=cfg.glu_act)
        self.input_layernorm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        self.post_attention_layernorm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        self.use_res = cfg.attn_res_block_size > 0
        if self.use_res:
            self.write_block = layer_idx % cfg.attn_res_block_size == 0
            self.self_attention_res_norm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
            self.mlp_res_norm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
            self.self_attention_res_proj = nn.Parameter(torch.zeros(H, dtype=dtype, device=device), requires_grad=False)
            self.mlp_res_proj = nn.Parameter(torch.zeros(H, dtype=dtype, device=device), requires_grad=False)
            self._score_w = None

    def score_weights(self):
        """fp32 (norm weight * projection) vectors of the two residual sites; rebuilt by `refresh` after a weight change."""
        if self._score_w is None:
            self._score_w = ((self.self_attention_res_norm.weight.float() * self.self_attention_res_proj.float()).contiguous(),
                             (self.mlp_res_norm.weight.float() * self.mlp_res_proj.float()).contiguous())
        return self._score_w

    def refresh(self):
        if self.use_res:
            self._score_w = None

    def _attn(self, x, positions, ctx, rope_cache):
        return self.linear_attn(x, ctx) if self.kind == "linear_attention" else self.self_attn(x, positions, ctx, rope_cache)

    def forward(self, hidden, prefix, bank: Optional[ResidualBank], positions, ctx, rope_cache):
        if bank is None:                                   # plain pre-norm residual stream
            if prefix is None:
                prefix, x = hidden, self.input_layernorm(hidden)
            else:
                x, prefix = self.input_layernorm(hidden, prefix)
            a = self._attn(x, positions, ctx, rope_cache)
            x, prefix = self.post_attention_layernorm(a, prefix)
            return (self.mlp(x, ctx) if self.is_moe else self.mlp(x)), prefix
        wa, wm = self.score_weights()
        x, prefix = bank.aggregate(prefix, hidden, wa, self.input_layernorm, write=self.write_block)
        if self.write_block:
            prefix = None
        a = self._attn(x, positions, ctx, rope_cache)
        x, prefix = bank.aggregate(prefix, a, wm, self.post_attention_layernorm)
        out = self.mlp(x, ctx, prefix) if self.is_moe else self.mlp(x) + prefix
        return out, None


class _Inner(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        H = cfg.hidden_size
        self.embed_tokens = nn.Embedding(cfg.vocab_size, H, dtype=dtype, device=device)
        self.layers = nn.ModuleDict({str(i): KimiDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)})
        self.norm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        if cfg.attn_res_block_size > 0:
            self.output_attn_res_norm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
            self.output_attn_res_proj = nn.Parameter(torch.zeros(H, dtype=dtype, device=device), requires_grad=False)


class KimiK3ForConditionalGeneration(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", layer_range=None):
        super().__init__()
        assert layer_range is None, "pipeline stages are not offered for the attention-residual family"
        assert get_dist_context().attn_tp_size == 1, "the attention-residual family runs with attention_tp = 1"
        self.cfg, self.dtype = cfg, dtype
        self.model = _Inner(cfg, dtype, device)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        rd = cfg.qk_rope_head_dim
        if cfg.mla_skip_rope:
            # no rotary embedding: one row of (cos = 1 | sin = 0), addressed with position 0 for every token
            rc = torch.cat([torch.ones(1, rd // 2), torch.zeros(1, rd // 2)], 1)
        else:
            rc = ref.rope_cos_sin_cache(rd, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_scaling)
        self.register_buffer("rope_cache", rc.float().to(device), persistent=False)
        self.blocks = math.ceil(cfg.num_hidden_layers / cfg.attn_res_block_size) if cfg.attn_res_block_size > 0 else 0
        self._out_w = None
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def num_cache_layers(self) -> int:
        return self.cfg.num_layers_of("full_attention")

    def refresh(self):
        """Drop the vectors derived from the residual norms / projections (call after writing those weights)."""
        self._out_w = None
        for L in self.model.layers.values():
            L.refresh()

    def forward(self, input_ids, positions, ctx: ForwardContext, inputs_embeds=None):
        hidden = inputs_embeds if inputs_embeds is not None else self.model.embed_tokens(input_ids)
        pos = torch.zeros_like(positions) if self.cfg.mla_skip_rope else positions
        bank = ResidualBank(hidden, self.blocks) if self.blocks else None
        prefix = None
        for i in range(self.cfg.num_hidden_layers):
            hidden, prefix = self.model.layers[str(i)](hidden, prefix, bank, pos, ctx, self.rope_cache)
        if bank is None:
            h, _ = self.model.norm(hidden, prefix)
            return h
        if self._out_w is None:
            self._out_w = (self.model.output_attn_res_norm.weight.float() * self.model.output_attn_res_proj.float()).contiguous()
        h, _ = bank.aggregate(prefix, hidden, self._out_w, self.model.norm)
        return h

    def compute_logits(self, hidden):
        return ops.lm_head(hidden, self.lm_head.weight)

    # ---- weights ---------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        from .weights import load_deepseek_weights
        cfg = self.cfg
        n = 0
        attn_re = re.compile(r"model\.layers\.(\d+)\.self_attn\.(.+)$")
        layer_re = re.compile(r"model\.layers\.(\d+)\.(.+)$")
        expert_re = re.compile(r"(model\.layers\.\d+\.mlp\.experts\.\d+)\.(w[123])\.(weight|weight_packed|weight_scale|weight_scale_inv)$")
        packed = {}
        proj_name = {"w1": "gate_proj", "w2": "down_proj", "w3": "up_proj"}

        def rest():
            nonlocal n
            for name, t in weights:
                if name.startswith(("vision_tower.", "mm_projector.")):
                    continue
                if name.startswith("language_model."):
                    name = name[len("language_model."):]
                name = name.replace(".block_sparse_moe.", ".mlp.").replace(".mlp.e_score_correction_bias", ".mlp.gate.e_score_correction_bias")
                e = expert_re.match(name)
                if e:
                    base, proj, kind = f"{e.group(1)}.{proj_name[e.group(2)]}", e.group(2), e.group(3)
                    if kind in ("weight_packed", "weight_scale"):          # MXFP4: e2m1 nibbles + e8m0 scales per 32 values
                        g = packed.setdefault(base, {})
                        g[kind] = t
                        if len(g) == 2:
                            yield base + ".weight", ref.mxfp4_dequant(g["weight_packed"], g["weight_scale"])
                            packed.pop(base)
                    else:
                        yield f"{base}.{kind}", t
                    continue
                m = attn_re.match(name)
                if m and int(m.group(1)) < cfg.num_hidden_layers and cfg.layer_type(int(m.group(1))) == "linear_attention":
                    if self.model.layers[m.group(1)].linear_attn.load(m.group(2), t):
                        n += 1
                    continue
                m = layer_re.match(name)
                if m and int(m.group(1)) < cfg.num_hidden_layers:
                    L, leaf = self.model.layers[m.group(1)], m.group(2)
                    if leaf in ("self_attention_res_norm.weight", "mlp_res_norm.weight"):
                        getattr(L, leaf[:-7]).weight.copy_(t.to(self.dtype)); n += 1; continue
                    if leaf in ("self_attention_res_proj.weight", "mlp_res_proj.weight"):
                        getattr(L, leaf[:-7]).copy_(t.reshape(-1).to(self.dtype)); n += 1; continue
                    if leaf.startswith("mlp.routed_expert_") and L.is_moe:
                        mod = getattr(L.mlp, leaf[4:-7])
                        (mod.weight.copy_(t.to(self.dtype)) if isinstance(mod, RMSNorm) else mod.set_weight(t.float())); n += 1; continue
                if name == "model.output_attn_res_norm.weight":
                    self.model.output_attn_res_norm.weight.copy_(t.to(self.dtype)); n += 1; continue
                if name == "model.output_attn_res_proj.weight":
                    self.model.output_attn_res_proj.copy_(t.reshape(-1).to(self.dtype)); n += 1; continue
                yield name, t

        with torch.no_grad():
            n += load_deepseek_weights(self, rest())
        if packed:
            raise ValueError(f"incomplete checkpoint: packed expert tensors without their scales {list(packed)[:3]}")
        for i in range(cfg.num_hidden_layers):
            L = self.model.layers[str(i)]
            if L.kind == "linear_attention" and L.linear_attn.pending():
                raise ValueError(f"incomplete checkpoint: layer {i} delta-attention parts {L.linear_attn.pending()}")
        self.refresh()
        return n
