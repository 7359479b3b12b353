"""Gemma4 family (text stack): grouped-query attention where sliding-window layers and global layers have their own head
dims and rotary tables, the last layers read the keys / values an earlier layer of their type stored, q / k / v RMSNorm with
a softmax scale of one, GeGLU MLPs between sandwich norms, per-layer input embeddings, a learned scalar per layer, scaled
and tied embeddings and soft-capped logits.

Parity: reference runtime/models/gemma4/gemma4.py - rotary tables :43-87, attention :131-245 (KV sharing :142-150,
:228-241), MLP :248-276, decoder layer :279-350, per-layer inputs :401-440, model :353-470, logits :488-493; loader
gemma4_loader.py:14-116 (K / V tensors of KV-sharing layers are skipped).

B200-first differences: q, k and v of a layer are one GEMM; the per-layer-input table lives on the device (the reference
keeps it in host memory and copies rows per step) so the whole step replays from one CUDA graph; the window is a kernel
argument of the paged attention, not a separate cache type; cache layers with a smaller head dim use the front of
equally sized slabs.
"""
from __future__ import annotations

import math
import re
from typing import Iterable, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..parallel.dist import get_dist_context
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .layers import QLinear, RMSNorm, SwiGLUMLP


def gemma_rope_cache(head_dim: int, max_pos: int, theta: float, partial: float = 1.0, proportional: bool = False) -> torch.Tensor:
    """[max_pos, head_dim] fp32 (cos | sin) for pairs (i, i + head_dim / 2).  `proportional`: only the first
    partial * head_dim / 2 pairs rotate (with exponents spaced over the full head dim), the rest keep angle zero."""
    half = head_dim // 2
    if proportional:
        rot = int(partial * head_dim // 2)
        inv = 1.0 / (theta ** (torch.arange(0, 2 * rot, 2, dtype=torch.float32) / head_dim))
        inv = torch.cat([inv, torch.zeros(half - rot)]) if rot < half else inv
    else:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    f = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.cat([f.cos(), f.sin()], -1)


class Gemma4Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, cache_idx: int, dtype, device):
        super().__init__()
        self.kind = cfg.attn_layer_type(layer_idx)
        self.window = cfg.sliding_window if self.kind == "sliding_attention" else 0
        self.shared = cfg.kv_source_layer(layer_idx) != layer_idx        # reads another layer's keys / values, stores none
        self.cache_idx = cache_idx
        self.hq, self.hkv, self.hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.attn_head_dim(layer_idx)
        out = self.hq * self.hd + (0 if self.shared else 2 * self.hkv * self.hd)
        self.qkv_proj = QLinear(cfg.hidden_size, out, dtype, device, None, bias=cfg.attention_bias)
        self.o_proj = QLinear(self.hq * self.hd, cfg.hidden_size, dtype, device, None)
        self.q_norm = RMSNorm(self.hd, cfg.rms_norm_eps, dtype, device)
        if not self.shared:
            self.k_norm = RMSNorm(self.hd, cfg.rms_norm_eps, dtype, device)
            self.v_norm = RMSNorm(self.hd, cfg.rms_norm_eps, dtype, device)

    def forward(self, x, positions, ctx: ForwardContext, rope_cache):
        T, hq, hkv, hd = x.shape[0], self.hq, self.hkv, self.hd
        qkv = self.qkv_proj(x)
        q = self.q_norm(qkv[:, : hq * hd].reshape(-1, hd)).view(T, hq, hd)
        q = ops.apply_rope(q, positions, rope_cache, False)
        kc, vc = ctx.kv_caches[self.cache_idx]
        if not self.shared:
            k = self.k_norm(qkv[:, hq * hd: (hq + hkv) * hd].reshape(-1, hd)).view(T, hkv, hd)
            v = self.v_norm(qkv[:, (hq + hkv) * hd:].reshape(-1, hd)).view(T, hkv, hd)
            k = ops.apply_rope(k, positions, rope_cache, False)
            ops.gqa_kv_store(kc, vc, ctx.slot_mapping, k, v)
        o = ops.gqa_attention_paged(q, kc, vc, ctx.block_tables, ctx.cu_seqlens_q, ctx.context_lens, 1.0, self.window)
        return self.o_proj(o.reshape(T, hq * hd))


class Gemma4DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, cache_idx: int, dtype, device):
        super().__init__()
        H, eps = cfg.hidden_size, cfg.rms_norm_eps
        self.self_attn = Gemma4Attention(cfg, layer_idx, cache_idx, dtype, device)
        wide = cfg.use_double_wide_mlp and self.self_attn.shared
        self.mlp = SwiGLUMLP(H, cfg.intermediate_size * (2 if wide else 1), dtype, device, None, act=cfg.glu_act)
        self.input_layernorm = RMSNorm(H, eps, dtype, device)
        self.post_attention_layernorm = RMSNorm(H, eps, dtype, device)
        self.pre_feedforward_layernorm = RMSNorm(H, eps, dtype, device)
        self.post_feedforward_layernorm = RMSNorm(H, eps, dtype, device)
        self.layer_scalar = nn.Parameter(torch.ones(1, dtype=dtype, device=device), requires_grad=False)
        self.P = cfg.hidden_size_per_layer_input
        if self.P:
            self.per_layer_input_gate = QLinear(H, self.P, dtype, device, None)
            self.per_layer_projection = QLinear(self.P, H, dtype, device, None)
            self.post_per_layer_input_norm = RMSNorm(H, eps, dtype, device)
        self.act = cfg.glu_act

    def forward(self, h, positions, ctx, rope_cache, per_layer_input):
        a = self.self_attn(self.input_layernorm(h), positions, ctx, rope_cache)
        h = h + self.post_attention_layernorm(a)
        m = self.mlp(self.pre_feedforward_layernorm(h))
        h = h + self.post_feedforward_layernorm(m)
        if self.P:
            g = self.per_layer_input_gate(h)
            g = ops.silu_and_mul(torch.cat([g, per_layer_input], -1), act=self.act)         # act(gate) * per-layer input
            h = h + self.post_per_layer_input_norm(self.per_layer_projection(g))
        return h * self.layer_scalar


class _Inner(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        H, L, P = cfg.hidden_size, cfg.num_hidden_layers, cfg.hidden_size_per_layer_input
        self.embed_tokens = nn.Embedding(cfg.vocab_size, H, dtype=dtype, device=device)
        own = [i for i in range(L) if cfg.kv_source_layer(i) == i]
        self.layers = nn.ModuleDict({str(i): Gemma4DecoderLayer(cfg, i, own.index(cfg.kv_source_layer(i)), dtype, device) for i in range(L)})
        self.norm = RMSNorm(H, cfg.rms_norm_eps, dtype, device)
        if P:
            self.embed_tokens_per_layer = nn.Embedding(cfg.vocab_size_per_layer_input or cfg.vocab_size, L * P, dtype=dtype, device=device)
            self.per_layer_model_projection = QLinear(H, L * P, dtype, device, None)
            self.per_layer_projection_norm = RMSNorm(P, cfg.rms_norm_eps, dtype, device)


class Gemma4ForCausalLM(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", layer_range=None):
        super().__init__()
        assert layer_range is None and get_dist_context().attn_tp_size == 1, "this family runs with attention_tp = pp = 1"
        self.cfg, self.dtype = cfg, dtype
        self.model = _Inner(cfg, dtype, device)
        self.lm_head = None if cfg.tie_word_embeddings else nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        self.embed_scale = math.sqrt(cfg.hidden_size)
        rp = cfg.rope_parameters_by_type or {}
        for kind in ("sliding_attention", "full_attention"):
            r = rp.get(kind, {})
            hd = cfg.global_head_dim if (kind == "full_attention" and cfg.global_head_dim) else cfg.head_dim
            rc = gemma_rope_cache(hd, cfg.max_position_embeddings, float(r.get("rope_theta", cfg.rope_theta)),
                                  float(r.get("partial_rotary_factor", 1.0)), r.get("rope_type") == "proportional")
            self.register_buffer("rope_" + kind, rc.to(device), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def num_cache_layers(self) -> int:
        return sum(1 for i in range(self.cfg.num_hidden_layers) if self.cfg.kv_source_layer(i) == i)

    def _per_layer_inputs(self, input_ids, h):
        cfg = self.cfg
        L, P = cfg.num_hidden_layers, cfg.hidden_size_per_layer_input
        M = self.model
        tok = M.embed_tokens_per_layer(input_ids).view(-1, L, P) * math.sqrt(P)
        proj = (M.per_layer_model_projection(h) * cfg.hidden_size ** -0.5).view(-1, L, P)
        proj = M.per_layer_projection_norm(proj.reshape(-1, P)).view(-1, L, P)
        return (proj + tok) * 2.0 ** -0.5

    def forward(self, input_ids, positions, ctx: ForwardContext, inputs_embeds=None):
        cfg = self.cfg
        h = inputs_embeds if inputs_embeds is not None else self.model.embed_tokens(input_ids) * self.embed_scale
        pli = self._per_layer_inputs(input_ids, h) if cfg.hidden_size_per_layer_input else None
        for i in range(cfg.num_hidden_layers):
            rope = self.rope_sliding_attention if cfg.attn_layer_type(i) == "sliding_attention" else self.rope_full_attention
            h = self.model.layers[str(i)](h, positions, ctx, rope, pli[:, i].contiguous() if pli is not None else None)
        return self.model.norm(h)

    def compute_logits(self, hidden):
        w = self.model.embed_tokens.weight if self.lm_head is None else self.lm_head.weight
        logits = ops.lm_head(hidden, w)
        cap = self.cfg.final_logit_softcapping
        return torch.tanh(logits / cap) * cap if cap else logits

    # ---- weights ---------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        cfg = self.cfg
        n = 0
        skip = ("rotary_emb.", "vision_tower.", "audio_tower.", "model.embed_audio.", "model.embed_vision.", "multi_modal_projector.")
        lre = re.compile(r"model\.layers\.(\d+)\.(.+)$")
        parts = {}
        with torch.no_grad():
            for name, t in weights:
                for pre in ("model.language_model.", "language_model.model.", "language_model."):
                    if name.startswith(pre):
                        name = "model." + name[len(pre):]
                        break
                if any(s in name for s in skip):
                    continue
                M = self.model
                if name == "model.embed_tokens.weight":
                    M.embed_tokens.weight.copy_(t.to(self.dtype)); n += 1; continue
                if name == "lm_head.weight":
                    if self.lm_head is not None:
                        self.lm_head.weight.copy_(t.to(self.dtype)); n += 1
                    continue
                if name == "model.norm.weight":
                    M.norm.weight.copy_(t.to(self.dtype)); n += 1; continue
                if name == "model.embed_tokens_per_layer.weight" and cfg.hidden_size_per_layer_input:
                    M.embed_tokens_per_layer.weight.copy_(t.to(self.dtype)); n += 1; continue
                if name == "model.per_layer_model_projection.weight" and cfg.hidden_size_per_layer_input:
                    M.per_layer_model_projection.set_weight(t.float()); n += 1; continue
                if name == "model.per_layer_projection_norm.weight" and cfg.hidden_size_per_layer_input:
                    M.per_layer_projection_norm.weight.copy_(t.to(self.dtype)); n += 1; continue
                m = lre.match(name)
                if not m or int(m.group(1)) >= cfg.num_hidden_layers:
                    continue
                L, leaf = M.layers[m.group(1)], m.group(2)
                A = L.self_attn
                if leaf == "layer_scalar":
                    L.layer_scalar.copy_(t.reshape(1).to(self.dtype)); n += 1; continue
                if not leaf.endswith(".weight"):
                    continue
                leaf = leaf[:-7]
                if leaf in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm",
                            "post_per_layer_input_norm"):
                    if hasattr(L, leaf):
                        getattr(L, leaf).weight.copy_(t.to(self.dtype)); n += 1
                    continue
                if leaf in ("per_layer_input_gate", "per_layer_projection"):
                    if L.P:
                        getattr(L, leaf).set_weight(t.float()); n += 1
                    continue
                if leaf in ("self_attn.q_norm", "self_attn.k_norm", "self_attn.v_norm"):
                    mod = getattr(A, leaf.split(".")[1], None)
                    if mod is not None:                       # KV-sharing layers keep no k / v norms
                        mod.weight.copy_(t.to(self.dtype)); n += 1
                    continue
                if leaf in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                    which = leaf.split(".")[1]
                    if A.shared:
                        if which == "q_proj":
                            A.qkv_proj.set_weight(t.float()); n += 1
                        continue                              # the checkpoint keeps K / V tensors these layers never use
                    g = parts.setdefault(m.group(1) + ".qkv", {})
                    g[which] = t.float()
                    if len(g) == 3:
                        A.qkv_proj.set_weight(torch.cat([g["q_proj"], g["k_proj"], g["v_proj"]], 0)); parts.pop(m.group(1) + ".qkv")
                    n += 1
                    continue
                if leaf == "self_attn.o_proj":
                    A.o_proj.set_weight(t.float()); n += 1; continue
                if leaf in ("mlp.gate_proj", "mlp.up_proj"):
                    g = parts.setdefault(m.group(1) + ".gu", {})
                    g[leaf.split(".")[1]] = t.float()
                    if len(g) == 2:
                        L.mlp.gate_up_proj.set_weight(torch.cat([g["gate_proj"], g["up_proj"]], 0)); parts.pop(m.group(1) + ".gu")
                    n += 1
                    continue
                if leaf == "mlp.down_proj":
                    L.mlp.down_proj.set_weight(t.float()); n += 1; continue
        if parts:
            raise ValueError(f"incomplete checkpoint: {list(parts)[:3]}")
        return n
