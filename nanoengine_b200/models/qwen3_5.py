"""Qwen3.5 dense and Qwen3.5-MoE: a hybrid stack of gated delta-net (linear attention) layers and gated full-attention layers.

Linear-attention layer   qkv / z / a / b projections -> causal depthwise conv (+SiLU) over [q | k | v] with a carried window
                         -> gated delta rule on a per-sequence state [Hv, Dv, Dk] -> RMSNorm gated by silu(z) -> out_proj.
Full-attention layer     GQA whose q projection also carries a per-head output gate; per-head q/k RMSNorm with (1 + w) weights;
                         RoPE on the first `partial_rotary_factor` of each head; paged attention; sigmoid(gate) * o -> o_proj.
Every RMSNorm of the stack stores its weight as the deviation from one.  The MoE variant routes with softmax top-k and adds one
always-on expert scaled by a per-token sigmoid gate.

The paged KV cache holds only the full-attention layers; the delta-net layers index the recurrent-state pools by the sequence's
state slot, so a layer carries two indices: its position among the layers of its own kind.

Attention tensor parallelism is not offered for this family (the delta-net projections would be replicated on every rank, as
the reference does); expert parallelism of the MoE variant works as for the other families.

Parity: reference runtime/models/qwen3_5/qwen3_5.py:34-350, models/qwen3_5_moe/qwen3_5_moe.py:57-340 (full attention :57-192,
sparse block :248-340), layers/backends/delta_net/generic.py:56-329, qwen3_5_loader.py:25-121.
"""
from __future__ import annotations

import re
from typing import Iterable, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..parallel.dist import get_dist_context
from ..parallel.ep import ep_moe_forward
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .layers import QLinear, RMSNorm, RoutedExperts, SwiGLUMLP


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, state_idx: int, dtype, device):
        super().__init__()
        self.state_idx = state_idx
        self.hk, self.hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
        self.conv_dim, self.conv_k = cfg.gdn_conv_dim, cfg.linear_conv_kernel_dim
        H = cfg.hidden_size
        self.eps = cfg.rms_norm_eps
        # one GEMM for [q | k | v | z]; the two small gate projections stay in the activation dtype
        self.in_proj = QLinear(H, self.conv_dim + self.value_dim, dtype, device, cfg.quant)
        self.in_proj_ab = QLinear(H, 2 * self.hv, dtype, device, None)
        self.out_proj = QLinear(self.value_dim, H, dtype, device, cfg.quant)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_dim, self.conv_k, dtype=dtype, device=device), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.ones(self.hv, dtype=torch.float32, device=device), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.hv, dtype=torch.float32, device=device), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.dv, dtype=dtype, device=device), requires_grad=False)

    def forward(self, x, ctx: ForwardContext):
        T = x.shape[0]
        proj = self.in_proj(x)
        ab = self.in_proj_ab(x)
        qkv, z = proj[:, : self.conv_dim], proj[:, self.conv_dim:]
        uniform_one = (not ctx.is_prefill) and ctx.q_len_uniform == 1
        y = ops.gdn_conv(qkv, self.conv_weight, ctx.conv_states[self.state_idx], ctx.state_slots, ctx.cu_seqlens_q, ctx.seq_fresh,
                         uniform_one)
        q = y[:, : self.key_dim].view(T, self.hk, self.dk)
        k = y[:, self.key_dim: 2 * self.key_dim].view(T, self.hk, self.dk)
        v = y[:, 2 * self.key_dim:].view(T, self.hv, self.dv)
        o = ops.gdn_recurrent(q, k, v, ab[:, : self.hv], ab[:, self.hv:], self.A_log, self.dt_bias, ctx.rec_states[self.state_idx],
                              ctx.state_slots, ctx.cu_seqlens_q, ctx.seq_fresh, z.reshape(T, self.hv, self.dv), self.norm_weight,
                              self.eps, ctx.max_seqlen_q, ctx.cu_seqlens_q_host)
        return self.out_proj(o)


def _rope_head_prefix(x, rot: int, positions, rope_cache):
    """Rotate the leading `rot` dims of every head of x [T, heads, head_dim]; the rest of each head passes through."""
    if x.is_cuda:
        part = x[..., :rot]
        ops.apply_rope(part, positions, rope_cache, False, part)      # in place on the strided view
        return x
    return torch.cat([ops.apply_rope(x[..., :rot], positions, rope_cache, False), x[..., rot:]], -1)


class GatedAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, cache_idx: int, dtype, device):
        super().__init__()
        self.cache_idx = cache_idx
        self.hd, self.hq, self.hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        self.gated = cfg.attn_output_gate
        self.rot = int(self.hd * cfg.partial_rotary_factor)
        self.qkv_proj = QLinear(cfg.hidden_size, (self.hq * (2 if self.gated else 1) + 2 * self.hkv) * self.hd, dtype, device, cfg.quant,
                                bias=cfg.attention_bias)
        self.o_proj = QLinear(self.hq * self.hd, cfg.hidden_size, dtype, device, cfg.quant)
        self.q_norm = RMSNorm(self.hd, cfg.rms_norm_eps, dtype, device, unit_offset=cfg.norm_unit_offset)
        self.k_norm = RMSNorm(self.hd, cfg.rms_norm_eps, dtype, device, unit_offset=cfg.norm_unit_offset)
        self.scale = self.hd ** -0.5

    def forward(self, x, positions, ctx: ForwardContext, rope_cache):
        T, hd, hq, hkv = x.shape[0], self.hd, self.hq, self.hkv
        qkv = self.qkv_proj(x)
        qw = hq * hd * (2 if self.gated else 1)
        qg, k, v = qkv.split([qw, hkv * hd, hkv * hd], -1)
        if self.gated:
            qg = qg.view(T, hq, 2 * hd)
            q, gate = qg[..., :hd], qg[..., hd:]
        else:
            q, gate = qg.view(T, hq, hd), None
        q = self.q_norm(q.reshape(-1, hd)).view(T, hq, hd)
        k = self.k_norm(k.reshape(-1, hd)).view(T, hkv, hd)
        v = v.reshape(T, hkv, hd)
        if self.rot > 0:
            q = _rope_head_prefix(q, self.rot, positions, rope_cache)
            k = _rope_head_prefix(k, self.rot, positions, rope_cache)
        kc, vc = ctx.kv_caches[self.cache_idx]
        ops.gqa_kv_store(kc, vc, ctx.slot_mapping, k, v)
        o = ops.gqa_attention_paged(q, kc, vc, ctx.block_tables, ctx.cu_seqlens_q, ctx.context_lens, self.scale)
        if gate is not None:
            o = ops.sigmoid_gate(o.reshape(T, hq, hd), gate)
        return self.o_proj(o.reshape(T, hq * hd))


class Qwen35MoE(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.gate_weight = nn.Parameter(torch.empty(cfg.n_routed_experts, cfg.hidden_size, dtype=torch.float32, device=device), requires_grad=False)
        self.experts = RoutedExperts(cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size, dtype, device, cfg.quant)
        self.shared_expert = None
        if cfg.shared_expert_intermediate_size:
            self.shared_expert = SwiGLUMLP(cfg.hidden_size, cfg.shared_expert_intermediate_size, dtype, device, cfg.quant)
            self.shared_gate_weight = nn.Parameter(torch.zeros(1, cfg.hidden_size, dtype=torch.float32, device=device), requires_grad=False)

    def forward(self, xq, ctx):
        c = self.cfg
        x = ops.dense(xq)
        logits = ops.router_logits(x, self.gate_weight)
        idx, w = ops.moe_route(logits, None, c.num_experts_per_tok, 1, 1, c.norm_topk_prob, 1.0, "softmax")
        add_in = None
        if self.shared_expert is not None:
            lg = ops.router_logits(x, self.shared_gate_weight)
            g = torch.sigmoid(lg.sum(0) if lg.dim() == 3 else lg)                      # [T, 1] fp32 (the CUDA body returns split-K planes)
            add_in = (self.shared_expert(xq).float() * g).to(x.dtype)
        return ep_moe_forward(self.experts, x, idx, w, ctx, add_in)


class Qwen35DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        uo = cfg.norm_unit_offset
        self.kind = cfg.layer_type(layer_idx)
        fp8 = cfg.quant == "fp8"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, unit_offset=uo, quant_out=fp8)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, unit_offset=uo, quant_out=fp8)
        if self.kind == "linear_attention":
            self.linear_attn = GatedDeltaNet(cfg, cfg.num_layers_of("linear_attention", layer_idx), dtype, device)
        elif self.kind == "full_attention":
            self.self_attn = GatedAttention(cfg, cfg.num_layers_of("full_attention", layer_idx), dtype, device)
        else:
            raise ValueError(f"unsupported layer type {self.kind}")
        self.is_moe = cfg.is_moe_layer(layer_idx)
        self.mlp = Qwen35MoE(cfg, dtype, device) if self.is_moe else SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quant)

    def forward(self, h, residual, positions, ctx, rope_cache):
        x, residual = self.input_layernorm(h, residual) if residual is not None else (self.input_layernorm(h), h)
        a = self.linear_attn(x, ctx) if self.kind == "linear_attention" else self.self_attn(x, positions, ctx, rope_cache)
        x, residual = self.post_attention_layernorm(a, residual)
        return (self.mlp(x, ctx) if self.is_moe else self.mlp(x)), residual


class Qwen35ForCausalLM(nn.Module):
    """Serves Qwen3_5ForConditionalGeneration (dense) and Qwen3_5MoeForConditionalGeneration (text stack only)."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", layer_range=None):
        super().__init__()
        assert get_dist_context().attn_tp_size == 1, "the hybrid delta-net family runs with attention_tp = 1"
        assert layer_range is None, "pipeline stages are not offered for the hybrid delta-net family"
        self.cfg, self.dtype = cfg, dtype
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([Qwen35DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, unit_offset=cfg.norm_unit_offset)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        rot = max(2, int(cfg.head_dim * cfg.partial_rotary_factor))
        rc = ref.rope_cos_sin_cache(rot, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_scaling)
        self.register_buffer("rope_cache", rc.to(device), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def num_cache_layers(self) -> int:
        return self.cfg.num_layers_of("full_attention")

    def forward(self, input_ids, positions, ctx: ForwardContext, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        residual = None
        for layer in self.layers:
            h, residual = layer(h, residual, positions, ctx, self.rope_cache)
        h, _ = self.norm(h, residual)
        return h

    def compute_logits(self, hidden):
        return ops.lm_head(hidden, self.lm_head.weight)

    # ---- weights ---------------------------------------------------------------------------
    @staticmethod
    def _normalise_name(name: str):
        """Checkpoints of this family nest the text stack under `model.language_model.` and also ship vision / MTP tensors."""
        for pre in ("model.language_model.", "language_model.model.", "language_model."):
            if name.startswith(pre):
                return "model." + name[len(pre):]
        if name.startswith(("model.embed_tokens.", "model.layers.", "model.norm.", "lm_head.")):
            return name
        return None

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        cfg = self.cfg
        n = 0
        pending, scales, wbuf = {}, {}, {}
        fp8 = torch.float8_e4m3fn
        saw_head = False

        def deq(w, s):
            return ref.dequant_fp8_block(w, s) if w.dtype == fp8 else w.float()

        def merge(key, part, value, order, setter):
            g = pending.setdefault(key, {})
            g[part] = value
            if len(g) == len(order):
                setter(torch.cat([g[o] for o in order], 0))
                pending.pop(key)

        def place(base, w, s):
            nonlocal n, saw_head
            n += 1
            if base == "model.embed_tokens":
                self.embed_tokens.weight.copy_(w.to(self.dtype)); return
            if base == "lm_head":
                saw_head = True
                self.lm_head.weight.copy_(w.to(self.dtype)); return
            if base == "model.norm":
                self.norm.weight.copy_(w.to(self.dtype)); return
            m = re.match(r"model\.layers\.(\d+)\.(.*)", base)
            if not m or int(m.group(1)) >= cfg.num_hidden_layers:
                n -= 1
                return
            li, rest = m.group(1), m.group(2)
            L = self.layers[int(li)]
            if rest in ("input_layernorm", "post_attention_layernorm"):
                getattr(L, rest).weight.copy_(w.to(self.dtype)); return
            if rest.startswith("linear_attn."):
                G, leaf = L.linear_attn, rest[len("linear_attn."):]
                if leaf in ("in_proj_qkv", "in_proj_z"):
                    merge(li + ".in_proj", leaf, deq(w, s), ("in_proj_qkv", "in_proj_z"), G.in_proj.set_weight)
                elif leaf in ("in_proj_a", "in_proj_b"):
                    merge(li + ".ab", leaf, w.float(), ("in_proj_a", "in_proj_b"), G.in_proj_ab.set_weight)
                elif leaf == "conv1d":
                    G.conv_weight.copy_(w.reshape(G.conv_dim, G.conv_k).to(self.dtype))
                elif leaf == "norm":
                    G.norm_weight.copy_(w.to(self.dtype))
                elif leaf == "out_proj":
                    G.out_proj.set_weight(w, s)
                elif leaf == "dt_bias":
                    G.dt_bias.copy_(w.float())
                elif leaf == "A_log":
                    G.A_log.copy_(w.float())
                else:
                    n -= 1
                return
            if rest.startswith("self_attn."):
                A, leaf = L.self_attn, rest[len("self_attn."):]
                if leaf in ("q_norm", "k_norm"):
                    getattr(A, leaf).weight.copy_(w.to(self.dtype))
                elif leaf in ("q_proj", "k_proj", "v_proj"):
                    merge(li + ".qkv", leaf, deq(w, s), ("q_proj", "k_proj", "v_proj"), A.qkv_proj.set_weight)
                elif leaf == "o_proj":
                    A.o_proj.set_weight(w, s)
                else:
                    n -= 1
                return
            if rest == "mlp.gate":
                L.mlp.gate_weight.copy_(w.float()); return
            if rest == "mlp.shared_expert_gate":
                L.mlp.shared_gate_weight.copy_(w.float().view(1, -1)); return
            e = re.match(r"mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)$", rest)
            if e:
                eid, which = int(e.group(1)), e.group(2)[:-5]
                ex = L.mlp.experts
                if not ex.load_expert(eid, which, w, s):
                    n -= 1
                return
            sm = re.match(r"mlp\.(shared_expert\.)?(gate_proj|up_proj|down_proj)$", rest)
            if sm:
                mlp = L.mlp.shared_expert if sm.group(1) else L.mlp
                if sm.group(2) == "down_proj":
                    mlp.down_proj.set_weight(w, s)
                else:
                    merge(li + (".sgu" if sm.group(1) else ".gu"), sm.group(2), deq(w, s), ("gate_proj", "up_proj"), mlp.gate_up_proj.set_weight)
                return
            n -= 1

        with torch.no_grad():
            for raw, t in weights:
                name = self._normalise_name(raw)
                if name is None:
                    continue
                if name.endswith(".weight_scale_inv"):
                    base = name[: -len(".weight_scale_inv")]
                    if base in wbuf:
                        place(base, wbuf.pop(base), t)
                    else:
                        scales[base] = t
                    continue
                if name.endswith((".dt_bias", ".A_log")):
                    place(name, t, None)
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
            if not saw_head and cfg.tie_word_embeddings:
                self.lm_head.weight.copy_(self.embed_tokens.weight)
        if pending or wbuf:
            raise ValueError(f"incomplete checkpoint: {list(pending)[:3]} {list(wbuf)[:3]}")
        return n
