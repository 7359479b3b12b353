"""DeepSeek-V4 family: every token owns ONE key / value row per layer (`head_dim` wide, the last `qk_rope_head_dim` dims rotated,
the rest kept as an fp8 cache would return them), all heads attend it (multi-query), and a token sees the last `window_size` raw
rows plus - in a compressing layer - every row pooled over `ratio` earlier tokens (softmax-weighted pooling with a learned
position-in-block bias; ratio 4 pools over two overlapping blocks), with one learned sink logit per head in the softmax
denominator.  The output is un-rotated, projected per head group to a low rank and then to the hidden size.  The hidden state is
`hc_mult` streams under manifold-constrained hyper-connections (contracted by a learned sigmoid mix in front of the final norm),
the FFN is a DeepSeek MoE with sqrt-softplus scores, a clamped SwiGLU in the routed experts and token-id ("hash") routing in the
first layers.

Parity: reference runtime/models/deepseek_v4/deepseek_v4.py - hyper-connection projector :743-822 and head :825-844, compressor
:858-1176, attention :1461-1593 (parameters), :1676-1785 (window + pooled candidates, sink softmax), :2381-2496 (forward), MoE
:2513-2700, decoder layer :2703-2804, model :2807-2861, config spellings :2894-2921; deepseek_v4_loader.py:49-82 (checkpoint
names), :101-137 (packed 4-bit experts).

How it runs here.  The linear layers, norms, hyper-connection mixes, router and experts are the kernels of this package.  The
compressor, the window / pooled-row gather and the sink softmax are stated in PyTorch ops (`ops.reference.dsv4_*`,
`sink_attention`) on either device: decode is one batched pass without host reads, prefill walks the sequences of the step in
query tiles.  The engine therefore runs this family eagerly, with attention_tp = pp = 1 and without speculative decoding.
Chunked prefill, preemption and PD migration work (the compressor carries its unfinished block per sequence slot); prefix reuse is
off, as for every family with per-sequence state.  With kv_cache_dtype = "fp8" the raw and the pooled rows are stored packed
(e4m3 values with one power-of-two scale byte per 64, bf16 rotated dims: 584 bytes per 512-wide row), otherwise as plain values.
"""
from __future__ import annotations

import re
from typing import Iterable, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..parallel.dist import get_dist_context
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .glm5_next import HyperConnection
from .layers import QLinear, RMSNorm, RoutedExperts, SwiGLUMLP

QUERY_TILE = 128


def rotate_tail(x: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor, rd: int, inverse: bool = False) -> torch.Tensor:
    """Rotate the last `rd` dims of x [T, ..., D] in place (pairs (2i, 2i+1)); `inverse` turns them back."""
    cs = cache[positions.long()]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [rd // 2]
    cos, sin = cs[:, : rd // 2].view(shape), cs[:, rd // 2:].view(shape)
    if inverse:
        sin = -sin
    t = x[..., -rd:].float()
    a, b = t[..., 0::2], t[..., 1::2]
    x[..., -rd:] = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2).to(x.dtype)
    return x


def cache_store(cache: torch.Tensor, page: torch.Tensor, off: torch.Tensor, rows: torch.Tensor, rd: int) -> None:
    """Write rows [N, D] at (page, off) of a cache [blocks, rows_per_page, D] - or [blocks, rows_per_page, row_bytes] uint8, packed."""
    cache[page, off] = ref.dsv4_pack_rows(rows, rd) if cache.dtype == torch.uint8 else rows.to(cache.dtype)


def cache_load(cache: torch.Tensor, page: torch.Tensor, off: torch.Tensor, d: int, rd: int, dtype) -> torch.Tensor:
    rows = cache[page, off]
    return ref.dsv4_unpack_rows(rows, d, rd, dtype) if cache.dtype == torch.uint8 else rows


class Compressor(nn.Module):
    """Pools the layer's input over blocks of `ratio` tokens into extra key / value rows."""

    def __init__(self, cfg: ModelConfig, ratio: int, dtype, device):
        super().__init__()
        self.ratio, self.d, self.rd = ratio, cfg.head_dim, cfg.qk_rope_head_dim
        self.c = 2 if ratio == 4 else 1
        w = self.c * self.d
        self.ape = nn.Parameter(torch.zeros(ratio, w, dtype=torch.float32, device=device), requires_grad=False)
        self.wkv_gate = nn.Parameter(torch.zeros(2 * w, cfg.hidden_size, dtype=torch.float32, device=device), requires_grad=False)  # [wkv ; wgate]
        self.norm = RMSNorm(self.d, cfg.rms_norm_eps, dtype, device)

    def _finish(self, pooled: torch.Tensor, block_pos: torch.Tensor, rope_cache, dtype) -> torch.Tensor:
        rows = self.norm(pooled.to(dtype).contiguous())
        rotate_tail(rows, block_pos, rope_cache, self.rd)
        rows[:, : -self.rd] = ref.fp8_qdq_pow2(rows[:, : -self.rd], 64)
        return rows

    def forward(self, x: torch.Tensor, positions: torch.Tensor, ctx: ForwardContext, layer_idx: int, rope_cache) -> None:
        r, d, w = self.ratio, self.d, self.c * self.d
        cache = ctx.comp_caches[layer_idx]                     # [blocks, entries_per_page, d]
        ks_all, ss_all = ctx.comp_kv_states[layer_idx], ctx.comp_score_states[layer_idx]
        bs = ctx.kv_caches[layer_idx].shape[1]
        epp = cache.shape[1]
        proj = x.float() @ self.wkv_gate.t()
        kv, score = proj[:, :w], proj[:, w:] + self.ape[positions.long() % r]
        bt = ctx.block_tables.long()
        if not ctx.is_prefill and ctx.q_len_uniform == 1:
            # one token per sequence: a batched pass; sequences that do not finish a block write their row to the spare page
            slots = ctx.state_slots.long()
            pooled, done = ref.dsv4_compress_decode(kv, score, ks_all, ss_all, slots, positions, r, d)
            start = (positions.long() + 1 - r).clamp_min(0)
            rows = self._finish(pooled, start, rope_cache, x.dtype)
            page = torch.where(done, bt.gather(1, (start // bs).unsqueeze(1)).squeeze(1), torch.full_like(start, cache.shape[0] - 1))
            cache_store(cache, page, torch.where(done, (start % bs) // r, torch.zeros_like(start)).clamp_max(epp - 1), rows, self.rd)
            return
        cu, cl = ctx.cu_seqlens_q_host, ctx.context_lens_host
        slots_h, fresh_h = ctx.extras["state_slots_host"], ctx.extras["fresh_host"]
        for i in range(ctx.num_seqs):
            qs, qe = cu[i], cu[i + 1]
            pos0 = cl[i] - (qe - qs)
            ks, ss = ks_all[slots_h[i]], ss_all[slots_h[i]]
            if fresh_h[i]:
                ks.zero_(); ss.fill_(float("-inf"))
            pooled = ref.dsv4_compress_extend(kv[qs:qe], score[qs:qe], ks, ss, pos0, r, d)
            if pooled.shape[0]:
                start = (pos0 - pos0 % r) + r * torch.arange(pooled.shape[0], device=x.device)
                cache_store(cache, bt[i][start // bs], (start % bs) // r, self._finish(pooled, start, rope_cache, x.dtype), self.rd)


class V4Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        H, D = cfg.num_attention_heads, cfg.head_dim
        self.layer_idx, self.H, self.D, self.rd, self.window = layer_idx, H, D, cfg.qk_rope_head_dim, cfg.window_size
        self.G, self.R = cfg.o_groups, cfg.o_lora_rank
        self.eps, self.scale = cfg.rms_norm_eps, D ** -0.5
        q = cfg.quant if cfg.quant == "fp8" else None
        self.attn_sink = nn.Parameter(torch.zeros(H, dtype=torch.float32, device=device), requires_grad=False)
        self.wq_a = QLinear(cfg.hidden_size, cfg.q_lora_rank, dtype, device, q)
        self.q_norm = RMSNorm(cfg.q_lora_rank, cfg.rms_norm_eps, dtype, device)
        self.wq_b = QLinear(cfg.q_lora_rank, H * D, dtype, device, q)
        self.wkv = QLinear(cfg.hidden_size, D, dtype, device, q)
        self.kv_norm = RMSNorm(D, cfg.rms_norm_eps, dtype, device)
        self.wo_a = nn.Parameter(torch.zeros(self.G, self.R, H * D // self.G, dtype=dtype, device=device), requires_grad=False)
        self.wo_b = QLinear(self.G * self.R, cfg.hidden_size, dtype, device, q)
        self.ratio = cfg.compress_ratio(layer_idx)
        self.compressor = Compressor(cfg, self.ratio, dtype, device) if self.ratio else None

    # ---- candidates ---------------------------------------------------------------------------
    def _attend_decode(self, q, positions, ctx):
        """One query row per sequence: gather the window and the pooled rows of every sequence, one masked softmax."""
        cache = ctx.kv_caches[self.layer_idx]
        bs, W, r = cache.shape[1], self.window, self.ratio
        bt, pos = ctx.block_tables.long(), positions.long()
        widx = pos.unsqueeze(1) - (W - 1) + torch.arange(W, device=q.device)
        wmask = widx >= 0
        widx = widx.clamp_min(0)
        kv = cache_load(cache, bt.gather(1, widx // bs), widx % bs, self.D, self.rd, q.dtype)      # [B, W, D]
        mask = wmask
        if r:
            comp = ctx.comp_caches[self.layer_idx]
            n = max(ctx.context_lens_host) // r if ctx.context_lens_host else ctx.max_seqlen_k // r
            if n:
                b = torch.arange(n, device=q.device).unsqueeze(0).expand(q.shape[0], n)
                cmask = b < ((pos + 1) // r).unsqueeze(1)
                tok = torch.where(cmask, b * r, torch.zeros_like(b))
                kv = torch.cat([kv, cache_load(comp, bt.gather(1, tok // bs), (tok % bs) // r, self.D, self.rd, q.dtype)], 1)
                mask = torch.cat([mask, cmask], 1)
        return ref.sink_attention(q, kv, mask, self.attn_sink, self.scale)

    def _attend_varlen(self, q, ctx):
        cache = ctx.kv_caches[self.layer_idx]
        bs, W, r = cache.shape[1], self.window, self.ratio
        cu, cl = ctx.cu_seqlens_q_host, ctx.context_lens_host
        out = torch.empty_like(q)
        for i in range(ctx.num_seqs):
            qs, qe = cu[i], cu[i + 1]
            n_ctx, pos0 = cl[i], cl[i] - (qe - qs)
            bt = ctx.block_tables[i].long()
            comp = None
            if r and n_ctx // r:
                tok = torch.arange(n_ctx // r, device=q.device) * r
                comp = cache_load(ctx.comp_caches[self.layer_idx], bt[tok // bs], (tok % bs) // r, self.D, self.rd, q.dtype)
            for t0 in range(0, qe - qs, QUERY_TILE):
                t1 = min(qe - qs, t0 + QUERY_TILE)
                qpos = pos0 + torch.arange(t0, t1, device=q.device)
                kpos = torch.arange(max(0, pos0 + t0 - W + 1), pos0 + t1, device=q.device)
                kv = cache_load(cache, bt[kpos // bs], kpos % bs, self.D, self.rd, q.dtype)
                mask = (kpos.unsqueeze(0) <= qpos.unsqueeze(1)) & (kpos.unsqueeze(0) > qpos.unsqueeze(1) - W)
                if comp is not None:
                    kv = torch.cat([kv, comp], 0)
                    mask = torch.cat([mask, torch.arange(comp.shape[0], device=q.device).unsqueeze(0) < ((qpos + 1) // r).unsqueeze(1)], 1)
                out[qs + t0: qs + t1] = ref.sink_attention(q[qs + t0: qs + t1], kv, mask, self.attn_sink, self.scale)
        return out

    def forward(self, x, positions, ctx: ForwardContext, rope_cache):
        T, H, D, rd = ops.dense(x).shape[0], self.H, self.D, self.rd
        kv = self.kv_norm(self.wkv(x)).contiguous()
        rotate_tail(kv, positions, rope_cache, rd)
        kv[:, :-rd] = ref.fp8_qdq_pow2(kv[:, :-rd], 64)
        q = self.wq_b(self.q_norm(self.wq_a(x))).view(T, H, D)
        qf = q.float()
        q = (qf * torch.rsqrt(qf.square().mean(-1, keepdim=True) + self.eps)).to(q.dtype)
        rotate_tail(q, positions, rope_cache, rd)
        cache = ctx.kv_caches[self.layer_idx]
        slot, bs = ctx.slot_mapping.long(), cache.shape[1]
        cache_store(cache, slot // bs, slot % bs, kv, rd)
        if self.compressor is not None:
            self.compressor(ops.dense(x), positions, ctx, self.layer_idx, rope_cache)
        o = self._attend_decode(q, positions, ctx) if (not ctx.is_prefill and ctx.q_len_uniform == 1) else self._attend_varlen(q, ctx)
        rotate_tail(o, positions, rope_cache, rd, inverse=True)
        o = torch.einsum("tgd,grd->tgr", o.reshape(T, self.G, -1), self.wo_a)
        return self.wo_b(o.reshape(T, self.G * self.R))


class V4Gate(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.hash = layer_idx < cfg.num_hash_layers
        self.weight = nn.Parameter(torch.zeros(cfg.n_routed_experts, cfg.hidden_size, dtype=torch.float32, device=device), requires_grad=False)
        self.e_score_correction_bias = self.tid2eid = None
        if self.hash:
            self.tid2eid = nn.Parameter(torch.zeros(cfg.vocab_size, cfg.num_experts_per_tok, dtype=torch.int32, device=device), requires_grad=False)
        else:
            self.e_score_correction_bias = nn.Parameter(torch.zeros(cfg.n_routed_experts, dtype=torch.float32, device=device), requires_grad=False)

    def forward(self, x, input_ids):
        c = self.cfg
        logits = ops.router_logits(x, self.weight)
        norm = c.scoring_func != "softmax"
        if not self.hash:
            from ..parallel.ep import routing_options
            return ops.moe_route(logits, self.e_score_correction_bias, c.num_experts_per_tok, 1, 1, norm, c.routed_scaling_factor, c.scoring_func,
                                 **routing_options(self.layer_idx, x.device))
        lf = logits.float().sum(0) if logits.dim() == 3 else logits.float()
        s = (torch.nn.functional.softplus(lf).sqrt() if c.scoring_func == "sqrtsoftplus" else lf.sigmoid() if c.scoring_func == "sigmoid"
             else lf.softmax(-1))
        idx = self.tid2eid[input_ids.long()].long()
        w = s.gather(1, idx)
        if norm:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return idx.to(torch.int32), (w * c.routed_scaling_factor).float()


class V4MoE(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.gate = V4Gate(cfg, layer_idx, device)
        self.experts = RoutedExperts(cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size, dtype, device, cfg.quant, layer_idx,
                                     act=cfg.glu_act)
        # the always-on expert is a plain SwiGLU: the clamp applies to the routed experts only
        self.shared_experts = SwiGLUMLP(cfg.hidden_size, cfg.moe_intermediate_size * max(1, cfg.n_shared_experts), dtype, device,
                                        cfg.quant if cfg.quant == "fp8" else None)

    def forward(self, xq, ctx: ForwardContext):
        from ..parallel.ep import ep_moe_forward
        x = ops.dense(xq)
        idx, w = self.gate(x, ctx.extras["input_ids"])
        return ep_moe_forward(self.experts, x, idx, w, ctx, add_in=self.shared_experts(xq))


class V4DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        fp8 = cfg.quant == "fp8"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8)
        self.self_attn = V4Attention(cfg, layer_idx, dtype, device)
        self.mlp = V4MoE(cfg, layer_idx, dtype, device)
        self.hc_attn = HyperConnection(cfg, device)
        self.hc_ffn = HyperConnection(cfg, device)

    def forward(self, streams, positions, ctx, ropes):
        x, post, comb = self.hc_attn(streams)
        a = self.self_attn(self.input_layernorm(x), positions, ctx, ropes[1 if self.self_attn.ratio else 0])
        streams = ops.mhc_post(a, streams, post, comb)
        x, post, comb = self.hc_ffn(streams)
        m = self.mlp(self.post_attention_layernorm(x), ctx)
        return ops.mhc_post(m, streams, post, comb)


class HCHead(nn.Module):
    """Contracts the streams in front of the final norm: y = sum_i (sigmoid(mix_i * scale + base_i) + eps) x_i with
    mix = fn (x flattened) * rsqrt(mean x^2 + eps)."""

    def __init__(self, cfg: ModelConfig, device):
        super().__init__()
        h = cfg.hc_mult
        self.eps = cfg.hc_eps
        self.fn = nn.Parameter(torch.zeros(h, h * cfg.hidden_size, dtype=torch.float32, device=device), requires_grad=False)
        self.base = nn.Parameter(torch.zeros(h, dtype=torch.float32, device=device), requires_grad=False)
        self.scale = nn.Parameter(torch.ones(1, dtype=torch.float32, device=device), requires_grad=False)

    def forward(self, streams):
        flat = streams.flatten(1).float()
        mix = (flat @ self.fn.t()) * torch.rsqrt(flat.square().mean(-1, keepdim=True) + self.eps)
        pre = torch.sigmoid(mix * self.scale + self.base) + self.eps
        return (pre.unsqueeze(-1) * streams.float()).sum(1).to(streams.dtype)


class _Inner(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleDict({str(i): V4DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)})
        self.hc_head = HCHead(cfg, device)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class DeepseekV4ForCausalLM(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", layer_range=None):
        super().__init__()
        assert layer_range is None, "pipeline stages are not offered for DeepSeek-V4"
        assert get_dist_context().attn_tp_size == 1, "DeepSeek-V4 runs with attention_tp = 1"
        assert 1 <= cfg.hc_mult <= 4 and (cfg.head_dim - cfg.qk_rope_head_dim) % 64 == 0 and (cfg.num_attention_heads * cfg.head_dim) % cfg.o_groups == 0
        self.cfg, self.dtype = cfg, dtype
        self.model = _Inner(cfg, dtype, device)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        # window-only layers rotate with the plain base; compressing layers with their own base under YaRN interpolation
        # without the magnitude factor
        rd = cfg.qk_rope_head_dim
        scaling = dict(cfg.rope_scaling, mscale=0.0, mscale_all_dim=0.0) if cfg.rope_scaling else None
        self.register_buffer("rope_window", ref.rope_cos_sin_cache(rd, cfg.max_position_embeddings, cfg.rope_theta, None).to(device), persistent=False)
        self.register_buffer("rope_compress", ref.rope_cos_sin_cache(rd, cfg.max_position_embeddings, cfg.compress_rope_theta or cfg.rope_theta,
                                                                     scaling).to(device), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def num_cache_layers(self) -> int:
        return self.cfg.num_hidden_layers

    def forward(self, input_ids, positions, ctx: ForwardContext, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else self.model.embed_tokens(input_ids)
        ctx.extras.setdefault("input_ids", input_ids)
        streams = h.unsqueeze(1).expand(-1, self.cfg.hc_mult, -1).contiguous()
        ropes = (self.rope_window, self.rope_compress)
        for i in range(self.cfg.num_hidden_layers):
            streams = self.model.layers[str(i)](streams, positions, ctx, ropes)
        return self.model.norm(self.model.hc_head(streams))

    def compute_logits(self, hidden):
        return ops.lm_head(hidden, self.lm_head.weight)

    # ---- weights ---------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        """Tensors under the release's own names: `embed`, `head`, `norm`, `hc_head_{fn,base,scale}`, `layers.N.{attn_norm,ffn_norm}`,
        `layers.N.hc_{attn,ffn}_{fn,base,scale}`, `layers.N.attn.{wq_a,q_norm,wq_b,wkv,kv_norm,wo_a,wo_b,attn_sink}`,
        `layers.N.attn.compressor.{ape,wkv,wgate,norm}`, `layers.N.ffn.gate.{weight,bias,tid2eid}`,
        `layers.N.ffn.{experts.E,shared_experts}.{w1,w2,w3}`; fp8 tensors come with `.scale` (128 x 128 blocks), 4-bit experts as
        int8 nibble pairs with one e8m0 `.scale` per 32 values.  `.attn.indexer.*` tensors are not used."""
        from .weights import load_deepseek_weights
        cfg = self.cfg
        n = 0
        fp8 = torch.float8_e4m3fn
        layer_re = re.compile(r"layers\.(\d+)\.(.+)$")
        proj = {"w1": "gate_proj", "w2": "down_proj", "w3": "up_proj"}
        pend = {}          # tensors waiting for their scale (or the other way round)

        def f32(t):
            return t.float() if t.dtype != torch.float32 else t

        def pair(key, kind, t):
            g = pend.setdefault(key, {})
            g[kind] = t
            return g if len(g) == 2 else None

        def set_linear(lin, key, leaf_kind, t):
            """weight / scale of a QLinear: an fp8 weight waits for its scale."""
            nonlocal n
            if leaf_kind == "weight" and t.dtype != fp8:
                lin.set_weight(t); n += 1; return
            g = pair(key, leaf_kind, t)
            if g:
                lin.set_weight(g["weight"], f32(g["scale"])); pend.pop(key); n += 2

        def rest():
            nonlocal n
            for name, t in weights:
                if name in ("embed.weight", "head.weight", "norm.weight"):
                    yield {"embed.weight": "model.embed_tokens.weight", "head.weight": "lm_head.weight", "norm.weight": "model.norm.weight"}[name], t
                    continue
                if name.startswith("hc_head_"):
                    getattr(self.model.hc_head, name[len("hc_head_"):]).copy_(f32(t).reshape(getattr(self.model.hc_head, name[len("hc_head_"):]).shape)); n += 1
                    continue
                m = layer_re.match(name)
                if not m or int(m.group(1)) >= cfg.num_hidden_layers:
                    continue
                li, leaf = m.group(1), m.group(2)
                L = self.model.layers[li]
                if leaf in ("attn_norm.weight", "ffn_norm.weight"):
                    yield f"model.layers.{li}.{'input_layernorm' if leaf[0] == 'a' else 'post_attention_layernorm'}.weight", t
                    continue
                h = re.match(r"(hc_attn|hc_ffn)_(fn|base|scale)$", leaf)
                if h:
                    p = getattr(getattr(L, h.group(1)), h.group(2))
                    p.copy_(f32(t).reshape(p.shape)); n += 1
                    continue
                if leaf.startswith("attn."):
                    A, a = L.self_attn, leaf[len("attn."):]
                    if a.startswith("indexer."):
                        continue
                    if a == "attn_sink":
                        A.attn_sink.copy_(f32(t)); n += 1
                    elif a in ("q_norm.weight", "kv_norm.weight"):
                        getattr(A, a[:-7]).weight.copy_(t.to(self.dtype)); n += 1
                    elif a.startswith("compressor.") and A.compressor is not None:
                        C, c = A.compressor, a[len("compressor."):]
                        w = C.c * C.d
                        if c == "ape":
                            C.ape.copy_(f32(t)); n += 1
                        elif c == "norm.weight":
                            C.norm.weight.copy_(t.to(self.dtype)); n += 1
                        elif c == "wkv.weight":
                            C.wkv_gate[:w].copy_(f32(t)); n += 1
                        elif c == "wgate.weight":
                            C.wkv_gate[w:].copy_(f32(t)); n += 1
                    elif a.split(".")[0] in ("wq_a", "wq_b", "wkv", "wo_b"):
                        set_linear(getattr(A, a.split(".")[0]), f"{li}.{a.split('.')[0]}", a.split(".")[1], t)
                    elif a.startswith("wo_a."):
                        if a == "wo_a.weight" and t.dtype != fp8:
                            A.wo_a.copy_(t.to(self.dtype).view(A.wo_a.shape)); n += 1
                        else:
                            g = pair(f"{li}.wo_a", a.split(".")[1], t)
                            if g:
                                A.wo_a.copy_(ref.dequant_fp8_block(g["weight"], f32(g["scale"])).to(self.dtype).view(A.wo_a.shape)); pend.pop(f"{li}.wo_a"); n += 2
                    continue
                if leaf.startswith("ffn."):
                    f = leaf[len("ffn."):]
                    G = L.mlp.gate
                    if f == "gate.weight":
                        G.weight.copy_(f32(t)); n += 1
                    elif f == "gate.bias":
                        if G.e_score_correction_bias is not None:
                            G.e_score_correction_bias.copy_(f32(t)); n += 1
                    elif f == "gate.tid2eid":
                        if G.tid2eid is not None:
                            G.tid2eid.copy_(t.to(torch.int32)); n += 1
                    else:
                        e = re.match(r"(experts\.\d+|shared_experts)\.(w[123])\.(weight|scale)$", f)
                        if not e:
                            continue
                        base = f"model.layers.{li}.mlp.{e.group(1)}.{proj[e.group(2)]}"
                        if e.group(1) != "shared_experts" and (t.dtype == torch.int8 or base in pend or (e.group(3) == "scale" and t.dim() == 2 and t.shape[0] > 128)):
                            # packed 4-bit expert: expanded here, then quantised (or kept) as the engine's expert format asks
                            g = pair(base, "weight" if e.group(3) == "weight" else "scale", t)
                            if g:
                                sc = g["scale"]
                                if sc.element_size() == 1:          # e8m0 bytes under any one-byte dtype
                                    sc = sc.view(torch.uint8)
                                else:                               # scales expanded to floats: back to their exponent bytes
                                    sc = (torch.log2(sc.float()).round() + 127).to(torch.uint8)
                                yield base + ".weight", ref.mxfp4_dequant(g["weight"].view(torch.uint8), sc)
                                pend.pop(base)
                            continue
                        yield base + (".weight" if e.group(3) == "weight" else ".weight_scale_inv"), (t if e.group(3) == "weight" else f32(t))

        with torch.no_grad():
            n += load_deepseek_weights(self, rest())
        if pend:
            raise ValueError(f"incomplete checkpoint: tensors without their partner {list(pend)[:4]}")
        for i in range(cfg.num_hidden_layers):
            L = self.model.layers[str(i)]
            L.hc_attn.refresh(); L.hc_ffn.refresh()
        return n


def dsv4_param_shapes(cfg: ModelConfig, out: dict) -> dict:
    """Every tensor of a high-precision checkpoint of this family under the release's names."""
    H, V, D, hc = cfg.hidden_size, cfg.vocab_size, cfg.head_dim, cfg.hc_mult
    out.clear()
    out.update({"embed.weight": (V, H), "head.weight": (V, H), "norm.weight": (H,), "hc_head_fn": (hc, hc * H), "hc_head_base": (hc,),
                "hc_head_scale": (1,)})
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        out[p + "attn_norm.weight"] = (H,)
        out[p + "ffn_norm.weight"] = (H,)
        for site in ("hc_attn", "hc_ffn"):
            out[p + site + "_fn"] = ((2 + hc) * hc, hc * H)
            out[p + site + "_base"] = ((2 + hc) * hc,)
            out[p + site + "_scale"] = (3,)
        a = p + "attn."
        out[a + "attn_sink"] = (cfg.num_attention_heads,)
        out[a + "wq_a.weight"] = (cfg.q_lora_rank, H)
        out[a + "q_norm.weight"] = (cfg.q_lora_rank,)
        out[a + "wq_b.weight"] = (cfg.num_attention_heads * D, cfg.q_lora_rank)
        out[a + "wkv.weight"] = (D, H)
        out[a + "kv_norm.weight"] = (D,)
        out[a + "wo_a.weight"] = (cfg.o_groups * cfg.o_lora_rank, cfg.num_attention_heads * D // cfg.o_groups)
        out[a + "wo_b.weight"] = (H, cfg.o_groups * cfg.o_lora_rank)
        r = cfg.compress_ratio(i)
        if r:
            w = (2 if r == 4 else 1) * D
            out[a + "compressor.ape"] = (r, w)
            out[a + "compressor.wkv.weight"] = (w, H)
            out[a + "compressor.wgate.weight"] = (w, H)
            out[a + "compressor.norm.weight"] = (D,)
        f = p + "ffn."
        out[f + "gate.weight"] = (cfg.n_routed_experts, H)
        if i < cfg.num_hash_layers:
            out[f + "gate.tid2eid"] = (V, cfg.num_experts_per_tok)
        else:
            out[f + "gate.bias"] = (cfg.n_routed_experts,)
        I = cfg.moe_intermediate_size
        for e in [f"experts.{j}" for j in range(cfg.n_routed_experts)] + ["shared_experts"]:
            Ie = I * max(1, cfg.n_shared_experts) if e == "shared_experts" else I
            out[f + e + ".w1.weight"] = (Ie, H)
            out[f + e + ".w3.weight"] = (Ie, H)
            out[f + e + ".w2.weight"] = (H, Ie)
    return out
