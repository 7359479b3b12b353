"""GLM5-next family: Kimi-delta-attention layers between DeepSeek sparse-attention (MLA + lightning indexer) layers, a
hidden state of `hc_mult` parallel streams mixed by manifold-constrained hyper-connections, and DeepSeek-style MoE with a
clamped SwiGLU.

Parity: reference runtime/models/glm5_next/glm5_next.py - hyper-connection projector :27-70, stream contraction at the
head :73-94, post-mix :96-97, decoder layer :100-152, model :155-192, checkpoint name normalisation :205-245.

B200-first differences: the pre-mix (coefficient product, sigmoid / softmax / Sinkhorn, stream contraction) is one CUDA
kernel that reads the streams once, the post-mix another; the attention and expert layers are the DeepSeek ones of this
package, the linear layers share the delta-rule kernels of the gated delta-net family.
"""
from __future__ import annotations

import re
from typing import Iterable, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..parallel.dist import get_dist_context
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .deepseek import DeepseekMoE, MLAAttention
from .kda import KimiDeltaAttention
from .layers import RMSNorm, SwiGLUMLP


class HyperConnection(nn.Module):
    """Coefficients of one hyper-connection site: fn [(2+h)h, h*D], base [(2+h)h], scale [3], all fp32."""

    def __init__(self, cfg: ModelConfig, device):
        super().__init__()
        h, D = cfg.hc_mult, cfg.hidden_size
        self.h, self.iters, self.eps = h, cfg.hc_sinkhorn_iters, cfg.hc_eps
        self.fn = nn.Parameter(torch.zeros((2 + h) * h, h * D, dtype=torch.float32, device=device), requires_grad=False)
        self.base = nn.Parameter(torch.zeros((2 + h) * h, dtype=torch.float32, device=device), requires_grad=False)
        self.scale = nn.Parameter(torch.ones(3, dtype=torch.float32, device=device), requires_grad=False)
        self._split = None          # bf16 head / remainder split of `fn` for the tensor-core product; rebuilt after a weight change

    def refresh(self):
        self._split = None

    def forward(self, streams):
        if streams.is_cuda and self._split is None:
            self._split = ops.mhc_split_weights(self.fn)
        return ops.mhc_pre(streams, self.fn, self.base, self.scale, self.iters, self.eps, self._split)


class Glm5NextDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        self.kind = cfg.layer_type(layer_idx)
        fp8 = cfg.quant == "fp8"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8 and self.kind != "linear_attention")
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, quant_out=fp8)
        if self.kind == "linear_attention":
            self.linear_attn = KimiDeltaAttention(cfg, cfg.num_layers_of("linear_attention", layer_idx), dtype, device)
        else:
            self.self_attn = MLAAttention(cfg, layer_idx, dtype, device, cache_idx=cfg.num_layers_of("full_attention", layer_idx))
        self.is_moe = cfg.is_moe_layer(layer_idx)
        self.mlp = (DeepseekMoE(cfg, dtype, device, layer_idx) if self.is_moe
                    else SwiGLUMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device, cfg.quant, act=cfg.glu_act))
        self.hc_attn = HyperConnection(cfg, device)
        self.hc_ffn = HyperConnection(cfg, device)

    def forward(self, streams, positions, ctx, rope_cache):
        x, post, comb = self.hc_attn(streams)
        x = self.input_layernorm(x)
        a = self.linear_attn(x, ctx) if self.kind == "linear_attention" else self.self_attn(x, positions, ctx, rope_cache)
        streams = ops.mhc_post(a, streams, post, comb)
        x, post, comb = self.hc_ffn(streams)
        x = self.post_attention_layernorm(x)
        m = self.mlp(x, ctx) if self.is_moe else self.mlp(x)
        return ops.mhc_post(m, streams, post, comb)


class _Inner(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleDict({str(i): Glm5NextDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)})
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class Glm5NextForConditionalGeneration(nn.Module):
    """Text stack of the GLM5-next checkpoints (vision towers are skipped by the loader)."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", layer_range=None):
        super().__init__()
        assert layer_range is None, "pipeline stages are not offered for the hyper-connection family"
        assert get_dist_context().attn_tp_size == 1, "the hyper-connection family runs with attention_tp = 1"
        assert 1 <= cfg.hc_mult <= 4, "hc_mult must be 1..4"
        self.cfg, self.dtype = cfg, dtype
        self.model = _Inner(cfg, dtype, device)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        rc = ref.rope_cos_sin_cache(cfg.qk_rope_head_dim, cfg.max_position_embeddings, cfg.rope_theta, cfg.rope_scaling)
        self.register_buffer("rope_cache", rc.to(device), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)

    @property
    def num_cache_layers(self) -> int:
        return self.cfg.num_layers_of("full_attention")

    def forward(self, input_ids, positions, ctx: ForwardContext, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else self.model.embed_tokens(input_ids)
        streams = h.unsqueeze(1).expand(-1, self.cfg.hc_mult, -1).contiguous()
        for i in range(self.cfg.num_hidden_layers):
            streams = self.model.layers[str(i)](streams, positions, ctx, self.rope_cache)
        # the streams are contracted by a plain mean in front of the final norm
        return self.model.norm(streams.float().mean(1).to(streams.dtype))

    def compute_logits(self, hidden):
        return ops.lm_head(hidden, self.lm_head.weight)

    # ---- weights ---------------------------------------------------------------------------
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        from .weights import load_deepseek_weights
        cfg = self.cfg
        n = 0
        hc_re = re.compile(r"model\.layers\.(\d+)\.(hc_attn|hc_ffn)[._](fn|base|scale)$")
        attn_re = re.compile(r"model\.layers\.(\d+)\.self_attn\.(.+)$")

        def rest():
            nonlocal n
            for name, t in weights:
                for pre in ("model.language_model.", "language_model.model.", "language_model."):
                    if name.startswith(pre):
                        name = "model." + name[len(pre):]
                        break
                m = hc_re.match(name)
                if m and int(m.group(1)) < cfg.num_hidden_layers:
                    getattr(getattr(self.model.layers[m.group(1)], m.group(2)), m.group(3)).copy_(t.float().reshape(-1) if m.group(3) != "fn" else t.float())
                    n += 1
                    continue
                m = attn_re.match(name)
                if m and int(m.group(1)) < cfg.num_hidden_layers and cfg.layer_type(int(m.group(1))) == "linear_attention":
                    if self.model.layers[m.group(1)].linear_attn.load(m.group(2), t):
                        n += 1
                    continue
                yield name, t

        with torch.no_grad():
            n += load_deepseek_weights(self, rest())
        for i in range(cfg.num_hidden_layers):
            L = self.model.layers[str(i)]
            L.hc_attn.refresh(); L.hc_ffn.refresh()
            if L.kind == "linear_attention" and L.linear_attn.pending():
                raise ValueError(f"incomplete checkpoint: layer {i} delta-attention parts {L.linear_attn.pending()}")
        return n
