"""Kimi delta attention (KDA): the linear-attention layer of the GLM5-next and Kimi-K3 families.

A delta-rule recurrence per head whose state [Dv, Dk] decays with a learned gate PER KEY CHANNEL, fed by short causal
convolutions of the q / k / v projections and read out through a sigmoid-gated RMSNorm.

Parity: reference layers/backends/delta_net/kda.py:27-377 (projections :71-160, decode :258-290, recurrence :300-370),
kernel/triton/fla/fused_recurrent.py:440-545 (one decode step), kernel/triton/generic/k3_output_norm.py.

B200-first differences: [q | k | v | output gate] is one GEMM for prefill and decode alike, and so is [forget-gate
bottleneck | beta]; the convolution and the recurrence are the same two CUDA kernels the gated delta-net layers use (the
recurrence keeps the 128 x 128 state of a head in registers across all tokens of a sequence and takes the per-channel
gate as a template variant), followed by the gated norm kernel.  The layer keeps its projections in the activation dtype
(the checkpoints ship them unquantised).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..parallel.dist import get_dist_context
from ..runtime.context import ForwardContext
from .config import ModelConfig
from .layers import QLinear


class KimiDeltaAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, state_idx: int, dtype, device):
        super().__init__()
        assert get_dist_context().attn_tp_size == 1, "delta-attention layers run with attention_tp = 1"
        self.state_idx = state_idx
        self.h = cfg.linear_num_value_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.h * self.dk, self.h * self.dv
        self.conv_dim, self.conv_k = cfg.gdn_conv_dim, cfg.linear_conv_kernel_dim
        self.lower_bound = cfg.kda_gate_lower_bound
        self.eps = cfg.rms_norm_eps
        H = cfg.hidden_size
        self.qkvg_proj = QLinear(H, self.conv_dim + self.value_dim, dtype, device, None)       # [q | k | v | output gate]
        # [forget-gate bottleneck | beta logits], rows padded to a multiple of 16 (the GEMM wants N % 8 == 0)
        self.fab_rows = (self.dk + self.h + 15) // 16 * 16
        self.fa_b_proj = QLinear(H, self.fab_rows, dtype, device, None)
        self.f_b_proj = QLinear(self.dk, self.key_dim, dtype, device, None)
        self.o_proj = QLinear(self.value_dim, H, dtype, device, None)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_dim, self.conv_k, dtype=dtype, device=device), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.h, dtype=torch.float32, device=device), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(self.key_dim, dtype=torch.float32, device=device), requires_grad=False)
        self.o_norm_weight = nn.Parameter(torch.ones(self.dv, dtype=dtype, device=device), requires_grad=False)
        self._parts = {}

    def forward(self, x, ctx: ForwardContext):
        T = x.shape[0]
        proj = self.qkvg_proj(x)
        ab = self.fa_b_proj(x)
        raw_g = self.f_b_proj(ab[:, : self.dk].contiguous())                                   # [T, H * Dk]
        qkv, gate = proj[:, : self.conv_dim], proj[:, self.conv_dim:]
        uniform_one = (not ctx.is_prefill) and ctx.q_len_uniform == 1
        y = ops.gdn_conv(qkv, self.conv_weight, ctx.conv_states[self.state_idx], ctx.state_slots, ctx.cu_seqlens_q, ctx.seq_fresh, uniform_one)
        q = y[:, : self.key_dim].view(T, self.h, self.dk)
        k = y[:, self.key_dim: 2 * self.key_dim].view(T, self.h, self.dk)
        v = y[:, 2 * self.key_dim:].view(T, self.h, self.dv)
        o = ops.kda_recurrent(q, k, v, raw_g, ab[:, self.dk: self.dk + self.h], self.A_log, self.dt_bias, self.lower_bound, ctx.rec_states[self.state_idx],
                              ctx.state_slots, ctx.cu_seqlens_q, ctx.seq_fresh, gate.view(T, self.h, self.dv), self.o_norm_weight, self.eps)
        return self.o_proj(o)

    # ---- weights ---------------------------------------------------------------------------
    @torch.no_grad()
    def load(self, leaf: str, w: torch.Tensor) -> bool:
        """One checkpoint tensor of this layer by its leaf name (`q_proj.weight`, `q_conv1d.weight`, `A_log`, ...).  Parts of the
        merged matrices are held until their group is complete.  Returns False for a name this layer does not know."""
        w = w.float()
        P = self._parts

        def group(key, part, order, setter):
            g = P.setdefault(key, {})
            g[part] = w
            if len(g) == len(order):
                setter(torch.cat([g[o] for o in order], 0))
                P.pop(key)
            return True

        name = leaf[:-len(".weight")] if leaf.endswith(".weight") else leaf
        if name in ("q_proj", "k_proj", "v_proj", "g_proj"):
            return group("qkvg", name, ("q_proj", "k_proj", "v_proj", "g_proj"), self.qkvg_proj.set_weight)
        if name in ("g_a_proj", "g_b_proj"):               # low-rank output gate of GLM5-next: merged into one matrix (b @ a)
            g = P.setdefault("g_lr", {})
            g[name] = w
            if len(g) == 2:
                self.load("g_proj.weight", g["g_b_proj"] @ g["g_a_proj"])
                P.pop("g_lr")
            return True
        if name in ("f_a_proj", "b_proj"):
            def set_fab(m):
                self.fa_b_proj.set_weight(torch.cat([m, m.new_zeros(self.fab_rows - m.shape[0], m.shape[1])], 0))
            return group("fab", name, ("f_a_proj", "b_proj"), set_fab)
        if name == "f_b_proj":
            self.f_b_proj.set_weight(w); return True
        if name == "o_proj":
            self.o_proj.set_weight(w); return True
        if name in ("q_conv1d", "k_conv1d", "v_conv1d"):
            return group("conv", name, ("q_conv1d", "k_conv1d", "v_conv1d"),
                         lambda m: self.conv_weight.copy_(m.reshape(self.conv_dim, self.conv_k).to(self.conv_weight.dtype)))
        if name == "conv1d":
            self.conv_weight.copy_(w.reshape(self.conv_dim, self.conv_k).to(self.conv_weight.dtype)); return True
        if name == "A_log":
            self.A_log.copy_(w.flatten()); return True
        if name == "dt_bias":
            self.dt_bias.copy_(w.flatten()); return True
        if name == "o_norm":
            self.o_norm_weight.copy_(w.to(self.o_norm_weight.dtype)); return True
        return False

    def pending(self):
        return list(self._parts)


def kda_param_shapes(cfg: ModelConfig, prefix: str, out: dict, low_rank_gate: Optional[int] = None) -> None:
    """Checkpoint tensor names and shapes of one KDA layer under `prefix` (`...self_attn.`)."""
    H, h, dk, dv, K = cfg.hidden_size, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.linear_conv_kernel_dim
    out[prefix + "q_proj.weight"] = (h * dk, H)
    out[prefix + "k_proj.weight"] = (h * dk, H)
    out[prefix + "v_proj.weight"] = (h * dv, H)
    if low_rank_gate:
        out[prefix + "g_a_proj.weight"] = (low_rank_gate, H)
        out[prefix + "g_b_proj.weight"] = (h * dv, low_rank_gate)
    else:
        out[prefix + "g_proj.weight"] = (h * dv, H)
    out[prefix + "b_proj.weight"] = (h, H)
    out[prefix + "f_a_proj.weight"] = (dk, H)
    out[prefix + "f_b_proj.weight"] = (h * dk, dk)
    out[prefix + "o_proj.weight"] = (H, h * dv)
    out[prefix + "q_conv1d.weight"] = (h * dk, 1, K)
    out[prefix + "k_conv1d.weight"] = (h * dk, 1, K)
    out[prefix + "v_conv1d.weight"] = (h * dv, 1, K)
    out[prefix + "A_log"] = (h,)
    out[prefix + "dt_bias"] = (h * dk,)
    out[prefix + "o_norm.weight"] = (dv,)
