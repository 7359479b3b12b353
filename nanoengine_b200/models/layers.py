"""Building blocks shared by the model families: quantisable linears, norms, SwiGLU MLP, routed experts.

Parity: reference runtime/layers/base_backend.py:91-211 (linear / experts factories),
layers/backends/linear/deep_gemm.py (fp8 block-scaled linears), layers/backends/experts/deep_gemm.py:138-175
(stacked expert weights ``gate_up_proj [E_local, 2I, H]``, ``down_proj [E_local, H, I]``, scales per 128x128
block), layers/layernorm.py:16-108, layers/activation.py:29-112.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from ..parallel.dist import get_dist_context


def _ceil_div(a, b):
    return (a + b - 1) // b


class QLinear(nn.Module):
    """y = x W^T with W [out, in] in the activation dtype or in fp8 e4m3 with 128x128 block scales."""

    def __init__(self, in_features: int, out_features: int, dtype, device, quant: Optional[str] = None, bias: bool = False):
        super().__init__()
        self.in_features, self.out_features, self.quant = in_features, out_features, quant
        if quant == "fp8":
            self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=torch.float8_e4m3fn, device=device), requires_grad=False)
            self.weight_scale_inv = nn.Parameter(torch.ones(_ceil_div(out_features, 128), _ceil_div(in_features, 128),
                                                            dtype=torch.float32, device=device), requires_grad=False)
        else:
            # the tensor-core GEMM wants a multiple of 8 output columns: a narrower projection keeps zero rows below its own
            rows = _ceil_div(out_features, 8) * 8 if not bias else out_features
            self.weight = nn.Parameter((torch.zeros if rows != out_features else torch.empty)(rows, in_features, dtype=dtype, device=device),
                                       requires_grad=False)
            self.weight_scale_inv = None
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device), requires_grad=False) if bias else None

    def forward(self, x):
        y = ops.linear(x, self.weight, self.weight_scale_inv, self.bias)
        return y if y.shape[-1] == self.out_features else y[..., : self.out_features]

    @torch.no_grad()
    def init_random(self, gen: torch.Generator, std: float = 0.02):
        w = torch.empty(self.out_features, self.in_features, dtype=torch.float32, device=self.weight.device)
        w.normal_(0.0, std, generator=gen)
        self.set_weight(w)

    @torch.no_grad()
    def set_weight(self, w: torch.Tensor, scale_inv: Optional[torch.Tensor] = None):
        """Accepts a high-precision weight (quantised here if needed) or an fp8 weight with its scales."""
        if self.quant == "fp8":
            if w.dtype == torch.float8_e4m3fn:
                w, scale_inv = ref.fp8_block_for_format(w.to(self.weight.device), scale_inv.to(self.weight.device))
                self.weight.copy_(w)
                self.weight_scale_inv.copy_(scale_inv)
            else:
                q, s = ref.quant_fp8_block(w.to(self.weight.device))
                self.weight.copy_(q)
                self.weight_scale_inv.copy_(s)
        else:
            if w.dtype == torch.float8_e4m3fn:
                w = ref.dequant_fp8_block(w, scale_inv)
            self.weight[: self.out_features].copy_(w.to(self.weight.dtype))


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype, device, quant_out: bool = False, unit_offset: bool = False):
        super().__init__()
        self.unit_offset = unit_offset  # stored weight is the deviation from one; the kernels apply (1 + w) in fp32
        self.weight = nn.Parameter((torch.zeros if unit_offset else torch.ones)(dim, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps
        self.quant_out = quant_out      # the consumers include fp8 linears: the kernel also emits their quantised input (ops.QAct)

    def forward(self, x, residual=None):
        """Without residual: y.  With residual: (y, x + residual) - the fused add + norm used between blocks.  With
        `quant_out` y is an `ops.QAct`: hand it to QLinear as it is, take `ops.dense(y)` wherever rows are read."""
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps, self.quant_out, self.unit_offset)
        return ops.add_rmsnorm(x, residual, self.weight, self.eps, self.unit_offset, self.quant_out)


class SwiGLUMLP(nn.Module):
    """Dense SwiGLU MLP with gate and up projections merged into one GEMM."""

    def __init__(self, hidden: int, inter: int, dtype, device, quant=None, act=None):
        super().__init__()
        self.gate_up_proj = QLinear(hidden, 2 * inter, dtype, device, quant)
        self.down_proj = QLinear(inter, hidden, dtype, device, quant)
        self.act = act          # gated activation other than SwiGLU: see ops.reference.glu_act

    def forward(self, x):
        return self.down_proj(ops.silu_and_mul(self.gate_up_proj(x), self.down_proj.quant == "fp8", act=self.act))

    def init_random(self, gen):
        self.gate_up_proj.init_random(gen)
        self.down_proj.init_random(gen)


class TPSwiGLUMLP(nn.Module):
    """Dense gated MLP sharded over the tensor-parallel group: gate / up column-parallel, down row-parallel.  Takes this
    rank's slice of the tokens and returns its slice of the result: all-gather -> GEMM and GEMM -> reduce-scatter, each one
    fused kernel pair on GPUs with peer access.
    Parity: reference layers/backends/linear (column / row parallel linears on `ffn_tp_group`), models/kimi_k3/kimi_k3.py:34-70."""

    def __init__(self, hidden: int, inter: int, dtype, device, quant=None, act=None, axis: str = "attn_tp"):
        super().__init__()
        d = get_dist_context()
        self.tp, self.tp_rank, self.axis = d.ffn_tp_size, d.ffn_tp_rank, axis
        assert inter % self.tp == 0 and (quant != "fp8" or (inter // self.tp) % 128 == 0), "intermediate size must split over ffn_tp (in 128-wide blocks for fp8)"
        self.inter, self.inter_local = inter, inter // self.tp
        self.gate_up_proj = QLinear(hidden, 2 * self.inter_local, dtype, device, quant)
        self.down_proj = QLinear(self.inter_local, hidden, dtype, device, quant)
        self.act = act

    def forward(self, x_slice, total_rows: int):
        from ..parallel.tp import tp_all_gather_linear, tp_linear_reduce_scatter
        g = tp_all_gather_linear(ops.dense(x_slice), total_rows, self.gate_up_proj, self.axis)
        return tp_linear_reduce_scatter(ops.silu_and_mul(g, act=self.act), self.down_proj, self.axis)

    def shard_rows(self):
        """Row range of gate_proj / up_proj (and column range of down_proj) this rank holds."""
        return self.tp_rank * self.inter_local, (self.tp_rank + 1) * self.inter_local


class VocabParallelEmbedding(nn.Module):
    """Embedding table split by vocabulary rows over the tensor-parallel group: each rank looks up the ids it owns (zeros for
    the rest) and the partial rows are summed.  `forward_scatter` returns this rank's slice of the tokens directly
    (reduce-scatter), which is what the token-sliced residual stream wants.
    Parity: reference layers/embed_head.py:49-94."""

    def __init__(self, vocab: int, hidden: int, dtype, device, axis: str = "attn_tp"):
        super().__init__()
        d = get_dist_context()
        self.tp, self.rank, self.axis = d.attn_tp_size, d.attn_tp_rank, axis
        self.vocab = vocab
        self.per = -(-vocab // self.tp)
        self.lo = self.rank * self.per
        self.weight = nn.Parameter(torch.zeros(self.per, hidden, dtype=dtype, device=device), requires_grad=False)

    def _partial(self, ids):
        local = ids - self.lo
        ok = (local >= 0) & (local < self.per)
        rows = self.weight[local.clamp(0, self.per - 1)]
        return rows * ok.unsqueeze(-1).to(rows.dtype)

    def forward(self, ids):
        from ..parallel.tp import tp_all_reduce
        return tp_all_reduce(self._partial(ids), self.axis)

    def forward_scatter(self, ids):
        from ..parallel.tp import tp_reduce_scatter
        return tp_reduce_scatter(self._partial(ids), self.axis)

    @torch.no_grad()
    def load_full(self, w: torch.Tensor):
        part = w[self.lo: self.lo + self.per]
        self.weight.zero_()
        self.weight[: part.shape[0]].copy_(part.to(self.weight.dtype))


class ParallelLMHead(nn.Module):
    """Output projection split by vocabulary rows: every rank computes the logits of its rows, the shards are gathered.
    Parity: reference layers/embed_head.py:97-131."""

    def __init__(self, vocab: int, hidden: int, dtype, device, axis: str = "attn_tp"):
        super().__init__()
        d = get_dist_context()
        self.tp, self.rank, self.axis = d.attn_tp_size, d.attn_tp_rank, axis
        self.vocab = vocab
        self.per = -(-vocab // self.tp)
        self.per = (self.per + 7) // 8 * 8
        self.lo = self.rank * self.per
        self.weight = nn.Parameter(torch.zeros(self.per, hidden, dtype=dtype, device=device), requires_grad=False)

    def forward(self, hidden):
        import torch.distributed as dist
        local = ops.lm_head(hidden, self.weight)                                  # [B, per] fp32
        g = get_dist_context().group(self.axis)
        if g is None:
            return local[:, : self.vocab]
        B = local.shape[0]
        out = local.new_empty(self.tp * B, self.per)                                # shard r occupies rows [r * B, (r + 1) * B)
        dist.all_gather_into_tensor(out, local.contiguous(), group=g)
        return out.view(self.tp, B, self.per).permute(1, 0, 2).reshape(B, self.tp * self.per)[:, : self.vocab]

    @torch.no_grad()
    def load_full(self, w: torch.Tensor):
        part = w[self.lo: self.lo + self.per]
        self.weight.zero_()
        self.weight[: part.shape[0]].copy_(part.to(self.weight.dtype))


class RoutedExperts(nn.Module):
    """The experts this rank owns: ids [ep_rank*E_local, (ep_rank+1)*E_local), stacked for grouped GEMMs."""

    def __init__(self, num_experts: int, hidden: int, inter: int, dtype, device, quant=None, layer_idx: Optional[int] = None, act=None):
        super().__init__()
        self.act = act          # gated activation other than SwiGLU: see ops.reference.glu_act
        d = get_dist_context()
        # under an expert-load-balancing plan the stacked tensors hold PHYSICAL slots (a hot expert may fill several, on
        # different ranks); `phy2log` names the logical expert behind each slot of this layer
        from ..parallel.eplb import active_plan
        plan = active_plan() if layer_idx is not None else None
        self.phy2log = None
        if plan is not None:
            assert plan.num_logical == num_experts, "the EPLB plan was made for another expert count"
            self.phy2log = plan.phy2log[layer_idx].tolist()
            num_experts = plan.num_physical
        assert num_experts % d.ep_size == 0, "experts must divide evenly over the EP group"
        # with ffn_tp > 1 every expert's intermediate dimension is split over the TP group (this rank holds rows
        # [tp_rank * I/tp, (tp_rank + 1) * I/tp) of gate / up and the same columns of down); the caller sums the partial outputs
        self.inter_full, self.ffn_tp, self.ffn_tp_rank = inter, d.ffn_tp_size, d.ffn_tp_rank
        if self.ffn_tp > 1:
            assert inter % self.ffn_tp == 0 and (quant != "fp8" or (inter // self.ffn_tp) % 128 == 0), "expert intermediate size must split over ffn_tp"
            inter = inter // self.ffn_tp
        self.num_experts, self.hidden, self.inter, self.quant = num_experts, hidden, inter, quant
        self.num_local = num_experts // d.ep_size
        self.expert_offset = d.ep_rank * self.num_local
        wdt = torch.float8_e4m3fn if quant == "fp8" else dtype
        E = self.num_local
        if quant == "nvfp4":
            self._init_nvfp4(E, hidden, inter, device)
            return
        self.gate_up_proj = nn.Parameter(torch.empty(E, 2 * inter, hidden, dtype=wdt, device=device), requires_grad=False)
        self.down_proj = nn.Parameter(torch.empty(E, hidden, inter, dtype=wdt, device=device), requires_grad=False)
        if quant == "fp8":
            self.gate_up_scale = nn.Parameter(torch.ones(E, _ceil_div(2 * inter, 128), _ceil_div(hidden, 128), dtype=torch.float32, device=device), requires_grad=False)
            self.down_scale = nn.Parameter(torch.ones(E, _ceil_div(hidden, 128), _ceil_div(inter, 128), dtype=torch.float32, device=device), requires_grad=False)
        else:
            self.gate_up_scale = self.down_scale = None

    # ---- NVFP4 (ModelOpt checkpoints: packed e2m1 weights, e4m3 scale per 16, fp32 scale per matrix, fp32 input scale) ----
    # Parity: reference layers/backends/experts/nvfp4.py:75-160 (parameters, load_expert_weight, process_weights_after_loading).
    NVFP4_DEFAULT_INPUT_SCALE = 32.0 / (6.0 * 448.0)       # weights quantised here (random init, bf16 checkpoints): activations up to 32

    def _init_nvfp4(self, E, hidden, inter, device):
        assert self.ffn_tp == 1, "NVFP4 experts are sharded over the expert-parallel axis only"
        assert hidden % 256 == 0 and inter % 256 == 0, "NVFP4 GEMMs take K in multiples of 256"
        u8, e4 = torch.uint8, torch.float8_e4m3fn
        P = lambda *shape, dtype: nn.Parameter(torch.zeros(*shape, dtype=dtype, device=device), requires_grad=False)
        self.gate_up_proj = P(E, 2 * inter, hidden // 2, dtype=u8)
        self.down_proj = P(E, hidden, inter // 2, dtype=u8)
        self.gate_up_scale = P(E, 2 * inter, hidden // 16, dtype=e4)
        self.down_scale = P(E, hidden, inter // 16, dtype=e4)
        self.gate_up_scale_2 = P(E, 2, dtype=torch.float32)            # [gate, up]
        self.down_scale_2 = P(E, dtype=torch.float32)
        self.gate_up_input_scale = P(E, 2, dtype=torch.float32)
        self.down_input_scale = P(E, dtype=torch.float32)
        self._nvfp4_ready = False

    @torch.no_grad()
    def load_expert_part(self, logical_id: int, which: str, kind: str, t: torch.Tensor) -> bool:
        """One tensor of an NVFP4 checkpoint: `kind` in {weight, weight_scale, weight_scale_2, input_scale}."""
        slots = self.local_slots_of(logical_id)
        for sl in slots:
            self._set_part(sl, which, kind, t)
        return bool(slots)

    @torch.no_grad()
    def _set_part(self, sl: int, which: str, kind: str, t: torch.Tensor) -> None:
        I = self.inter
        if True:
            if which == "down":
                tgt = {"weight": self.down_proj[sl], "weight_scale": self.down_scale[sl], "weight_scale_2": self.down_scale_2[sl],
                       "input_scale": self.down_input_scale[sl]}[kind]
            else:
                half = 0 if which == "gate" else 1
                rows = slice(half * I, (half + 1) * I)
                tgt = {"weight": self.gate_up_proj[sl, rows], "weight_scale": self.gate_up_scale[sl, rows],
                       "weight_scale_2": self.gate_up_scale_2[sl, half], "input_scale": self.gate_up_input_scale[sl, half]}[kind]
            src = t.to(tgt.device)
            tgt.copy_(src.view(tgt.dtype).reshape(tgt.shape) if src.dtype in (torch.uint8, torch.float8_e4m3fn) else src.reshape(tgt.shape))
        self._nvfp4_ready = False

    @torch.no_grad()
    def _prepare_nvfp4(self):
        """Scales the kernels take: one activation scale for GEMM 1 (the largest over all experts, over all EP ranks), one per expert
        for GEMM 2, and alpha = input_scale * weight_scale_2.  Gate and up halves whose weight_scale_2 differ are brought onto the
        gate's by rescaling the up half's block scales."""
        d = get_dist_context()
        in1 = self.gate_up_input_scale.max().float().reshape(1)
        if d.ep_size > 1:
            import torch.distributed as dist
            dist.all_reduce(in1, op=dist.ReduceOp.MAX, group=d.group("ffn_ep"))
        ratio = self.gate_up_scale_2[:, 1] / self.gate_up_scale_2[:, 0].clamp_min(1e-30)
        if bool(((ratio - 1).abs() > 1e-6).any()):
            I = self.inter
            up = self.gate_up_scale[:, I:].float() * ratio.view(-1, 1, 1)
            self.gate_up_scale[:, I:].copy_(up.clamp(max=448.0).to(torch.float8_e4m3fn))
            self.gate_up_scale_2[:, 1].copy_(self.gate_up_scale_2[:, 0])
        self.a1_gscale = (1.0 / in1).float().contiguous()
        self.alpha1 = (in1 * self.gate_up_scale_2[:, 0]).float().contiguous()
        self.a2_gscale = (1.0 / self.down_input_scale).float().contiguous()
        self.alpha2 = (self.down_input_scale * self.down_scale_2).float().contiguous()
        self._nvfp4_ready = True

    def owns(self, expert_id: int) -> bool:
        return bool(self.local_slots_of(expert_id))

    def local_slots_of(self, logical_id: int):
        """Local slot indices that hold logical expert `logical_id` on this rank (one without a plan, any number with one)."""
        lo, hi = self.expert_offset, self.expert_offset + self.num_local
        if self.phy2log is None:
            return [logical_id - lo] if lo <= logical_id < hi else []
        return [p - lo for p in range(lo, hi) if self.phy2log[p] == logical_id]

    @torch.no_grad()
    def load_expert(self, logical_id: int, which: str, w: torch.Tensor, scale_inv: Optional[torch.Tensor] = None) -> bool:
        """Store one logical expert's matrix into every local slot that holds it; False when this rank holds none.  A full-size
        matrix is cut to this rank's ffn_tp shard first."""
        slots = self.local_slots_of(logical_id)
        if slots and self.ffn_tp > 1:
            lo, hi = self.ffn_tp_rank * self.inter, (self.ffn_tp_rank + 1) * self.inter
            if which == "down" and w.shape[1] == self.inter_full:
                w = w[:, lo:hi].contiguous()
                if scale_inv is not None:
                    scale_inv = scale_inv[:, lo // 128: hi // 128].contiguous()
            elif which != "down" and w.shape[0] == self.inter_full:
                w = w[lo:hi].contiguous()
                if scale_inv is not None:
                    scale_inv = scale_inv[lo // 128: hi // 128].contiguous()
        for s in slots:
            self.set_expert(s, which, w, scale_inv)
        return bool(slots)

    def forward(self, x, topk_idx, topk_w, add_in=None):
        """Local part of the routed output for the tokens given (weights applied, zero rows where no expert is local);
        `add_in` (the shared-expert output) is summed in by the same gather pass."""
        if self.quant == "nvfp4":
            if not self._nvfp4_ready:
                self._prepare_nvfp4()
            return ops.moe_experts_nvfp4(x, topk_idx, topk_w, self.gate_up_proj, self.gate_up_scale, self.alpha1, self.a1_gscale, self.down_proj,
                                         self.down_scale, self.alpha2, self.a2_gscale, self.expert_offset, add_in, act=self.act)
        return ops.moe_experts(x, topk_idx, topk_w, self.gate_up_proj, self.down_proj, self.gate_up_scale, self.down_scale,
                               self.expert_offset, add_in, act=self.act)

    @torch.no_grad()
    def set_expert(self, local_idx: int, which: str, w: torch.Tensor, scale_inv: Optional[torch.Tensor] = None):
        """which in {gate, up, down}; w is one expert's HF-layout matrix (fp8 + scales, or high precision)."""
        I = self.inter
        if self.quant == "nvfp4":
            # a high-precision (or fp8) matrix: quantised here, with a nominal activation scale
            if w.dtype == torch.float8_e4m3fn:
                w = ref.dequant_fp8_block(w, scale_inv)
            q, sf, s2 = ref.nvfp4_quant_weight(w.to(self.gate_up_proj.device).float())
            for kind, t in (("weight", q), ("weight_scale", sf), ("weight_scale_2", s2),
                            ("input_scale", torch.tensor(self.NVFP4_DEFAULT_INPUT_SCALE, device=q.device))):
                self._set_part(local_idx, which, kind, t)
            return
        tgt, tscale, rows = {
            "gate": (self.gate_up_proj, self.gate_up_scale, slice(0, I)),
            "up": (self.gate_up_proj, self.gate_up_scale, slice(I, 2 * I)),
            "down": (self.down_proj, self.down_scale, slice(0, self.hidden)),
        }[which]
        if self.quant == "fp8":
            if w.dtype != torch.float8_e4m3fn:
                w, scale_inv = ref.quant_fp8_block(w.to(tgt.device))
            else:
                w, scale_inv = ref.fp8_block_for_format(w.to(tgt.device), scale_inv.to(tgt.device))
            tgt[local_idx, rows].copy_(w)
            srows = slice(rows.start // 128, _ceil_div(rows.stop, 128))
            tscale[local_idx, srows].copy_(scale_inv)
        else:
            if w.dtype == torch.float8_e4m3fn:
                w = ref.dequant_fp8_block(w, scale_inv)
            tgt[local_idx, rows].copy_(w.to(tgt.dtype))

    @torch.no_grad()
    def init_random(self, gen, std: float = 0.02):
        dev = self.gate_up_proj.device
        for e in range(self.num_local):
            for which, shape in (("gate", (self.inter, self.hidden)), ("up", (self.inter, self.hidden)), ("down", (self.hidden, self.inter))):
                w = torch.empty(*shape, dtype=torch.float32, device=dev).normal_(0.0, std, generator=gen)
                self.set_expert(e, which, w)
