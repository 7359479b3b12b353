"""Tensor-parallel communication for attention / dense FFN blocks and the hand-over between TP attention and EP experts.

Three collectives matter: the reduction after a row-parallel GEMM (o_proj, down_proj), and the reduce-scatter /
all-gather pair that turns "every TP rank holds all tokens" into "every rank owns a slice of the tokens" before the
expert-parallel MoE and back.  On CPU ranks (gloo) and as the measured baseline they are torch.distributed calls; on GPUs
with peer access the row-parallel GEMM writes its partial tiles straight into the owners' staging buffers through its
scatter epilogue and a small kernel reduces them (``FusedTP``: GEMM -> reduce-scatter), and the all-gather pushes rows
into every peer's gathered buffer ahead of the consuming GEMM.

Parity: reference layers/backends/linear/deep_gemm.py:491-499 + linear/generic.py:314-319 (all-reduce after row-parallel
GEMMs), layers/parallelism_transition.py:24-200 (AttnToFfn pad+chunk / reduce-scatter, FfnToAttn all-gather),
kernel/jit/sgl/csrc/kimi_k3/comm/sp_collective.cuh (NVLS reduce-scatter / all-gather kernels).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .dist import get_dist_context

_FUSED_TP = None


def set_fused_tp(obj) -> None:
    global _FUSED_TP
    _FUSED_TP = obj


def get_fused_tp():
    return _FUSED_TP


def tp_all_reduce(x: torch.Tensor, axis: str = "attn_tp") -> torch.Tensor:
    d = get_dist_context()
    g = d.group(axis)
    if g is None:
        return x
    if x.is_cuda and _FUSED_TP is not None and _FUSED_TP.axis == axis:
        return _FUSED_TP.all_reduce(x)
    dist.all_reduce(x, group=g)
    return x


def _pad_rows(x: torch.Tensor, mult: int) -> torch.Tensor:
    T = x.shape[0]
    pad = (-T) % mult
    if pad == 0:
        return x
    return torch.cat([x, x.new_zeros(pad, *x.shape[1:])], 0)


def tp_reduce_scatter(x: torch.Tensor, axis: str = "attn_tp") -> torch.Tensor:
    """Sum over the TP group and keep this rank's slice of the (padded) rows: [T, H] -> [ceil(T/tp), H]."""
    d = get_dist_context()
    g = d.group(axis)
    if g is None:
        return x
    tp = dist.get_world_size(g)
    xp = _pad_rows(x, tp)
    if x.is_cuda and _FUSED_TP is not None and _FUSED_TP.axis == axis:
        return _FUSED_TP.reduce_scatter(xp)
    out = xp.new_empty(xp.shape[0] // tp, *xp.shape[1:])
    if dist.get_backend(g) == "gloo":
        dist.all_reduce(xp, group=g)
        r = dist.get_rank(g)
        out.copy_(xp[r * out.shape[0]: (r + 1) * out.shape[0]])
    else:
        dist.reduce_scatter_tensor(out, xp.contiguous(), group=g)
    return out


def tp_all_gather(x: torch.Tensor, total_rows: Optional[int] = None, axis: str = "attn_tp") -> torch.Tensor:
    """Inverse of the scatter: [T/tp, H] per rank -> [T, H] on every rank (padding rows dropped)."""
    d = get_dist_context()
    g = d.group(axis)
    if g is None:
        return x
    tp = dist.get_world_size(g)
    if x.is_cuda and _FUSED_TP is not None and _FUSED_TP.axis == axis:
        out = _FUSED_TP.all_gather(x)
    else:
        out = x.new_empty(x.shape[0] * tp, *x.shape[1:])
        dist.all_gather_into_tensor(out, x.contiguous(), group=g)
    return out if total_rows is None else out[:total_rows]


def tp_linear_reduce_scatter(x: torch.Tensor, proj, axis: str = "attn_tp") -> torch.Tensor:
    """Row-parallel projection followed by the reduce-scatter over the TP group: [T, K_local] -> [ceil(T/tp), N].
    With the fused backend the GEMM's epilogue stores each tile straight into the owning rank's staging buffer."""
    d = get_dist_context()
    if d.group(axis) is not None and x.is_cuda and _FUSED_TP is not None and _FUSED_TP.axis == axis and proj.bias is None:
        return _FUSED_TP.gemm_reduce_scatter(x, proj.weight, proj.weight_scale_inv)
    return tp_reduce_scatter(proj(x), axis)


def tp_all_gather_linear(x_slice: torch.Tensor, total_rows: int, proj, axis: str = "attn_tp") -> torch.Tensor:
    """All-gather of the token slices followed by a column-parallel projection: [T/tp, H] per rank -> [T, N_local].
    With the fused backend (bf16 weight, no bias) the GEMM reads the receive buffer directly and its producer warp waits per
    source rank, so the product overlaps the arrival of the peers' rows; otherwise gather, then project."""
    d = get_dist_context()
    f = _FUSED_TP
    if (d.group(axis) is not None and x_slice.is_cuda and f is not None and f.axis == axis and proj.bias is None
            and proj.weight.dtype == torch.bfloat16 and 1 <= x_slice.shape[0] <= f.rpr_cap):
        return f.all_gather_gemm(x_slice, proj.weight)[:total_rows]
    return proj(tp_all_gather(x_slice, total_rows, axis))


def attn_to_ffn(x_partial: torch.Tensor) -> torch.Tensor:
    """After a row-parallel o_proj whose output is still a per-rank partial sum: reduce-scatter so every rank continues
    with its own slice of the tokens (what the EP experts want), instead of all-reduce + chunk."""
    return tp_reduce_scatter(x_partial, "attn_tp")


def ffn_to_attn(x_slice: torch.Tensor, total_rows: int) -> torch.Tensor:
    return tp_all_gather(x_slice, total_rows, "attn_tp")
