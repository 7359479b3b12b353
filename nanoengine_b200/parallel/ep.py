"""Expert-parallel MoE execution.

Three paths, chosen per call:

* EP = 1: the local grouped-GEMM path (padded ``[E, max_m, H]`` layout on the GPU, a loop on CPU).
* EP > 1 on CUDA with a symmetric heap: the fused sm_100a kernels - dispatch with fp8 1x128 quantisation
  written straight into the expert owner's receive buffer by peer stores, grouped tcgen05 GEMMs, and a
  combine that pushes weighted rows back to the token's source GPU (``parallel/fused_moe.py``).
* EP > 1 otherwise (CPU/gloo ranks, or no peer access): all-gather every rank's tokens, run the local
  experts on all of them, sum-reduce and keep the own slice.  This is the correctness oracle for the
  fused path and what the multi-process CPU tests run.

Parity: reference layers/backends/experts/generic.py:107-184 (all-gather / all-reduce EP fallback),
experts/local_dispatch.py:28-217 (EP = 1), experts/deep_gemm.py:611-837 + token_dispatcher.py (DeepEP paths).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .dist import get_dist_context

_FUSED = None  # set by parallel.fused_moe.install() when a symmetric heap is available

# Post-steps the routers apply to the expert ids they pick (see ops.reference.moe_route): set once per worker from the
# engine configuration.  `balance_ranks` > 0 is the `dummy_eplb` switch.
_ROUTING = {"balance_ranks": 0}


def set_routing_options(balance_ranks: int = 0) -> None:
    _ROUTING["balance_ranks"] = int(balance_ranks)


def routing_options(layer_idx: Optional[int] = None, device=None) -> dict:
    """Keyword arguments for `ops.moe_route`: the dummy-balance switch, and under an EPLB plan the logical -> physical tables
    of the layer."""
    out = dict(_ROUTING)
    if layer_idx is not None and not out["balance_ranks"]:
        from .eplb import active_plan
        plan = active_plan()
        if plan is not None:
            out["log2phy"], out["logcnt"] = plan.router_tables(layer_idx, device)
    return out


def set_fused_backend(obj) -> None:
    global _FUSED
    _FUSED = obj


def get_fused_backend():
    return _FUSED


def ep_moe_allgather(experts, x, topk_idx, topk_w, group, ep_size: int, ep_rank: int, max_tokens: Optional[int] = None):
    """Oracle EP: gather tokens of all ranks (padded to the largest count), compute, reduce, slice."""
    T, H = x.shape
    dev = x.device
    counts = torch.zeros(ep_size, dtype=torch.int64, device=dev)
    counts[ep_rank] = T
    dist.all_reduce(counts, group=group)
    m = int(counts.max()) if max_tokens is None else max_tokens
    K = topk_idx.shape[1]
    xp = torch.zeros(m, H, dtype=x.dtype, device=dev); xp[:T] = x
    ip = torch.full((m, K), -1, dtype=topk_idx.dtype, device=dev); ip[:T] = topk_idx
    wp = torch.zeros(m, K, dtype=topk_w.dtype, device=dev); wp[:T] = topk_w
    gx = torch.empty(ep_size * m, H, dtype=x.dtype, device=dev)
    gi = torch.empty(ep_size * m, K, dtype=topk_idx.dtype, device=dev)
    gw = torch.empty(ep_size * m, K, dtype=topk_w.dtype, device=dev)
    dist.all_gather_into_tensor(gx, xp, group=group)
    dist.all_gather_into_tensor(gi, ip, group=group)
    dist.all_gather_into_tensor(gw, wp, group=group)
    part = experts(gx, gi, gw).float()
    dist.all_reduce(part, group=group)
    return part[ep_rank * m: ep_rank * m + T].to(x.dtype)


def ep_moe_forward(experts, x, topk_idx, topk_w, ctx=None, add_in=None):
    """Routed-expert output for this rank's tokens; `add_in` (shared-expert output) is added to it."""
    d = get_dist_context()
    if d.ep_size == 1:
        return experts(x, topk_idx, topk_w, add_in)
    if x.is_cuda and _FUSED is not None:
        return _FUSED.forward(experts, x, topk_idx, topk_w, ctx, add_in)
    out = ep_moe_allgather(experts, x, topk_idx, topk_w, d.group("ffn_ep"), d.ep_size, d.ep_rank)
    if callable(add_in):
        add_in = add_in()
    return out if add_in is None else out + add_in
