"""Process-group layout: two views of the same ranks, one for attention and one for the FFN.

Attention view  (pp, attn_dp, attn_sp, attn_tp); FFN view (pp, ffn_dp, ffn_ep, ffn_tp).  Both must
multiply out to the world size.  Each axis gets a device group (NCCL on GPUs) and a host group
(gloo) for control traffic.  Global rank = pp*(dp*sp*tp) + dp*(sp*tp) + sp*tp + tp.

Parity: reference runtime/context/distributed.py:12-316 (two DeviceMeshes with gloo + NCCL
groups :55-87, size check :89-102, PP neighbour helpers :281-315).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

_CTX: Optional["DistContext"] = None


@dataclass
class ParallelSpec:
    attention_dp: int = 1
    attention_sp: int = 1
    attention_tp: int = 1
    ffn_dp: int = 1
    ffn_ep: int = 1
    ffn_tp: int = 1
    pp: int = 1

    @property
    def world_size(self) -> int:
        return self.pp * self.attention_dp * self.attention_sp * self.attention_tp

    def validate(self) -> None:
        a = self.pp * self.attention_dp * self.attention_sp * self.attention_tp
        f = self.pp * self.ffn_dp * self.ffn_ep * self.ffn_tp
        if a != f:
            raise ValueError(f"attention layout ({a} ranks) and FFN layout ({f} ranks) must cover the same world size")
        for name in ("attention_dp", "attention_sp", "attention_tp", "ffn_dp", "ffn_ep", "ffn_tp", "pp"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")


def _axis_groups(shape: Tuple[int, ...], axis: int) -> List[List[int]]:
    """All rank lists that vary only along `axis` of a row-major mesh of the given shape."""
    strides = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        strides[i] = strides[i + 1] * shape[i + 1]
    others = [range(s) if i != axis else [0] for i, s in enumerate(shape)]
    out = []
    for coord in itertools.product(*others):
        base = sum(c * st for c, st in zip(coord, strides))
        out.append([base + k * strides[axis] for k in range(shape[axis])])
    return out


@dataclass
class DistContext:
    spec: ParallelSpec = field(default_factory=ParallelSpec)
    rank: int = 0
    world_size: int = 1
    device: torch.device = torch.device("cpu")
    groups: Dict[str, object] = field(default_factory=dict)        # device groups per axis name
    host_groups: Dict[str, object] = field(default_factory=dict)   # gloo groups per axis name
    coords_attn: Tuple[int, int, int, int] = (0, 0, 0, 0)
    coords_ffn: Tuple[int, int, int, int] = (0, 0, 0, 0)
    group_ranks: Dict[str, List[int]] = field(default_factory=dict)

    # -- coordinates
    @property
    def pp_rank(self) -> int: return self.coords_attn[0]
    @property
    def attn_dp_rank(self) -> int: return self.coords_attn[1]
    @property
    def attn_tp_rank(self) -> int: return self.coords_attn[3]
    @property
    def ep_rank(self) -> int: return self.coords_ffn[2]
    @property
    def ffn_tp_rank(self) -> int: return self.coords_ffn[3]
    @property
    def ep_size(self) -> int: return self.spec.ffn_ep
    @property
    def attn_tp_size(self) -> int: return self.spec.attention_tp
    @property
    def ffn_tp_size(self) -> int: return self.spec.ffn_tp
    @property
    def is_first_pp(self) -> bool: return self.pp_rank == 0
    @property
    def is_last_pp(self) -> bool: return self.pp_rank == self.spec.pp - 1

    def group(self, axis: str):
        return self.groups.get(axis)

    def host_group(self, axis: str):
        return self.host_groups.get(axis)

    def pp_neighbor(self, delta: int) -> int:
        per_stage = self.world_size // self.spec.pp
        return (self.rank + delta * per_stage) % self.world_size


def unflatten(rank: int, shape: Tuple[int, ...]) -> Tuple[int, ...]:
    out = []
    for s in reversed(shape):
        out.append(rank % s)
        rank //= s
    return tuple(reversed(out))


def init_dist_context(spec: ParallelSpec, rank: int = 0, world_size: int = 1, device=None,
                      create_groups: bool = True) -> DistContext:
    """Build the context; with world_size > 1 torch.distributed must already be initialised."""
    global _CTX
    spec.validate()
    if spec.world_size != world_size:
        raise ValueError(f"parallel layout needs {spec.world_size} ranks, world has {world_size}")
    a_shape = (spec.pp, spec.attention_dp, spec.attention_sp, spec.attention_tp)
    f_shape = (spec.pp, spec.ffn_dp, spec.ffn_ep, spec.ffn_tp)
    ctx = DistContext(spec=spec, rank=rank, world_size=world_size,
                      device=torch.device(device) if device is not None else torch.device("cpu"),
                      coords_attn=unflatten(rank, a_shape), coords_ffn=unflatten(rank, f_shape))
    axes = {"pp": (a_shape, 0), "attn_dp": (a_shape, 1), "attn_sp": (a_shape, 2), "attn_tp": (a_shape, 3),
            "ffn_dp": (f_shape, 1), "ffn_ep": (f_shape, 2), "ffn_tp": (f_shape, 3)}
    for name, (shape, axis) in axes.items():
        for ranks in _axis_groups(shape, axis):
            mine = rank in ranks
            if mine:
                ctx.group_ranks[name] = ranks
            if world_size > 1 and create_groups and len(ranks) > 1:
                # every rank must take part in every new_group call, in the same order
                backend = dist.get_backend()
                g = dist.new_group(ranks)
                hg = g if "gloo" in str(backend) and "nccl" not in str(backend) else dist.new_group(ranks, backend="gloo")
                if mine:
                    ctx.groups[name], ctx.host_groups[name] = g, hg
    _CTX = ctx
    return ctx


def get_dist_context() -> DistContext:
    global _CTX
    if _CTX is None:
        _CTX = DistContext()
    return _CTX


def set_dist_context(ctx: Optional[DistContext]) -> None:
    global _CTX
    _CTX = ctx
