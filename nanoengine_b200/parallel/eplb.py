"""Expert-parallel load balancing: replicate hot experts into redundant slots, pack the physical experts onto GPUs so the
per-GPU load is even, and remap logical expert ids chosen by the router to physical slots.

  rebalance_experts(load [L, E], num_physical, num_gpus, num_groups=1, num_nodes=1)
      -> phy2log [L, P], log2phy [L, E, R] (-1 padded), logcnt [L, E]
  map_logical_to_physical(topk_idx, log2phy, logcnt, token_ids)  picks a replica per (token, expert) by hashing the token id,
      so a token always meets the same replica and replicas share the load evenly.

With groups > 1 and nodes > 1 the packing is hierarchical: expert groups are first spread over nodes (keeps DeepSeek's
group-limited routing node-local), replicas are created inside each node, then packed onto that node's GPUs.

Parity: reference layers/backends/experts/eplb.py:11-455 (hierarchical rebalance, replicate, logical->physical map),
triton/generic/moe.py:561 (hash map kernel), experts/deep_gemm.py:47-67 (dummy balance switch).
"""
from __future__ import annotations

from typing import Tuple

import torch


def balanced_packing(weight: torch.Tensor, num_packs: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """weight [L, n] -> (pack_index [L, n], rank_in_pack [L, n]); every pack gets n/num_packs items, loads as even as a
    longest-processing-time greedy can make them."""
    L, n = weight.shape
    assert n % num_packs == 0
    per = n // num_packs
    pack_index = torch.full((L, n), -1, dtype=torch.int64)
    rank_in_pack = torch.full((L, n), -1, dtype=torch.int64)
    order = weight.float().sort(-1, descending=True).indices
    for l in range(L):
        loads = [0.0] * num_packs
        counts = [0] * num_packs
        for i in order[l].tolist():
            p = min((q for q in range(num_packs) if counts[q] < per), key=lambda q: loads[q])
            pack_index[l, i], rank_in_pack[l, i] = p, counts[p]
            loads[p] += float(weight[l, i]); counts[p] += 1
    return pack_index, rank_in_pack


def replicate_experts(weight: torch.Tensor, num_phy: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Give the num_phy - E redundant slots to the experts with the highest load per replica, one at a time.
    Returns phy2log [L, num_phy], rank (replica index) [L, num_phy], logcnt [L, E]."""
    L, E = weight.shape
    assert num_phy >= E
    phy2log = torch.arange(num_phy, dtype=torch.int64).repeat(L, 1)
    rank = torch.zeros(L, num_phy, dtype=torch.int64)
    logcnt = torch.ones(L, E, dtype=torch.int64)
    ar = torch.arange(L)
    for i in range(E, num_phy):
        hot = (weight.float() / logcnt).argmax(-1)
        phy2log[:, i] = hot
        rank[:, i] = logcnt[ar, hot]
        logcnt[ar, hot] += 1
    return phy2log, rank, logcnt


def rebalance_experts(load: torch.Tensor, num_physical: int, num_gpus: int, num_groups: int = 1, num_nodes: int = 1):
    load = load.float().cpu()
    L, E = load.shape
    assert num_physical % num_gpus == 0 and num_gpus % num_nodes == 0
    if num_groups > 1 and num_nodes > 1 and num_groups % num_nodes == 0 and E % num_groups == 0 and num_physical % num_nodes == 0:
        # 1) groups -> nodes
        gsz = E // num_groups
        gload = load.view(L, num_groups, gsz).sum(-1)
        gpack, grank = balanced_packing(gload, num_nodes)
        gpn = num_groups // num_nodes
        log2mlog = (((gpack * gpn + grank) * gsz).unsqueeze(-1) + torch.arange(gsz)).flatten(-2)     # logical -> node-major order
        mlog2log = torch.empty_like(log2mlog)
        mlog2log.scatter_(1, log2mlog, torch.arange(E).repeat(L, 1))
        # 2) replicate inside each node, 3) pack onto the node's GPUs
        per_node_log, per_node_phy = E // num_nodes, num_physical // num_nodes
        w_node = load.gather(1, mlog2log).view(L * num_nodes, per_node_log)
        p2m, prank, mcnt = replicate_experts(w_node, per_node_phy)
        w_phy = (w_node / mcnt).gather(1, p2m)
        pack, prk = balanced_packing(w_phy, num_gpus // num_nodes)
        per_gpu = num_physical // num_gpus
        slot = pack * per_gpu + prk
        pp2p = torch.empty_like(slot)
        pp2p.scatter_(1, slot, torch.arange(per_node_phy).repeat(L * num_nodes, 1))
        pp2m = p2m.gather(1, pp2p)
        pp2m = (pp2m.view(L, num_nodes, -1) + torch.arange(0, E, per_node_log).view(1, -1, 1)).flatten(-2)
        phy2log = mlog2log.gather(1, pp2m)
        phyrank = prank.gather(1, pp2p).view(L, -1)
        logcnt = mcnt.view(L, -1).gather(1, log2mlog)
    else:
        p2l, prank, logcnt = replicate_experts(load, num_physical)
        w_phy = (load / logcnt).gather(1, p2l)
        pack, prk = balanced_packing(w_phy, num_gpus)
        per_gpu = num_physical // num_gpus
        slot = pack * per_gpu + prk
        order = torch.empty_like(slot)
        order.scatter_(1, slot, torch.arange(num_physical).repeat(L, 1))
        phy2log, phyrank = p2l.gather(1, order), prank.gather(1, order)
    R = int(logcnt.max())
    log2phy = torch.full((L, E, R), -1, dtype=torch.int64)
    log2phy.view(L, -1).scatter_(1, phy2log * R + phyrank, torch.arange(num_physical).repeat(L, 1))
    return phy2log, log2phy, logcnt


def map_logical_to_physical(topk_idx: torch.Tensor, log2phy_layer: torch.Tensor, logcnt_layer: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """topk_idx [T, K] logical ids -> physical ids; replica = hash(token) mod replica count."""
    dev = topk_idx.device
    cnt = logcnt_layer.to(dev)[topk_idx.long()]                                       # [T, K]
    h = (token_ids.to(dev).long().unsqueeze(1) * 2654435761 + torch.arange(topk_idx.shape[1], device=dev) * 40503) & 0x7FFFFFFF
    rep = h % cnt
    return log2phy_layer.to(dev)[topk_idx.long(), rep].to(topk_idx.dtype)


def dummy_balanced_topk(num_tokens: int, top_k: int, num_experts: int, device="cpu") -> torch.Tensor:
    """Round-robin expert ids (perfectly balanced), for capacity benchmarks with random-init routers."""
    base = torch.arange(num_tokens * top_k, device=device) % num_experts
    return base.view(num_tokens, top_k).to(torch.int32)


# ---- the plan a worker serves under ------------------------------------------------------------------------------------
class EplbPlan:
    """Physical expert layout of a model: `phy2log [L, P]` (which logical expert every physical slot holds; slots are dealt to
    the EP ranks in contiguous runs of P / ep), `log2phy [L, E, R]` (-1 padded) and `logcnt [L, E]` for the routers.  Rows are
    indexed by the model's layer index; dense layers carry an identity row nobody reads."""

    def __init__(self, phy2log: torch.Tensor, log2phy: torch.Tensor, logcnt: torch.Tensor):
        self.phy2log, self.log2phy, self.logcnt = phy2log.long(), log2phy.long(), logcnt.long()
        self.num_layers, self.num_physical = self.phy2log.shape
        self.num_logical = self.logcnt.shape[1]
        self._dev = {}

    @classmethod
    def from_load(cls, load: torch.Tensor, num_redundant: int, ep_size: int, num_groups: int = 1) -> "EplbPlan":
        L, E = load.shape
        P = E + num_redundant
        if P % ep_size:
            raise ValueError(f"{E} experts + {num_redundant} redundant slots do not divide over {ep_size} EP ranks")
        return cls(*rebalance_experts(load, P, ep_size, num_groups, 1))

    def slots_of(self, layer: int, logical: int):
        row = self.log2phy[layer, logical]
        return [int(p) for p in row.tolist() if p >= 0]

    def router_tables(self, layer: int, device):
        """(log2phy [E, R] int32, logcnt [E] int32) of one layer on `device`, as the routing kernel reads them."""
        key = (layer, str(device))
        if key not in self._dev:
            self._dev[key] = (self.log2phy[layer].to(torch.int32).contiguous().to(device), self.logcnt[layer].to(torch.int32).contiguous().to(device))
        return self._dev[key]


_ACTIVE = None


def set_active_plan(plan) -> None:
    global _ACTIVE
    _ACTIVE = plan


def active_plan():
    return _ACTIVE
