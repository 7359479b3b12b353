"""KV-cache families, byte accounting and allocation.

MLA latent cache   [L, blocks, block_size, R + rope]   bf16/fp32, or fp8 e4m3 raw rows (576 B per token per layer
                                                        for DeepSeek-V3: clamped cast, no scales)
indexer key cache  [L, blocks, block_size * (D + 4)] u8 per page: block_size fp8 keys, then block_size fp32 scales
GQA cache          [2, L, blocks, block_size, kv_heads_local, head_dim]
recurrent state    hybrid models with gated delta-net layers keep, per sequence slot and linear layer, the delta-rule state
                   [Hv, Dv, Dk] fp32 and the convolution window [K-1, conv_dim]; the paged GQA cache then covers only the
                   full-attention layers.  Slot `state_slots` (one past the scheduler-visible range) is scratch.

DeepSeek-V4        one shared key / value row per token and layer in the latent-cache layout [L, blocks, block_size, head_dim];
                   every compressing layer adds pooled rows [blocks, max(1, block_size / ratio), head_dim] addressed through the
                   same block table (pooled row b of a sequence sits in the page of token b * ratio) and, per sequence slot, the
                   compressor's carry [c * ratio, c * head_dim] fp32 twice (values and scores; c = 2 for ratio 4).  With an fp8 cache a row
                   is 584 packed bytes (448 e4m3 values, 64 bf16 rotated dims, 7 scale bytes + pad) instead of head_dim values.

One extra block past the scheduler-visible range is reserved as the scratch page that dummy batches of idle
DP ranks write into.

Parity: reference runtime/context/cache/__init__.py:153-472 (budget :366-372, blocks :431-432),
cache/mla.py:45-199 (formats and shapes), cache/indexer.py:45-77, cache/gqa.py:56-71, cache/hca.py and cache/csa.py (the
compressed caches of DeepSeek-V4).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..models.config import ModelConfig


def torch_dtype(name: str):
    return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "fp8": torch.float8_e4m3fn}[name]


@dataclass
class CachePlan:
    mla: bool
    gqa: bool
    indexer: bool
    num_layers: int            # target layers + MTP layers held on this rank
    block_size: int
    kv_dtype: torch.dtype
    row_dim: int               # MLA: R + rope ; GQA: head_dim
    kv_heads_local: int = 1
    index_dim: int = 0
    # recurrent-state layers (gated delta-net)
    gdn: bool = False
    gdn_layers: int = 0
    state_slots: int = 0
    conv_dim: int = 0
    conv_k: int = 0
    gdn_heads: int = 0
    gdn_dv: int = 0
    gdn_dk: int = 0
    # GQA families whose layers have different head dims: the head dim of every cache layer (row_dim is their maximum; a
    # layer with a smaller one uses the front of its slab)
    layer_dims: Optional[List[int]] = None
    # hot / cold tier (DSA decode engines): the latent pages live in pinned host memory, `hot_rows` rows per sequence slot
    # and layer on the device
    # DeepSeek-V4: compression ratio of every layer (0 = window only); the width of a key / value row (row_dim is its stored size:
    # the same number, or the bytes of a packed row when the cache keeps fp8 values)
    dsv4_ratios: Optional[List[int]] = None
    dsv4_head_dim: int = 0
    hisparse: bool = False
    hot_rows: int = 0
    hs_slots: int = 0
    max_ctx: int = 0

    @property
    def dsv4(self) -> bool:
        return self.dsv4_ratios is not None

    @property
    def needs_state_slots(self) -> bool:
        return self.gdn or self.dsv4

    def comp_entries_per_page(self, ratio: int) -> int:
        return max(1, self.block_size // ratio)

    @property
    def state_slot_bytes(self) -> int:
        """Bytes one sequence slot takes over all layers that keep per-sequence state."""
        if self.dsv4:
            return sum(2 * 4 * (2 if r == 4 else 1) ** 2 * r * self.dsv4_head_dim for r in self.dsv4_ratios if r)
        if not self.gdn:
            return 0
        e = 2 if self.kv_dtype in (torch.bfloat16, torch.float16, torch.float8_e4m3fn) else 4
        return self.gdn_layers * (self.gdn_heads * self.gdn_dv * self.gdn_dk * 4 + (self.conv_k - 1) * self.conv_dim * e)

    @property
    def state_bytes(self) -> int:
        return (self.state_slots + 1) * self.state_slot_bytes

    @property
    def kv_block_bytes(self) -> int:
        e = torch.empty(0, dtype=self.kv_dtype).element_size()
        if self.dsv4:
            return (self.num_layers * self.block_size + sum(self.comp_entries_per_page(r) for r in self.dsv4_ratios if r)) * self.row_dim * e
        if self.mla:
            return self.num_layers * self.block_size * self.row_dim * e
        return 2 * self.num_layers * self.block_size * self.kv_heads_local * self.row_dim * e

    @property
    def indexer_block_bytes(self) -> int:
        return self.num_layers * self.block_size * (self.index_dim + 4) if self.indexer else 0

    @property
    def block_bytes(self) -> int:
        """Device bytes one logical page costs (under the hot / cold tier only the indexer keys of a page are on the device)."""
        return (0 if self.hisparse else self.kv_block_bytes) + self.indexer_block_bytes

    @property
    def hisparse_device_bytes(self) -> int:
        if not self.hisparse:
            return 0
        n = self.hs_slots + 1
        return self.num_layers * n * (self.hot_rows * (self.row_dim + 8) + self.max_ctx * 4 + 4)

    def plan_bits(self) -> int:
        from .._native import _core as C
        if self.dsv4:                    # shared-row pages + pooled-row pages with their per-sequence carry
            return C.PLAN_HCA | C.PLAN_CSA
        bits = C.PLAN_MLA if self.mla else C.PLAN_GQA
        if self.indexer:
            bits |= C.PLAN_INDEXER
        if self.gdn:
            bits |= C.PLAN_GDN          # one state slot per running sequence; no prefix reuse
        if self.hisparse:
            bits |= C.PLAN_HISPARSE
        return bits


def make_cache_plan(mc: ModelConfig, kv_dtype_name: str, block_size: int, attn_tp: int = 1, num_mtp_layers: int = 0,
                    use_indexer: bool = True, num_layers: Optional[int] = None, state_slots: int = 0, hisparse_rows: int = 0,
                    max_ctx: int = 0) -> CachePlan:
    plan = _make_cache_plan(mc, kv_dtype_name, block_size, attn_tp, num_mtp_layers, use_indexer, num_layers, state_slots)
    if hisparse_rows:
        assert plan.mla and plan.indexer, "the hot / cold tier needs an MLA cache with the DSA indexer"
        plan.hisparse, plan.hot_rows, plan.hs_slots, plan.max_ctx = True, hisparse_rows, state_slots, max_ctx
    return plan


def _make_cache_plan(mc: ModelConfig, kv_dtype_name: str, block_size: int, attn_tp: int = 1, num_mtp_layers: int = 0,
                     use_indexer: bool = True, num_layers: Optional[int] = None, state_slots: int = 0) -> CachePlan:
    L = (num_layers if num_layers is not None else mc.num_hidden_layers) + num_mtp_layers
    dt = torch_dtype(kv_dtype_name)
    if mc.is_dsv4:
        for r in mc.compress_ratios or []:
            assert r == 0 or block_size % r == 0 or r % block_size == 0, "a compression ratio must divide the page size or be a multiple of it"
        # every row passes an e4m3 round trip with one power-of-two scale per 64 values before it is stored; an fp8 cache keeps
        # it packed (e4m3 values, bf16 rotated dims, scale bytes: 584 bytes for 512 dims), any other dtype keeps the values
        packed = dt == torch.float8_e4m3fn
        from ..ops.reference import dsv4_row_bytes
        return CachePlan(True, False, False, mc.num_hidden_layers, block_size, torch.uint8 if packed else dt,
                         dsv4_row_bytes(mc.head_dim, mc.qk_rope_head_dim) if packed else mc.head_dim, state_slots=state_slots,
                         dsv4_ratios=[mc.compress_ratio(i) for i in range(mc.num_hidden_layers)], dsv4_head_dim=mc.head_dim)
    if mc.is_hybrid_gdn and mc.is_mla:
        # delta-attention layers between MLA layers (GLM5-next, Kimi-K3): latent pages for the full-attention layers (and the
        # MTP layers), one state slot per sequence for the linear ones
        return CachePlan(True, False, mc.has_indexer and use_indexer, mc.num_layers_of("full_attention") + num_mtp_layers, block_size, dt,
                         mc.mla_cache_dim, index_dim=mc.index_head_dim, gdn=True, gdn_layers=mc.num_layers_of("linear_attention"),
                         state_slots=state_slots, conv_dim=mc.gdn_conv_dim, conv_k=mc.linear_conv_kernel_dim,
                         gdn_heads=mc.linear_num_value_heads, gdn_dv=mc.linear_value_head_dim, gdn_dk=mc.linear_key_head_dim)
    if mc.is_hybrid_gdn:
        return CachePlan(False, True, False, mc.num_layers_of("full_attention"), block_size, dt, mc.head_dim,
                         kv_heads_local=max(1, mc.num_key_value_heads // attn_tp), gdn=True, gdn_layers=mc.num_layers_of("linear_attention"),
                         state_slots=state_slots, conv_dim=mc.gdn_conv_dim, conv_k=mc.linear_conv_kernel_dim,
                         gdn_heads=mc.linear_num_value_heads, gdn_dv=mc.linear_value_head_dim, gdn_dk=mc.linear_key_head_dim)
    if mc.is_mla:
        return CachePlan(True, False, mc.has_indexer and use_indexer, L, block_size, dt, mc.mla_cache_dim,
                         index_dim=mc.index_head_dim)
    if mc.num_kv_shared_layers or mc.global_head_dim:
        # window / global layers with their own head dims; KV-sharing layers own no cache layer
        own = [i for i in range(mc.num_hidden_layers) if mc.kv_source_layer(i) == i]
        dims = [mc.attn_head_dim(i) for i in own]
        return CachePlan(False, True, False, len(own), block_size, dt, max(dims), kv_heads_local=max(1, mc.num_key_value_heads // attn_tp),
                         layer_dims=dims)
    return CachePlan(False, True, False, L, block_size, dt, mc.head_dim, kv_heads_local=max(1, mc.num_key_value_heads // attn_tp))


def kv_budget_blocks(plan: CachePlan, total: int, utilization: float, used: int, peak: int, current: int, reserved: int = 0) -> int:
    """blocks = (total*util - used - peak + current - reserved) // bytes_per_block."""
    budget = int(total * utilization) - used - peak + current - reserved
    return max(0, budget // plan.block_bytes)


class KVCache:
    def __init__(self, plan: CachePlan, num_blocks: int, device):
        self.plan, self.num_blocks, self.device = plan, num_blocks, torch.device(device)
        nb = num_blocks + 1   # + scratch page
        self.scratch_block = num_blocks
        self.hisparse = None
        if plan.mla:
            # under the hot / cold tier the logical pages are the cold tier: pinned host memory the staging kernel reads
            # through the unified address space
            kv_dev = "cpu" if plan.hisparse else device
            self.kv = torch.zeros(plan.num_layers, nb, plan.block_size, plan.row_dim, dtype=torch.uint8 if plan.kv_dtype == torch.float8_e4m3fn else plan.kv_dtype, device=kv_dev)
            if plan.hisparse and self.device.type == "cuda":
                self.kv = self.kv.pin_memory()
            if plan.kv_dtype == torch.float8_e4m3fn:
                self.kv = self.kv.view(torch.float8_e4m3fn)
            self.layers: List = [self.kv[l] for l in range(plan.num_layers)]
        else:
            self.kv = torch.zeros(2, plan.num_layers, nb, plan.block_size, plan.kv_heads_local, plan.row_dim, dtype=plan.kv_dtype, device=device)
            self.layers = [(self.kv[0, l], self.kv[1, l]) for l in range(plan.num_layers)]
            if plan.layer_dims:
                def front(t, d):          # a contiguous [blocks, block_size, heads, d] cache at the front of the layer's slab
                    return t.reshape(-1)[: nb * plan.block_size * plan.kv_heads_local * d].view(nb, plan.block_size, plan.kv_heads_local, d)
                self.layers = [(front(self.kv[0, l], d), front(self.kv[1, l], d)) for l, d in enumerate(plan.layer_dims)]
        self.indexer = None
        self.indexer_layers = None
        if plan.indexer:
            self.indexer = torch.zeros(plan.num_layers, nb, plan.block_size * (plan.index_dim + 4), dtype=torch.uint8, device=device)
            self.indexer_layers = [self.indexer[l] for l in range(plan.num_layers)]
        if plan.hisparse:
            from .hisparse import HiSparseTier
            es = torch.empty(0, dtype=plan.kv_dtype).element_size()
            self.hisparse = HiSparseTier(plan.num_layers, plan.hs_slots, plan.hot_rows, plan.max_ctx, plan.row_dim * es,
                                         [self.kv[l] for l in range(plan.num_layers)], device)
        self.host_kv = None
        self.host_families = {}
        self.comp = self.comp_kv_state = self.comp_score_state = None
        if plan.dsv4:
            ns = plan.state_slots + 1
            self.comp, self.comp_kv_state, self.comp_score_state = [], [], []
            for r in plan.dsv4_ratios:
                if not r:
                    self.comp.append(None); self.comp_kv_state.append(None); self.comp_score_state.append(None)
                    continue
                c = 2 if r == 4 else 1
                self.comp.append(torch.zeros(nb, plan.comp_entries_per_page(r), plan.row_dim, dtype=plan.kv_dtype, device=device))
                self.comp_kv_state.append(torch.zeros(ns, c * r, c * plan.dsv4_head_dim, dtype=torch.float32, device=device))
                self.comp_score_state.append(torch.full((ns, c * r, c * plan.dsv4_head_dim), float("-inf"), dtype=torch.float32, device=device))
        self.rec_states = self.conv_states = None
        self.scratch_slot = plan.state_slots
        if plan.gdn:
            ns = plan.state_slots + 1   # + scratch slot for padded graph rows and dummy batches
            cdt = torch.bfloat16 if plan.kv_dtype == torch.float8_e4m3fn else plan.kv_dtype
            self.rec = torch.zeros(plan.gdn_layers, ns, plan.gdn_heads, plan.gdn_dv, plan.gdn_dk, dtype=torch.float32, device=device)
            self.conv = torch.zeros(plan.gdn_layers, ns, plan.conv_k - 1, plan.conv_dim, dtype=cdt, device=device)
            self.rec_states = [self.rec[l] for l in range(plan.gdn_layers)]
            self.conv_states = [self.conv[l] for l in range(plan.gdn_layers)]

    # ---- byte layout of the per-page cache families (what a PD transfer or any other page mover needs to know) ----
    def page_families(self) -> List[dict]:
        """One entry per cache family that is indexed by page id: `tensor` (the whole family), `planes` (how many
        [pages, page_bytes] arrays it is made of: layers, or 2 x layers for separate K and V), `plane_stride` and `page_bytes`
        in bytes.  Page `p` of plane `i` starts at byte `i * plane_stride + p * page_bytes` of the family.
        Parity: reference runtime/disagg/p2p/cache_layout.py:14-240 (strides of the KV, indexer and state families)."""
        def fam(name, t, planes):
            es = t.element_size()
            per_plane = t.numel() * es // planes
            pages = self.num_blocks + 1
            return {"name": name, "tensor": t, "planes": planes, "plane_stride": per_plane, "page_bytes": per_plane // pages}
        out = [fam("mla_kv" if self.plan.mla else "gqa_kv", self.kv, self.kv.shape[0] if self.plan.mla else 2 * self.kv.shape[1])]
        if self.indexer is not None:
            out.append(fam("indexer", self.indexer, self.indexer.shape[0]))
        for l, t in enumerate(self.comp or []):
            if t is not None:
                out.append(fam(f"dsv4_pooled_{l}", t, 1))
        return out

    def slot_families(self) -> List[dict]:
        """Cache families indexed by a per-sequence state slot instead of a page id (gated delta-net state and convolution
        window, compressor carries): same description, with `slot_bytes` in place of `page_bytes` and `slot_dim`, the tensor dimension
        the slot indexes."""
        out = []
        if self.plan.gdn:
            for name, t in (("gdn_state", self.rec), ("gdn_conv", self.conv)):
                planes = t.shape[0]
                per_plane = t.numel() * t.element_size() // planes
                out.append({"name": name, "tensor": t, "planes": planes, "plane_stride": per_plane, "slot_bytes": per_plane // t.shape[1], "slot_dim": 1})
        for l, t in enumerate(self.comp_kv_state or []):
            if t is not None:
                for name, u in ((f"dsv4_carry_kv_{l}", t), (f"dsv4_carry_score_{l}", self.comp_score_state[l])):
                    out.append({"name": name, "tensor": u, "planes": 1, "plane_stride": u.numel() * 4, "slot_bytes": u.numel() * 4 // u.shape[0], "slot_dim": 0})
        return out

    def transfer_families(self) -> List[dict]:
        """Everything a sequence owns, for a PD transfer: the per-slot families first (`by` = "slot", `page_bytes` = bytes per
        slot), then the per-page ones (`by` = "page")."""
        slots = [dict(f, by="slot", page_bytes=f["slot_bytes"]) for f in self.slot_families()]
        return slots + [dict(f, by="page") for f in self.page_families()]

    def allocate_host(self, num_host_blocks: int):
        """Pinned host tier used by preemption swap: one host array per page family (KV and, for DSA models, the indexer keys),
        so a swapped-in sequence finds every per-page cache it had.  Per-sequence state slots (gated delta-net) are not part
        of it: a swapped-out sequence keeps its slot on the device."""
        self.host_families = {}
        if num_host_blocks <= 0:
            return
        for f in self.page_families():
            self.host_families[f["name"]] = torch.zeros(f["planes"], num_host_blocks, f["page_bytes"], dtype=torch.uint8,
                                                        pin_memory=self.device.type == "cuda")
        self.host_kv = self.host_families["mla_kv" if self.plan.mla else "gqa_kv"]

    def block_views(self, bid: int) -> List[torch.Tensor]:
        """Byte views of everything block `bid` holds (all layers of every cache family), for the file-backed tier."""
        kv = self.kv.view(torch.uint8) if self.kv.dtype == torch.float8_e4m3fn else self.kv
        out = [kv[:, bid] if self.plan.mla else kv[:, :, bid]]
        if self.indexer is not None:
            out.append(self.indexer[:, bid])
        for t in self.comp or []:
            if t is not None:
                out.append(t[bid])
        return out

    def swap(self, src: List[int], dst: List[int], to_host: bool):
        """Copy whole pages (all planes of every page family) between the device caches and the host tier."""
        if not src:
            return
        for f in self.page_families():
            host = self.host_families[f["name"]]
            t = f["tensor"]
            dev = (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).reshape(-1).view(torch.uint8).view(f["planes"], -1, f["page_bytes"])
            if self.device.type == "cuda" and host.is_pinned():
                # one kernel copies every (plane, page) pair straight between the pinned host tier and the device cache
                from ..ops import sm100 as _k
                import ctypes as _c
                d_stride, h_stride = f["plane_stride"], host.shape[1] * f["page_bytes"]
                si = torch.tensor(src, dtype=torch.int32).to(self.device, non_blocking=True)
                di = torch.tensor(dst, dtype=torch.int32).to(self.device, non_blocking=True)
                dst_t, src_t, ds, ss = (host, dev, h_stride, d_stride) if to_host else (dev, host, d_stride, h_stride)
                _k._ck(_k.lib().ne_kv_swap(_c.c_void_p(dst_t.data_ptr()), _c.c_void_p(src_t.data_ptr()), _k._p(si), _k._p(di), _c.c_int(len(src)),
                                           _c.c_int(f["planes"]), _c.c_longlong(f["page_bytes"]), _c.c_longlong(ds), _c.c_longlong(ss), _k._st()),
                       "ne_kv_swap")
                continue        # stream order is enough: later kernels that reuse the pages run behind this copy
            s_ = torch.as_tensor(src, dtype=torch.long)
            d_ = torch.as_tensor(dst, dtype=torch.long)
            if to_host:
                host.index_copy_(1, d_, dev.index_select(1, s_.to(dev.device)).to("cpu"))
            else:
                dev.index_copy_(1, d_.to(dev.device), host.index_select(1, s_).to(dev.device, non_blocking=True))
