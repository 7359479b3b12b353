"""Fused expert-parallel MoE: dispatch, grouped GEMMs and combine over NVLink peer memory (kernels in csrc/comm/ep.cu).

``FusedEP`` owns the symmetric receive buffers of one EP group and runs one MoE layer as five launches (dispatch, gate_up
GEMM whose prologue waits for the peers, SwiGLU + requant, down GEMM whose epilogue is the combine send and whose last
CTA signals the peers, weighted reduce) with no host synchronisation, so it can be captured in the decode CUDA graph.  Capacity per local expert (`cap`) bounds the
rows an expert can receive in one layer; a pair that finds its expert full is dropped and reported through the kernel
status words (size `cap` from the token budget: the default is four times the balanced load, never less than 256).

Parity: reference runtime/context/expert.py:42-224 (buffer sizing, low-latency mode with at most 128 dispatch tokens
per rank) and layers/backends/experts/deep_gemm.py:611-837 (dispatch -> grouped GEMMs -> combine data flow).
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional

import torch

from ..ops import sm100 as _k
from .symm import MAX_PEERS, SymmetricHeap

FP8 = torch.float8_e4m3fn


class EpLayout(_c.Structure):
    _fields_ = [("peer_base", _c.c_ulonglong * MAX_PEERS),
                ("off_cnt", _c.c_longlong), ("off_aq", _c.c_longlong), ("off_as", _c.c_longlong), ("off_abf", _c.c_longlong),
                ("off_info", _c.c_longlong), ("off_ret", _c.c_longlong), ("off_arrive", _c.c_longlong), ("off_done", _c.c_longlong),
                ("rank", _c.c_int), ("world", _c.c_int), ("E_local", _c.c_int), ("cap", _c.c_int), ("H", _c.c_int), ("top_k", _c.c_int),
                ("fp8", _c.c_int)]


def ep_heap_bytes(E_local: int, cap: int, H: int, max_tokens: int, top_k: int, fp8: bool) -> int:
    rows = E_local * cap
    act = rows * H + rows * (H // 128) * 4 if fp8 else rows * H * 2
    return act + rows * 8 + max_tokens * top_k * H * 2 + E_local * 4 + 64 * 1024


class FusedEP:
    def __init__(self, group, ep_rank: int, ep_size: int, num_experts: int, hidden: int, inter: int, top_k: int, max_tokens: int,
                 fp8: bool, cap: Optional[int] = None, spin_limit: int = 1 << 22):
        lib = _k.lib()
        assert lib.ne_ep_layout_size() == _c.sizeof(EpLayout), "EpLayout mismatch between Python and the kernel library"
        self.E_local = num_experts // ep_size
        self.H, self.I, self.K, self.fp8 = hidden, inter, top_k, fp8
        self.max_tokens = max_tokens
        balanced = -(-ep_size * max_tokens * top_k // num_experts)
        self.cap = cap if cap is not None else max(256, min(ep_size * max_tokens, 4 * balanced))
        self.cap = (self.cap + 127) // 128 * 128
        self.spin_limit = spin_limit
        E, C, H = self.E_local, self.cap, hidden
        self.heap = SymmetricHeap(ep_heap_bytes(E, C, H, max_tokens, top_k, fp8), group)
        assert self.heap.rank == ep_rank and self.heap.world_size == ep_size
        hp = self.heap
        self.b_cnt = hp.alloc(E * 4)
        self.b_arrive = hp.alloc(MAX_PEERS * 4)
        self.b_done = hp.alloc(MAX_PEERS * 4)
        self.b_info = hp.alloc(E * C * 8)
        self.b_ret = hp.alloc(max_tokens * top_k * H * 2)
        if fp8:
            self.b_aq = hp.alloc(E * C * H)
            self.b_as = hp.alloc(E * (H // 128) * C * 4)
            self.b_abf = None
        else:
            self.b_abf = hp.alloc(E * C * H * 2)
            self.b_aq = self.b_as = None
        L = EpLayout()
        for r in range(ep_size):
            L.peer_base[r] = hp.peer_ptrs[r]
        L.off_cnt, L.off_arrive, L.off_done, L.off_info, L.off_ret = (self.b_cnt.offset, self.b_arrive.offset, self.b_done.offset,
                                                                     self.b_info.offset, self.b_ret.offset)
        L.off_aq = self.b_aq.offset if fp8 else 0
        L.off_as = self.b_as.offset if fp8 else 0
        L.off_abf = 0 if fp8 else self.b_abf.offset
        L.rank, L.world, L.E_local, L.cap, L.H, L.top_k, L.fp8 = ep_rank, ep_size, E, C, H, top_k, int(fp8)
        self.layout = L
        dev = hp.device
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)       # [epoch, dispatch / down-GEMM / reduce CTA counters]
        self._comm1 = self._comm2 = None
        self.g = torch.empty(E, C, 2 * inter, dtype=torch.bfloat16, device=dev)
        if fp8:
            self.h_q = torch.empty(E, C, inter, dtype=FP8, device=dev)
            self.h_s = torch.empty(E, inter // 128, C, dtype=torch.float32, device=dev)
        else:
            self.h = torch.empty(E, C, inter, dtype=torch.bfloat16, device=dev)
        self.pair_ok = torch.zeros(max_tokens * top_k, dtype=torch.int32, device=dev)
        hp.barrier()

    def _comms(self):
        """The two GemmComm records of a layer (built once: they hold addresses only, the epoch is read on the device)."""
        if self._comm1 is None:
            L, hp = self.layout, self.heap
            me = hp.peer_ptrs[L.rank]
            epoch = self.state.data_ptr()
            c1 = _k.GemmComm()
            c1.wait_epoch, c1.wait_flags, c1.wait_world, c1.wait_spin = epoch, me + L.off_arrive, L.world, self.spin_limit
            c2 = _k.GemmComm()
            c2.scatter_mode, c2.row_info = 2, me + L.off_info
            for r in range(L.world):
                c2.scatter_base[r] = hp.peer_ptrs[r] + L.off_ret
                c2.tail_flag[r] = hp.peer_ptrs[r] + L.off_done + 4 * L.rank
            c2.tail_counter, c2.tail_epoch, c2.tail_world = self.state.data_ptr() + 8, epoch, L.world
            c2.tail_clear, c2.tail_clear_n = me + L.off_cnt, self.E_local
            self._comm1, self._comm2 = c1, c2
        return self._comm1, self._comm2

    def forward(self, experts, x, topk_idx, topk_w, ctx=None, add_in=None):
        lib = _k.lib()
        T, H = x.shape
        K, E, C, I = self.K, self.E_local, self.cap, self.I
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens exceed the EP buffer size {self.max_tokens}")
        x = _k._as_bf16_2d(x)
        idx = topk_idx.to(torch.int32).contiguous()
        w = topk_w.float().contiguous()
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        L = _c.byref(self.layout)
        epoch, ctr = _k._p(self.state), _c.c_void_p(self.state.data_ptr() + 4)
        st = _k._st()
        c1, c2 = self._comms()
        act = _k._act_args(getattr(experts, "act", None))
        cnt = self.heap.peer_ptrs[self.layout.rank] + self.layout.off_cnt       # per-expert row counts, filled by the senders' atomics
        _k._ck(lib.ne_ep_dispatch(L, _k._p(x), _k._p(idx), _k._p(self.pair_ok), _c.c_int(T * K), epoch, ctr, st), "ne_ep_dispatch")
        if self.fp8:
            aq = self.b_aq.view(FP8, (E, C, H))
            a_s = self.b_as.view(torch.float32, (E, H // 128, C))
            # about 128 rows per local expert or fewer (decode): weight-bound tiles.  Measured on the DeepSeek-V3 shapes with 32 rows
            # per expert: gate_up (N = 4096) 167 us with the scales on the CUDA cores against 170 us on the tensor cores, down
            # (N = 7168 = 32 x 224) 99 us against 85 us; so only the first GEMM keeps the CUDA-core scaling
            few = T * K * self.layout.world <= 128 * E * self.layout.world
            _k._gemm_comm(aq, H, C * H, experts.gate_up_proj, self.g, 2 * I, C * 2 * I, C, 2 * I, H, E, cnt, True, a_s, C,
                          (H // 128) * C, experts.gate_up_scale, c1, few_rows=few)
            _k._ck(lib.ne_act_mul(_k._p(self.g), _k._p(None), _k._p(self.h_q), _k._p(self.h_s), _c.c_int(C), _c.c_longlong((I // 128) * C),
                                  _c.c_void_p(cnt), _k._p(None), _c.c_int(E), _c.c_int(C), _c.c_int(I), *act, st), "ne_act_mul")
            _k._gemm_comm(self.h_q, I, C * I, experts.down_proj, self.g, H, 0, C, H, I, E, cnt, True, self.h_s, C,
                          (I // 128) * C, experts.down_scale, c2, few_rows=few and H % 224 != 0)
        else:
            ab = self.b_abf.view(torch.bfloat16, (E, C, H))
            _k._gemm_comm(ab, H, C * H, experts.gate_up_proj, self.g, 2 * I, C * 2 * I, C, 2 * I, H, E, cnt, False, None, 0, 0, None, c1)
            _k._ck(lib.ne_act_mul(_k._p(self.g), _k._p(self.h), _k._p(None), _k._p(None), _c.c_int(0), _c.c_longlong(0),
                                  _c.c_void_p(cnt), _k._p(None), _c.c_int(E), _c.c_int(C), _c.c_int(I), *act, st), "ne_act_mul")
            _k._gemm_comm(self.h, I, C * I, experts.down_proj, self.g, H, 0, C, H, I, E, cnt, False, None, 0, 0, None, c2)
        if callable(add_in):
            add_in = add_in()      # shared-expert output from the side stream: joined right before it is consumed
        _k._ck(lib.ne_ep_reduce(L, _k._p(self.pair_ok), _k._p(w), _k._p(add_in), _k._p(out), _c.c_int(T), epoch, _c.c_int(self.spin_limit),
                                _c.c_void_p(self.state.data_ptr() + 12), st), "ne_ep_reduce")
        return out


def install(config, dist_ctx) -> Optional[FusedEP]:
    """Create the fused backend for this rank's EP group when peers are reachable; returns None otherwise."""
    from . import ep
    from .symm import peers_reachable
    mc = config.model_config
    if dist_ctx.ep_size == 1 or not config.use_fused_comm or not torch.cuda.is_available():
        return None
    if mc.quant == "nvfp4":
        return None        # NVFP4 experts take the collective path (all-gather, local W4A4 experts, all-reduce): no fused form is built
    group = dist_ctx.group("ffn_ep")
    if not peers_reachable(group):
        return None
    max_tokens = max(config.max_num_batched_tokens, config.max_num_seqs * (1 + config.num_speculative_tokens))
    from .eplb import active_plan
    plan = active_plan()
    be = FusedEP(group, dist_ctx.ep_rank, dist_ctx.ep_size, plan.num_physical if plan is not None else mc.n_routed_experts,
                 mc.routed_expert_hidden_size or mc.hidden_size,      # latent experts exchange the down-projected rows
                 mc.moe_intermediate_size,
                 mc.num_experts_per_tok, max_tokens, mc.quant == "fp8")
    ep.set_fused_backend(be)
    return be
