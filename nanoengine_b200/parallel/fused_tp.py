"""Tensor-parallel collectives fused with their GEMMs over NVLink peer memory (kernels in csrc/comm/tp.cu).

``FusedTP`` owns the symmetric staging buffers of one TP group.  ``gemm_reduce_scatter`` runs the row-parallel GEMM with
its scatter epilogue, so each tile of the local partial product is stored into the owning rank's stage while later tiles
are still being computed, and the owner adds the partials; ``all_gather`` pushes this rank's rows into every peer and
returns the gathered rows as a view of local memory for the consuming GEMM.  Every step is a kernel on the caller's
stream (no host synchronisation), so the sequence can be captured in a CUDA graph.  Waits are bounded and report through
the kernel status words.

Parity: reference layers/parallelism_transition.py:67-200 (reduce-scatter / all-gather between TP attention and EP
experts), layers/backends/linear/deep_gemm.py:491-499 (all-reduce after row-parallel linears) and the push / pull kernels
of kernel/jit/sgl/csrc/kimi_k3/comm/sp_collective.cuh.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional

import torch

from ..ops import sm100 as _k
from .symm import MAX_PEERS, SymmetricHeap

FP8 = torch.float8_e4m3fn


class TpLayout(_c.Structure):
    _fields_ = [("peer_base", _c.c_ulonglong * MAX_PEERS),
                ("off_stage", _c.c_longlong), ("off_gather", _c.c_longlong), ("off_flags", _c.c_longlong),
                ("rank", _c.c_int), ("world", _c.c_int), ("rows_per_rank", _c.c_int), ("H", _c.c_int)]


class FusedTP:
    def __init__(self, group, axis: str, hidden: int, max_rows: int, spin_limit: int = 1 << 22):
        lib = _k.lib()
        assert lib.ne_tp_layout_size() == _c.sizeof(TpLayout), "TpLayout mismatch between Python and the kernel library"
        import torch.distributed as dist
        self.axis, self.group, self.H = axis, group, hidden
        self.world = dist.get_world_size(group)
        self.rpr_cap = -(-max_rows // self.world)                 # rows one rank can own in one call
        self.spin_limit = spin_limit
        slot = self.world * self.rpr_cap * hidden * 2
        self.heap = SymmetricHeap(2 * slot + 2 * slot + 64 * 1024, group)
        hp = self.heap
        self.rank = hp.rank
        self.b_flags = hp.alloc(2 * MAX_PEERS * 4)
        self.b_stage = hp.alloc(2 * slot)
        self.b_gather = hp.alloc(2 * slot)
        L = TpLayout()
        for r in range(self.world):
            L.peer_base[r] = hp.peer_ptrs[r]
        L.off_stage, L.off_gather, L.off_flags = self.b_stage.offset, self.b_gather.offset, self.b_flags.offset
        L.rank, L.world, L.rows_per_rank, L.H = self.rank, self.world, self.rpr_cap, hidden
        self.layout = L
        dev = hp.device
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)        # [epoch, push CTA counter, -, -]
        self.row_dst = torch.zeros(self.world * self.rpr_cap, dtype=torch.int64, device=dev)
        self.gather_view = self.b_gather.view(torch.bfloat16, (2, self.world * self.rpr_cap, hidden))
        self._epoch_host = 0                                              # mirrors the device epoch for buffer parity of views
        hp.barrier()

    # ---- helpers ----
    def _args(self):
        return _c.byref(self.layout), _k._p(self.state), _c.c_void_p(self.state.data_ptr() + 4), _k._st()

    def _advance(self):
        _k._ck(_k.lib().ne_tp_advance(_k._p(self.state), _k._st()), "ne_tp_advance")
        self._epoch_host += 1

    def _rpr(self, total_rows: int) -> int:
        rpr = -(-total_rows // self.world)
        if rpr > self.rpr_cap:
            raise ValueError(f"{total_rows} rows exceed the TP staging capacity {self.rpr_cap * self.world}")
        return rpr

    # ---- GEMM -> reduce-scatter ----
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, w_scale: Optional[torch.Tensor] = None, add_in=None) -> torch.Tensor:
        """x [T, K_local] @ w[N, K_local]^T summed over the group; returns this rank's rows [ceil(T / world), N]
        (rows past T are zero-padding sums and must be ignored by the caller)."""
        lib = _k.lib()
        N, K = w.shape
        assert N == self.H
        rpr = self._rpr(x.shape[0])
        T = self.world * rpr
        if x.shape[0] != T:               # pad to a multiple of the group size: the extra rows produce zeros in their owners' slots
            x = torch.cat([x, x.new_zeros(T - x.shape[0], x.shape[1])], 0)
        L, epoch, ctr, st = self._args()
        _k._ck(lib.ne_tp_row_dst(L, _k._p(self.row_dst), _c.c_int(rpr), epoch, st), "ne_tp_row_dst")
        dummy = self.row_dst            # D is unused: every row has an explicit destination
        x2 = _k._as_bf16_2d(x)
        if w.dtype == FP8:
            pre = getattr(x, "_ne_q", None)
            q, s = pre if (pre is not None and pre[0].shape == (T, K)) else _k.quant_fp8_1x128_raw(x2)
            _k._gemm(q, K, 0, w, dummy, N, 0, T, N, K, 1, None, None, True, s, T, 0, w_scale, False, row_dst=self.row_dst)
        else:
            _k._gemm(x2, x2.stride(0), 0, w, dummy, N, 0, T, N, K, 1, None, None, False, None, 0, 0, None, False, row_dst=self.row_dst)
        _k._ck(lib.ne_tp_signal(L, _c.c_int(0), epoch, st), "ne_tp_signal")
        out = torch.empty(rpr, N, dtype=torch.bfloat16, device=x.device)
        _k._ck(lib.ne_tp_reduce(L, _k._p(add_in), _k._p(out), _c.c_int(rpr), epoch, _c.c_int(self.spin_limit), st), "ne_tp_reduce")
        self._advance()
        return out

    # ---- plain collectives ----
    def reduce_scatter(self, xp: torch.Tensor) -> torch.Tensor:
        """xp [world * rpr, H] partial sums -> this rank's [rpr, H] of the total."""
        lib = _k.lib()
        rows = xp.shape[0]
        assert rows % self.world == 0 and xp.shape[1] == self.H
        rpr = self._rpr(rows)
        xp = _k._as_bf16_2d(xp).contiguous()
        L, epoch, ctr, st = self._args()
        _k._ck(lib.ne_tp_push(L, _k._p(xp), _c.c_int(rows), _c.c_int(rpr), _c.c_int(1), epoch, ctr, st), "ne_tp_push")
        out = torch.empty(rpr, self.H, dtype=torch.bfloat16, device=xp.device)
        _k._ck(lib.ne_tp_reduce(L, _k._p(None), _k._p(out), _c.c_int(rpr), epoch, _c.c_int(self.spin_limit), st), "ne_tp_reduce")
        self._advance()
        return out

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """x [rpr, H] on every rank -> [world * rpr, H]: a view of this rank's gather buffer, valid until the second
        next collective of this object."""
        lib = _k.lib()
        rpr = x.shape[0]
        assert x.shape[1] == self.H and rpr <= self.rpr_cap
        x = _k._as_bf16_2d(x).contiguous()
        L, epoch, ctr, st = self._args()
        parity = (self._epoch_host + 1) & 1
        _k._ck(lib.ne_tp_push(L, _k._p(x), _c.c_int(rpr), _c.c_int(max(rpr, 1)), _c.c_int(0), epoch, ctr, st), "ne_tp_push")
        _k._ck(lib.ne_tp_wait(L, _c.c_int(1), epoch, _c.c_int(self.spin_limit), st), "ne_tp_wait")
        self._advance()
        return self.gather_view[parity, : self.world * rpr]

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        if 0 < T <= self.rpr_cap:
            # few rows: every rank stores its partial into every peer's stage and adds the slots itself (one hop)
            lib = _k.lib()
            x = _k._as_bf16_2d(x).contiguous()
            L, epoch, ctr, st = self._args()
            _k._ck(lib.ne_tp_push(L, _k._p(x), _c.c_int(T), _c.c_int(T), _c.c_int(2), epoch, ctr, st), "ne_tp_push")
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=x.device)
            _k._ck(lib.ne_tp_reduce(L, _k._p(None), _k._p(out), _c.c_int(T), epoch, _c.c_int(self.spin_limit), st), "ne_tp_reduce")
            self._advance()
            return out
        pad = (-T) % self.world
        xp = x if pad == 0 else torch.cat([x, x.new_zeros(pad, x.shape[1])], 0)
        return self.all_gather(self.reduce_scatter(xp))[:T].clone()


def install(config, dist_ctx, axis: str = "attn_tp") -> Optional[FusedTP]:
    """Create the fused TP backend for this rank's group when peers are reachable; returns None otherwise."""
    from . import tp
    from .symm import peers_reachable
    group = dist_ctx.group(axis)
    if group is None or not config.use_fused_comm or not torch.cuda.is_available() or not peers_reachable(group):
        return None
    max_rows = max(config.max_num_batched_tokens, config.max_num_seqs * (1 + config.num_speculative_tokens))
    be = FusedTP(group, axis, config.model_config.hidden_size, max_rows)
    tp.set_fused_tp(be)
    return be
