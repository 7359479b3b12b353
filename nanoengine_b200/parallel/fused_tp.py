"""Tensor-parallel collectives fused with their GEMMs over NVLink peer memory (kernels in csrc/comm/tp.cu).

``FusedTP`` owns the symmetric staging buffers of one TP group.  ``gemm_reduce_scatter`` runs the row-parallel GEMM with
its scatter epilogue, so each tile of the local partial product is stored into the owning rank's stage while later tiles
are still being computed, and the owner adds the partials; ``all_gather_gemm`` pushes this rank's rows into every peer and
runs the consuming GEMM straight on the receive buffer, its producer warp gated per source rank.  Every step is a kernel on the caller's
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


class NvlsLayout(_c.Structure):
    _fields_ = [("mc_base", _c.c_ulonglong), ("local_base", _c.c_ulonglong), ("off_buf", _c.c_longlong), ("off_out", _c.c_longlong),
                ("off_flags", _c.c_longlong), ("rank", _c.c_int), ("world", _c.c_int), ("rows_cap", _c.c_int), ("H", _c.c_int)]


class NvlsCollectives:
    """All-reduce, reduce-scatter and all-gather of bf16 rows through the NVSwitch (multimem instructions over a multicast
    mapping of a symmetric buffer; kernel in csrc/comm/nvls.cu).  Opt-in: needs NE_NVLS=1 in every rank's environment before
    the first symmetric heap is created, and a fabric that offers a multicast object to the group - `available` says whether
    both held.  One kernel per call, capturable in a CUDA graph, bounded waits."""

    def __init__(self, group, hidden: int, max_rows: int, spin_limit: int = 1 << 22):
        lib = _k.lib()
        assert lib.ne_nvls_layout_size() == _c.sizeof(NvlsLayout), "NvlsLayout mismatch between Python and the kernel library"
        import torch.distributed as dist
        self.H, self.group = hidden, group
        self.world = dist.get_world_size(group)
        self.rows_cap = -(-max_rows // self.world) * self.world
        self.spin_limit = spin_limit
        nbytes = self.rows_cap * hidden * 2
        self.heap = SymmetricHeap(2 * nbytes + 64 * 1024, group)
        hp = self.heap
        self.available = bool(hp.multicast_ptr)
        self.b_flags = hp.alloc(64)
        self.b_buf = hp.alloc(nbytes)
        self.b_out = hp.alloc(nbytes)
        L = NvlsLayout()
        L.mc_base, L.local_base = hp.multicast_ptr, hp.peer_ptrs[hp.rank]
        L.off_buf, L.off_out, L.off_flags = self.b_buf.offset, self.b_out.offset, self.b_flags.offset
        L.rank, L.world, L.rows_cap, L.H = hp.rank, self.world, self.rows_cap, hidden
        self.layout = L
        self.state = torch.zeros(4, dtype=torch.int32, device=hp.device)
        hp.barrier()

    def _run(self, x: torch.Tensor, out: torch.Tensor, rows: int, mode: int):
        if not self.available:
            raise RuntimeError("no NVLink multicast object for this group (set NE_NVLS=1 on every rank; needs NVSwitch multicast support)")
        _k._ck(_k.lib().ne_nvls_collective(_c.byref(self.layout), _k._p(x), _k._p(out), _c.c_int(rows), _c.c_int(mode), _k._p(self.state),
                                           _c.c_int(self.spin_limit), _k._st()), "ne_nvls_collective")
        return out

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        x = _k._as_bf16_2d(x).contiguous()
        return self._run(x, torch.empty_like(x), x.shape[0], 0)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        x = _k._as_bf16_2d(x).contiguous()
        assert x.shape[0] % self.world == 0
        return self._run(x, torch.empty(x.shape[0] // self.world, self.H, dtype=torch.bfloat16, device=x.device), x.shape[0], 1)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        x = _k._as_bf16_2d(x).contiguous()
        return self._run(x, torch.empty(x.shape[0] * self.world, self.H, dtype=torch.bfloat16, device=x.device), x.shape[0], 2)


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
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)        # [epoch, push / GEMM-tail / reduce CTA counters]
        self._comm_rs = None
        hp.barrier()
        # in-switch variants of the stand-alone collectives, when the process opted in and the fabric offers multicast
        import os
        self.nvls = None
        if os.environ.get("NE_NVLS", "0") == "1":
            nv = NvlsCollectives(group, hidden, max_rows, spin_limit)
            self.nvls = nv if nv.available else None

    # ---- helpers ----
    def _args(self):
        return _c.byref(self.layout), _k._p(self.state), _c.c_void_p(self.state.data_ptr() + 4), _k._st()

    def _ctr(self, i: int):
        return _c.c_void_p(self.state.data_ptr() + 4 * i)

    def _rpr(self, total_rows: int) -> int:
        rpr = -(-total_rows // self.world)
        if rpr > self.rpr_cap:
            raise ValueError(f"{total_rows} rows exceed the TP staging capacity {self.rpr_cap * self.world}")
        return rpr

    def _stage_slot_bytes(self) -> int:
        return self.rpr_cap * self.H * 2

    # ---- GEMM -> reduce-scatter ----
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, w_scale: Optional[torch.Tensor] = None, add_in=None) -> torch.Tensor:
        """x [T, K_local] @ w[N, K_local]^T summed over the group; returns this rank's rows [ceil(T / world), N]
        (rows past T are zero-padding sums and must be ignored by the caller).  Two launches: the GEMM, whose epilogue stores
        every row into its owner's stage and whose last CTA raises the flags, and the owner-side reduce."""
        lib = _k.lib()
        N, K = w.shape
        assert N == self.H
        rpr = self._rpr(x.shape[0])
        T = self.world * rpr
        if x.shape[0] != T:               # pad to a multiple of the group size: the extra rows produce zeros in their owners' slots
            x = torch.cat([x, x.new_zeros(T - x.shape[0], x.shape[1])], 0)
        L, epoch, ctr, st = self._args()
        hp, Ly = self.heap, self.layout
        cm = _k.GemmComm()
        cm.scatter_mode, cm.scatter_rpr, cm.scatter_epoch = 3, rpr, self.state.data_ptr()
        cm.scatter_parity_bytes = self.world * self._stage_slot_bytes()
        for r in range(self.world):
            cm.scatter_base[r] = hp.peer_ptrs[r] + Ly.off_stage + self.rank * self._stage_slot_bytes()      # my slot in r's stage
            cm.tail_flag[r] = hp.peer_ptrs[r] + Ly.off_flags + 4 * self.rank                               # flags[0][me] at r
        cm.tail_counter, cm.tail_epoch, cm.tail_world = self.state.data_ptr() + 8, self.state.data_ptr(), self.world
        x2 = _k._as_bf16_2d(x)
        dummy = self.state               # D is unused: every row has a destination in some rank's stage
        if w.dtype == FP8:
            q, s = _k.quant_fp8_1x128_raw(x2)
            _k._gemm_comm(q, K, 0, w, dummy, N, 0, T, N, K, 1, None, True, s, T, 0, w_scale, cm)
        else:
            _k._gemm_comm(x2, x2.stride(0), 0, w, dummy, N, 0, T, N, K, 1, None, False, None, 0, 0, None, cm)
        out = torch.empty(rpr, N, dtype=torch.bfloat16, device=x.device)
        _k._ck(lib.ne_tp_reduce(L, _k._p(add_in), _k._p(out), _c.c_int(rpr), epoch, _c.c_int(self.spin_limit), self._ctr(3), st), "ne_tp_reduce")
        return out

    # ---- all-gather -> GEMM ----
    def all_gather_gemm(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """x [rpr, H] on every rank, w [N, H] bf16 -> gathered rows times w^T: [world * rpr, N].  Two launches: the push of this
        rank's rows into every peer's gather buffer, and the GEMM whose producer warp waits (bounded) for the source ranks of
        each row block right before loading it - this rank's own rows first - so the product starts while peers' rows are still
        arriving.  The GEMM's last CTA advances the epoch."""
        lib = _k.lib()
        rpr = x.shape[0]
        N, K = w.shape
        assert K == self.H and x.shape[1] == self.H and 1 <= rpr <= self.rpr_cap and w.dtype == torch.bfloat16
        x = _k._as_bf16_2d(x).contiguous()
        L, epoch, ctr, st = self._args()
        _k._ck(lib.ne_tp_push(L, _k._p(x), _c.c_int(rpr), _c.c_int(rpr), _c.c_int(0), epoch, ctr, st), "ne_tp_push")
        hp, Ly = self.heap, self.layout
        me = hp.peer_ptrs[self.rank]
        cm = _k.GemmComm()
        cm.gate_epoch, cm.gate_flags = self.state.data_ptr(), me + Ly.off_flags + 4 * self.world
        cm.gate_rpr, cm.gate_world, cm.gate_parity_rows, cm.gate_spin = rpr, self.world, self.world * self.rpr_cap, self.spin_limit
        cm.mb_rot = (self.rank * rpr) // 128 if rpr % 128 == 0 else 0
        cm.tail_counter, cm.tail_epoch, cm.tail_world, cm.tail_advance = self.state.data_ptr() + 8, self.state.data_ptr(), 0, self.state.data_ptr()
        T = self.world * rpr
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        _k._gemm_comm(me + Ly.off_gather, self.H, 0, w, out, N, 0, T, N, K, 1, None, False, None, 0, 0, None, cm,
                      a_rows_total=2 * self.world * self.rpr_cap)
        return out

    # ---- plain collectives ----
    def reduce_scatter(self, xp: torch.Tensor) -> torch.Tensor:
        """xp [world * rpr, H] partial sums -> this rank's [rpr, H] of the total."""
        if self.nvls is not None and xp.shape[0] <= self.nvls.rows_cap:
            return self.nvls.reduce_scatter(xp)
        lib = _k.lib()
        rows = xp.shape[0]
        assert rows % self.world == 0 and xp.shape[1] == self.H
        rpr = self._rpr(rows)
        xp = _k._as_bf16_2d(xp).contiguous()
        L, epoch, ctr, st = self._args()
        _k._ck(lib.ne_tp_push(L, _k._p(xp), _c.c_int(rows), _c.c_int(rpr), _c.c_int(1), epoch, ctr, st), "ne_tp_push")
        out = torch.empty(rpr, self.H, dtype=torch.bfloat16, device=xp.device)
        _k._ck(lib.ne_tp_reduce(L, _k._p(None), _k._p(out), _c.c_int(rpr), epoch, _c.c_int(self.spin_limit), self._ctr(3), st), "ne_tp_reduce")
        return out

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """x [rpr, H] on every rank -> [world * rpr, H] in a tensor of its own (copied out of the receive buffer by the
        waiting kernel, so the result does not depend on the parity of the call and stays valid for as long as it is held)."""
        if self.nvls is not None and x.shape[0] * self.world <= self.nvls.rows_cap and x.shape[0] > 0:
            return self.nvls.all_gather(x)
        lib = _k.lib()
        rpr = x.shape[0]
        assert x.shape[1] == self.H and rpr <= self.rpr_cap
        x = _k._as_bf16_2d(x).contiguous()
        L, epoch, ctr, st = self._args()
        _k._ck(lib.ne_tp_push(L, _k._p(x), _c.c_int(rpr), _c.c_int(max(rpr, 1)), _c.c_int(0), epoch, ctr, st), "ne_tp_push")
        out = torch.empty(self.world * rpr, self.H, dtype=torch.bfloat16, device=x.device)
        _k._ck(lib.ne_tp_wait_copy(L, _k._p(out), _c.c_int(self.world * rpr), epoch, _c.c_int(self.spin_limit), self._ctr(3), st), "ne_tp_wait_copy")
        return out

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        if self.nvls is not None and 0 < T <= self.nvls.rows_cap:
            return self.nvls.all_reduce(x)
        if 0 < T <= self.rpr_cap:
            # few rows: every rank stores its partial into every peer's stage and adds the slots itself (one hop)
            lib = _k.lib()
            x = _k._as_bf16_2d(x).contiguous()
            L, epoch, ctr, st = self._args()
            _k._ck(lib.ne_tp_push(L, _k._p(x), _c.c_int(T), _c.c_int(T), _c.c_int(2), epoch, ctr, st), "ne_tp_push")
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=x.device)
            _k._ck(lib.ne_tp_reduce(L, _k._p(None), _k._p(out), _c.c_int(T), epoch, _c.c_int(self.spin_limit), self._ctr(3), st), "ne_tp_reduce")
            return out
        pad = (-T) % self.world
        xp = x if pad == 0 else torch.cat([x, x.new_zeros(pad, x.shape[1])], 0)
        return self.all_gather(self.reduce_scatter(xp))[:T]


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
