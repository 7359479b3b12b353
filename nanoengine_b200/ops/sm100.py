"""CUDA (sm_100a) bodies of the operators: ctypes calls into ``_native/libne_kernels.so``.

Every function mirrors the signature of its namesake in ``ops.reference``.  The library is loaded on first
use and its absence is an error: on a GPU there is no silent PyTorch fallback.  Kernels run on the current
torch stream; scratch buffers come from torch's caching allocator, which keeps the sequence capturable in
CUDA graphs.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import reference as ref

FP8 = torch.float8_e4m3fn
_LIB = None
_c = ctypes


def lib():
    global _LIB
    if _LIB is None:
        # NE_DEBUG_BOUNDS=1 selects the bounds-checked build of the same kernels (python -m nanoengine_b200.build_native --debug-bounds)
        dbg = os.environ.get("NE_DEBUG_BOUNDS", "0") not in ("", "0")
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_native", "libne_kernels_dbg.so" if dbg else "libne_kernels.so")
        if not os.path.exists(path):
            raise RuntimeError(f"CUDA kernel library missing: {path}; run `python -m nanoengine_b200.build_native{' --debug-bounds' if dbg else ''}`")
        _LIB = ctypes.CDLL(path)
    return _LIB


def debug_set_bounds(cache_rows: int = 0, cache_pages: int = 0, state_slots: int = 0, experts: int = 0) -> bool:
    """Register the bounds the bounds-checked build compares table entries with; False (and no effect) in the ordinary build."""
    return bool(lib().ne_debug_set_bounds(_c.c_longlong(cache_rows), _c.c_longlong(cache_pages), _c.c_longlong(state_slots), _c.c_longlong(experts)))


def _p(t: Optional[torch.Tensor]):
    return _c.c_void_p(0 if t is None else t.data_ptr())


def _st():
    return _c.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = [0]          # kernels of this library launched so far (a call that launches several counts them all)
_KERNELS_PER_CALL = {"ne_moe_dispatch_local": 3}


def _ck(rc: int, name: str):
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    LAUNCHES[0] += _KERNELS_PER_CALL.get(name, 1)


def kernel_status():
    """Status words written by a kernel whose bounded wait ran out (all zero = healthy)."""
    buf = (_c.c_int * 8)()
    _ck(lib().ne_get_status(buf), "ne_get_status")
    return list(buf)


def clear_kernel_status():
    _ck(lib().ne_clear_status(), "ne_clear_status")


# ---- scale format ----------------------------------------------------------------------------------
def set_scale_format(fmt: Optional[str]) -> None:
    """"ue8m0": every fp8 quantiser of the library rounds its group scales up to powers of two and the block-scaled GEMMs
    hand them to the tensor cores (tcgen05.mma.kind::mxf8f6f4.block_scale); "fp32" (or None): plain amax / 448 scales, applied
    on the CUDA cores between K blocks.  Weights must have been quantised (or re-quantised: `fp8_block_for_format`) under the
    same setting.  CUDA graphs keep the setting they were captured with."""
    ref.set_scale_format(fmt)
    lib().ne_set_scale_pow2(_c.c_int(1 if ref.SCALE_POW2[0] else 0))


scale_format = ref.scale_format


def _fp8_dtype(fp8) -> int:
    return (2 if ref.SCALE_POW2[0] else 1) if fp8 else 0


TC_SCALED_GEMMS = [0]       # GEMM launches whose block scales the tensor cores applied (more than 128 rows per group, "ue8m0" format)


# ---- GEMM ----------------------------------------------------------------------------------------
def _gemm(A, lda, a_gs, B, D, ldd, d_gs, M, N, K, groups, masked_m, row_start, fp8, sa, sa_ld, sa_gs, sb, out_fp32, bn=0, row_dst=None):
    if fp8 and ref.SCALE_POW2[0] and (M // groups if row_start is not None else M) > 128:
        TC_SCALED_GEMMS[0] += 1
    rc = lib().ne_gemm(_p(A), _c.c_longlong(lda), _c.c_longlong(a_gs), _p(B), _p(D), _c.c_longlong(ldd), _c.c_longlong(d_gs),
                       _c.c_int(M), _c.c_int(N), _c.c_int(K), _c.c_int(groups), _p(masked_m), _p(row_start), _c.c_int(_fp8_dtype(fp8)),
                       _p(sa), _c.c_int(sa_ld), _c.c_longlong(sa_gs), _p(sb), _c.c_int(int(out_fp32)), _c.c_int(bn), _p(row_dst), _st())     # output: 0 bf16, 1 fp32, 2 e4m3
    _ck(rc, "ne_gemm")


class GemmComm(_c.Structure):
    """Mirror of `ne::GemmComm` (csrc/kernels/gemm.cu): the collective hooks of one GEMM launch."""
    _fields_ = [("wait_epoch", _c.c_void_p), ("wait_flags", _c.c_void_p), ("wait_world", _c.c_int), ("wait_spin", _c.c_uint),
                ("gate_epoch", _c.c_void_p), ("gate_flags", _c.c_void_p), ("gate_rpr", _c.c_int), ("gate_world", _c.c_int),
                ("gate_parity_rows", _c.c_int), ("mb_rot", _c.c_int), ("gate_spin", _c.c_uint),
                ("scatter_mode", _c.c_int), ("row_info", _c.c_void_p), ("scatter_base", _c.c_ulonglong * 16), ("scatter_rpr", _c.c_int),
                ("scatter_parity_bytes", _c.c_longlong), ("scatter_epoch", _c.c_void_p),
                ("tail_counter", _c.c_void_p), ("tail_epoch", _c.c_void_p), ("tail_flag", _c.c_ulonglong * 16), ("tail_world", _c.c_int),
                ("tail_clear", _c.c_void_p), ("tail_clear_n", _c.c_int), ("tail_advance", _c.c_void_p)]


def _gemm_comm(A, lda, a_gs, B, D, ldd, d_gs, M, N, K, groups, masked_m, fp8, sa, sa_ld, sa_gs, sb, comm: GemmComm, a_rows_total=0, bn=0,
               few_rows=False):
    """`_gemm` with a fused collective; `masked_m` may be a raw device address (an int) inside a symmetric region.  `few_rows`:
    the groups hold far fewer rows than `M` allows (a decode step through prefill-sized buffers): keep the CUDA-core scaling."""
    l = lib()
    if not getattr(l, "_comm_checked", False):
        assert l.ne_gemm_comm_size() == _c.sizeof(GemmComm), "GemmComm mismatch between Python and the kernel library"
        l._comm_checked = True
    mm = _c.c_void_p(masked_m) if isinstance(masked_m, int) else _p(masked_m)
    rc = l.ne_gemm_comm(_p(A) if not isinstance(A, int) else _c.c_void_p(A), _c.c_longlong(lda), _c.c_longlong(a_gs), _p(B), _p(D), _c.c_longlong(ldd),
                        _c.c_longlong(d_gs), _c.c_int(M), _c.c_int(N), _c.c_int(K), _c.c_int(groups), mm, _p(None), _c.c_int(1 if (fp8 and few_rows) else _fp8_dtype(fp8)),
                        _p(sa) if not isinstance(sa, int) else _c.c_void_p(sa), _c.c_int(sa_ld), _c.c_longlong(sa_gs), _p(sb), _c.c_int(0), _c.c_int(bn),
                        _c.byref(comm), _c.c_int(a_rows_total), _st())
    _ck(rc, "ne_gemm_comm")


def quant_fp8_1x128(x: torch.Tensor, ue8m0: Optional[bool] = None):
    """bf16 [T, K] -> (e4m3 [T, K], scales [T, K/128]).  The kernel writes scales column-major ([K/128, T]);
    the returned view presents them in the reference's [T, K/128] orientation.  The scales follow the process's scale format."""
    assert ue8m0 is None or bool(ue8m0) == ref.SCALE_POW2[0], "the CUDA quantisers follow set_scale_format()"
    T, K = x.shape
    x = x if x.stride(-1) == 1 else x.contiguous()
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = torch.empty(K // 128, T, dtype=torch.float32, device=x.device)
    _ck(lib().ne_quant_1x128(_p(x), _c.c_longlong(x.stride(0)), _p(q), _p(s), _c.c_int(T), _c.c_int(T), _c.c_int(K), _st()), "ne_quant_1x128")
    return q, s.t()


def quant_fp8_1x128_raw(x: torch.Tensor):
    """bf16 [T, K] -> (e4m3 [T, K], scales [K/128, T]) exactly as the block-scaled GEMM reads them."""
    T, K = x.shape
    q = torch.empty(T, K, dtype=FP8, device=x.device)
    s = torch.empty(K // 128, T, dtype=torch.float32, device=x.device)
    _ck(lib().ne_quant_1x128(_p(x), _c.c_longlong(x.stride(0)), _p(q), _p(s), _c.c_int(T), _c.c_int(T), _c.c_int(K), _st()), "ne_quant_1x128")
    return q, s


def _as_bf16_2d(x):
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype != torch.bfloat16:
        x2 = x2.to(torch.bfloat16)
    if x2.stride(-1) != 1 or (x2.stride(0) * 2) % 16 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    return x2


QAct, dense = ref.QAct, ref.dense


class PrequantizedActivation:
    """An activation that exists only in its 1x128 block-quantised form: e4m3 [T, K] and scales [K/128, T], as left by a
    fused producer (SwiGLU + quant).  `linear` with an fp8 weight consumes it directly.
    Parity: reference layers/base_backend.py:14-26."""
    __slots__ = ("q", "scales", "shape", "device")

    def __init__(self, q: torch.Tensor, scales: torch.Tensor):
        self.q, self.scales, self.shape, self.device = q, scales, q.shape, q.device


def linear(x, w: torch.Tensor, w_scale: Optional[torch.Tensor] = None, bias=None, out_fp32: bool = False) -> torch.Tensor:
    N, K = w.shape
    if isinstance(x, PrequantizedActivation):
        assert w.dtype == FP8 and x.shape[-1] == K, "a pre-quantised activation feeds fp8 linears only"
        T = x.shape[0]
        out = torch.empty(T, N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
        if T > 0:
            _gemm(x.q, K, 0, w, out, N, 0, T, N, K, 1, None, None, True, x.scales, T, 0, w_scale, out_fp32)
        return out if bias is None else out + bias
    pre = None
    if isinstance(x, QAct):                   # (e4m3 [T, K], scales [K/128, T]) left by a fused norm + quant kernel
        pre = (x.q, x.scales) if x.q is not None else None
        x = x.x
    x2 = _as_bf16_2d(x)
    T = x2.shape[0]
    out = torch.empty(T, N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
    if T > 0:
        if w.dtype == FP8:
            if pre is not None and pre[0].shape == (T, K):
                q, s = pre
            else:
                q = torch.empty(T, K, dtype=FP8, device=x.device)
                s = torch.empty(K // 128, T, dtype=torch.float32, device=x.device)
                _ck(lib().ne_quant_1x128(_p(x2), _c.c_longlong(x2.stride(0)), _p(q), _p(s), _c.c_int(T), _c.c_int(T), _c.c_int(K), _st()), "ne_quant_1x128")
            _gemm(q, K, 0, w, out, N, 0, T, N, K, 1, None, None, True, s, T, 0, w_scale, out_fp32)
        else:
            assert w.dtype == torch.bfloat16, "CUDA linears take bf16 or fp8 weights"
            _gemm(x2, x2.stride(0), 0, w, out, N, 0, T, N, K, 1, None, None, False, None, 0, 0, None, out_fp32)
    if bias is not None:
        out = out + bias
    return out.view(*x.shape[:-1], N)


def kmajor(w: torch.Tensor) -> torch.Tensor:
    """w [H, A, B] -> bf16 [H, B, A] contiguous: the K-major operand `bmm_absorb` multiplies with.  Owners of a weight build
    this once when the weight is set (and again after an in-place update) and pass it as `wt`."""
    return w.to(torch.bfloat16).transpose(1, 2).contiguous()


def router_logits(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x bf16 [T, H] against the fp32 gate weight [E, H] on CUDA cores (N is far too small for a tensor-core tile).

    Returns partial logits [P, T, E] (the hidden dimension is split into P slices so enough CTAs pull the weight at
    once); `moe_route` adds the planes up, any other consumer calls `.sum(0)`."""
    x2 = _as_bf16_2d(x)
    T, H = x2.shape
    E = w.shape[0]
    assert w.dtype == torch.float32 and w.is_contiguous() and x2.stride(0) == H
    out = torch.empty(lib().ne_router_planes(_c.c_int(H)), T, E, dtype=torch.float32, device=x.device)
    _ck(lib().ne_router_gemv(_p(x2), _p(w), _p(out), _c.c_int(T), _c.c_int(E), _c.c_int(H), _st()), "ne_router_gemv")
    return out


def lm_head(hidden: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return linear(hidden, w, out_fp32=True)


def bmm_absorb(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, wt: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, H, A] (any row/head strides, unit inner stride), w [H, A, B] -> [T, H, B]: a grouped GEMM with one group per head.
    `out` may be a strided view; a one-byte `out` (uint8 / e4m3) makes the epilogue write clamped e4m3 instead of bf16.
    `wt` is `kmajor(w)` kept by the weight's owner; without it the transposed copy is made on every call (nothing is cached
    here: a cache keyed on the weight's address would outlive the weight)."""
    T, H, A = x.shape
    Bd = w.shape[2]
    if wt is None:
        wt = kmajor(w)                                                                     # [H, B, A], K-major
    assert wt.shape == (H, Bd, A) and wt.dtype == torch.bfloat16 and wt.is_contiguous()
    if x.dtype != torch.bfloat16 or x.stride(2) != 1 or (x.stride(0) * 2) % 16 or (x.stride(1) * 2) % 16 or x.data_ptr() % 16:
        x = x.to(torch.bfloat16).contiguous()
    if out is None:
        out = torch.empty(T, H, Bd, dtype=torch.bfloat16, device=x.device)
    es = out.element_size()
    assert es in (1, 2) and out.stride(2) == 1 and (out.stride(0) * es) % 16 == 0 and (out.stride(1) * es) % 16 == 0 and out.data_ptr() % 16 == 0
    if T > 0:
        _gemm(x, x.stride(0), x.stride(1), wt, out, out.stride(0), out.stride(1), T, Bd, A, H, None, None, False, None, 0, 0, None,
              2 if es == 1 else 0)
    return out


# ---- norms / activation ----------------------------------------------------------------------------
def _rmsnorm(x, res_in, w, eps, want_res, quant=False, unit_offset=False):
    T, H = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    res_out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device) if want_res else None
    if res_in is not None:
        res_in = res_in.contiguous()
    q = sc = None
    if quant and H % 128 == 0 and T > 0:
        q = torch.empty(T, H, dtype=FP8, device=x.device)
        sc = torch.empty(H // 128, T, dtype=torch.float32, device=x.device)
    _ck(lib().ne_rmsnorm(_p(x), _c.c_longlong(x.stride(0)), _p(res_in), _p(w), _p(out), _c.c_longlong(H), _p(res_out), _p(q), _p(sc),
                         _c.c_int(T), _c.c_int(T), _c.c_int(H), _c.c_float(eps), _c.c_float(1.0 if unit_offset else 0.0), _st()), "ne_rmsnorm")
    if quant:
        out = QAct(out, q, sc)               # q stays None when the width is not a multiple of 128: the consumer quantises itself
    return out, res_out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, quant: bool = False, unit_offset: bool = False):
    """`quant`: the same kernel also writes the e4m3 1x128 copy for the fp8 linear that consumes the result; both travel in a
    `QAct`."""
    if x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    return _rmsnorm(x, None, w, eps, False, quant, unit_offset)[0]


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], w: torch.Tensor, eps: float, unit_offset: bool = False, quant: bool = False):
    if x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    if residual is None:
        return _rmsnorm(x, None, w, eps, False, quant, unit_offset)[0], x
    return _rmsnorm(x, residual, w, eps, True, quant, unit_offset)


def layernorm(x, w, b, eps):
    """One warp per row of the last dimension."""
    shape = x.shape
    D = shape[-1]
    x2 = x.reshape(-1, D)
    if x2.dtype != torch.bfloat16 or x2.stride(-1) != 1:
        x2 = x2.to(torch.bfloat16).contiguous()
    y = torch.empty(x2.shape[0], D, dtype=torch.bfloat16, device=x.device)
    wb = None if w is None else w.to(torch.bfloat16).contiguous()
    bb = None if b is None else b.to(torch.bfloat16).contiguous()
    _ck(lib().ne_layernorm(_p(x2), _c.c_longlong(x2.stride(0)), _p(wb), _p(bb), _c.c_float(eps), _p(y), _c.c_longlong(x2.shape[0]), _c.c_int(D), _st()),
        "ne_layernorm")
    return y.view(shape).to(x.dtype)


def _act_args(act):
    """(mode, p0, p1) of the gated activation for ne_act_mul; see ops.reference.glu_act."""
    if act is None:
        return _c.c_int(0), _c.c_float(0.0), _c.c_float(0.0)
    if act[0] == "clamp":
        return _c.c_int(1), _c.c_float(float(act[1])), _c.c_float(0.0)
    if act[0] == "situ":
        return _c.c_int(2), _c.c_float(float(act[1])), _c.c_float(float(act[2] or 0.0))
    if act[0] == "gelu_tanh":
        return _c.c_int(3), _c.c_float(1.0), _c.c_float(0.0)
    raise ValueError(f"unknown gated activation {act!r}")


def silu_and_mul(x: torch.Tensor, quant: bool = False, act=None):
    """Gated activation of [gate | up] (SwiGLU unless `act` says otherwise).  `quant`: return only the 1x128 block-quantised
    result (for an fp8 down projection)."""
    T, I2 = x.shape
    I = I2 // 2
    x = x.contiguous()
    if quant and I % 128 == 0 and T > 0:
        q = torch.empty(T, I, dtype=FP8, device=x.device)
        sc = torch.empty(I // 128, T, dtype=torch.float32, device=x.device)
        _ck(lib().ne_act_mul(_p(x), _p(None), _p(q), _p(sc), _c.c_int(T), _c.c_longlong(0), _p(None), _p(None), _c.c_int(1), _c.c_int(T), _c.c_int(I),
                             *_act_args(act), _st()), "ne_act_mul")
        return PrequantizedActivation(q, sc)
    y = torch.empty(T, I, dtype=torch.bfloat16, device=x.device)
    _ck(lib().ne_act_mul(_p(x), _p(y), _p(None), _p(None), _c.c_int(0), _c.c_longlong(0), _p(None), _p(None), _c.c_int(1), _c.c_int(T), _c.c_int(I),
                         *_act_args(act), _st()), "ne_act_mul")
    return y


# ---- rotary / KV ----------------------------------------------------------------------------------
def apply_rope(x: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor, interleaved: bool, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotates `x` (which may be a strided view of a projection output) in place, or into `out` when given."""
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
    y = x if out is None else out
    assert y.dtype == torch.bfloat16 and y.stride(-1) == 1 and y.shape == x.shape
    T, D = x.shape[0], x.shape[-1]
    heads, hs, yhs = (x.shape[1], x.stride(1), y.stride(1)) if x.dim() == 3 else (1, 0, 0)
    pos = positions if positions.dtype == torch.int64 else positions.long()
    _ck(lib().ne_rope(_p(x), _c.c_longlong(x.stride(0)), _c.c_int(hs), _p(y), _c.c_longlong(y.stride(0)), _c.c_int(yhs), _c.c_int(heads),
                      _c.c_int(0), _c.c_int(D), _p(pos), _p(cache), _c.c_int(1 if interleaved else 0), _c.c_int(T), _st()), "ne_rope")
    return y


def mla_absorb_rope(q: torch.Tensor, kc: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor, nope: int, kc_t=None) -> torch.Tensor:
    """Absorbed query of MLA in one buffer: [q_nope @ W_UK | rope(q_pe)] -> [T, H, R + rope], no concatenation pass."""
    T, H, _ = q.shape
    R = kc.shape[2]
    rope = q.shape[2] - nope
    out = torch.empty(T, H, R + rope, dtype=torch.bfloat16, device=q.device)
    if T == 0:
        return out
    bmm_absorb(q[..., :nope], kc, out=out[..., :R], wt=kc_t)
    apply_rope(q[..., nope:], positions, cache, True, out=out[..., R:])
    return out


def mla_query(q: torch.Tensor, kc: torch.Tensor, positions: torch.Tensor, rope_cache: torch.Tensor, nope: int, kv_cache: torch.Tensor,
              dense: bool = True, kc_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Absorbed MLA query.  For the fp8 tensor-core attention kernels, dense or sparse (fp8 cache of 64-token pages, 512 + 64
    wide rows, at most 128 heads) the result is e4m3 [T, H, 576]: the per-head GEMM's epilogue writes the latent part as e4m3 straight into it
    and one small kernel rotates and casts the 64-wide tail, instead of a bf16 latent query, a RoPE pass and a cast pass."""
    T, H, _ = q.shape
    R = kc.shape[2]
    rope = q.shape[2] - nope
    if not (kv_cache.dtype == FP8 and R == 512 and rope == 64 and kv_cache.shape[1] == 64 and H <= 128 and T > 0):      # dense and sparse alike
        return mla_absorb_rope(q, kc, positions, rope_cache, nope, kc_t)
    q8 = torch.empty(T, H, R + rope, dtype=torch.uint8, device=q.device)
    bmm_absorb(q[..., :nope], kc, out=q8[..., :R], wt=kc_t)
    pe = q[..., nope:]
    pos = positions if positions.dtype == torch.int64 else positions.long()
    _ck(lib().ne_mla_q_finalize(_p(None), _p(pe), _c.c_longlong(pe.stride(0)), _c.c_int(pe.stride(1)), _p(pos), _p(rope_cache), _p(q8),
                                _c.c_int(T), _c.c_int(H), _c.c_int(R), _c.c_int(rope), _st()), "ne_mla_q_finalize")
    return q8.view(FP8)


def mla_kv_prepare(kv_a: torch.Tensor, norm_w: torch.Tensor, eps: float, positions: torch.Tensor, rope_cache: torch.Tensor,
                   kv_cache: torch.Tensor, slot_mapping: torch.Tensor, R: int) -> None:
    """RMSNorm of the compressed KV, RoPE of the key tail and the cache write in one kernel (one warp per token)."""
    T = kv_a.shape[0]
    rope = kv_a.shape[1] - R
    fp8 = kv_cache.dtype == FP8
    assert kv_a.dtype == torch.bfloat16 and kv_a.stride(1) == 1 and (fp8 or kv_cache.dtype == torch.bfloat16)
    assert kv_cache.shape[-1] == R + rope and norm_w.dtype == torch.bfloat16
    pos = positions if positions.dtype == torch.int64 else positions.long()
    _ck(lib().ne_mla_kv_prepare(_p(kv_a), _c.c_longlong(kv_a.stride(0)), _p(norm_w), _c.c_float(eps), _p(pos), _p(rope_cache), _p(kv_cache),
                                _p(slot_mapping), _c.c_int(T), _c.c_int(R), _c.c_int(rope), _c.c_int(1 if fp8 else 0), _st()), "ne_mla_kv_prepare")


def mla_kv_store(cache: torch.Tensor, slot_mapping: torch.Tensor, ckv: torch.Tensor, k_pe: torch.Tensor) -> None:
    T, R = ckv.shape
    rope = k_pe.shape[1]
    assert ckv.stride(1) == 1 and k_pe.stride(1) == 1
    fp8 = cache.dtype == FP8
    assert fp8 or cache.dtype == torch.bfloat16
    _ck(lib().ne_mla_kv_store(_p(ckv), _c.c_longlong(ckv.stride(0)), _p(k_pe), _c.c_longlong(k_pe.stride(0)), _p(cache), _p(slot_mapping),
                              _c.c_int(T), _c.c_int(R), _c.c_int(rope), _c.c_int(1 if fp8 else 0), _st()), "ne_mla_kv_store")


def gqa_kv_store(k_cache, v_cache, slot_mapping, k, v):
    """k, v [T, Hkv, D] (row stride free) -> rows `slot_mapping` of the paged caches [blocks, block_size, Hkv, D]."""
    T = k.shape[0]
    row = k.shape[1] * k.shape[2]
    ok = (k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
          and k_cache.is_contiguous() and v_cache.is_contiguous() and row % 8 == 0)
    if not ok:
        raise ValueError("gqa_kv_store: the CUDA path stores bf16 rows of a multiple of 8 elements into contiguous bf16 caches")
    k2, v2 = k.reshape(T, row), v.reshape(T, row)
    if k2.stride(1) != 1 or k2.stride(0) % 8 or k2.data_ptr() % 16:
        k2 = k2.contiguous()
    if v2.stride(1) != 1 or v2.stride(0) % 8 or v2.data_ptr() % 16:
        v2 = v2.contiguous()
    _ck(lib().ne_gqa_kv_store(_p(k2), _p(v2), _c.c_longlong(k2.stride(0)), _c.c_longlong(v2.stride(0)), _p(k_cache), _p(v_cache),
                              _p(_i64c(slot_mapping)), _c.c_int(T), _c.c_int(row), _st()), "ne_gqa_kv_store")


def _i64c(t):
    return t if (t.dtype == torch.int64 and t.is_contiguous()) else t.long().contiguous()


def gqa_qkv_prepare(qkv, hq, hkv, hd, q_norm_w, k_norm_w, eps, unit_offset, positions, rope_cache, k_cache, v_cache, slot_mapping):
    """One kernel for head split, q / k RMSNorm, rotary embedding and the paged K / V store (head dim 128 or 256 with the whole
    head rotated, bf16 caches); other shapes run the same steps as separate kernels."""
    T = qkv.shape[0]
    fused = (hd in (128, 256) and rope_cache.shape[1] == hd and qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.stride(0) % 2 == 0
             and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
             and rope_cache.dtype == torch.float32 and rope_cache.is_contiguous())
    if not fused:
        q, k, v = qkv.split([hq * hd, hkv * hd, hkv * hd], -1)
        q, k, v = q.reshape(T, hq, hd), k.reshape(T, hkv, hd), v.reshape(T, hkv, hd)
        if q_norm_w is not None:
            q = rmsnorm(q.reshape(-1, hd), q_norm_w, eps, False, unit_offset).view(T, hq, hd)
        if k_norm_w is not None:
            k = rmsnorm(k.reshape(-1, hd), k_norm_w, eps, False, unit_offset).view(T, hkv, hd)
        q = apply_rope(q.contiguous(), positions, rope_cache, False)
        k = apply_rope(k.contiguous(), positions, rope_cache, False)
        gqa_kv_store(k_cache, v_cache, slot_mapping, k, v.contiguous())
        return q
    q = torch.empty(T, hq, hd, dtype=torch.bfloat16, device=qkv.device)
    qw = None if q_norm_w is None else q_norm_w.to(torch.bfloat16).contiguous()
    kw = None if k_norm_w is None else k_norm_w.to(torch.bfloat16).contiguous()
    _ck(lib().ne_gqa_qkv_prepare(_p(qkv), _c.c_longlong(qkv.stride(0)), _c.c_int(hq), _c.c_int(hkv), _c.c_int(hd), _p(qw), _p(kw), _c.c_float(eps),
                                 _c.c_float(1.0 if unit_offset else 0.0), _p(_i64c(positions)), _p(rope_cache), _p(q), _p(k_cache), _p(v_cache),
                                 _p(_i64c(slot_mapping)), _c.c_int(T), _st()), "ne_gqa_qkv_prepare")
    return q


# ---- MoE -----------------------------------------------------------------------------------------
def moe_route(logits, bias, top_k, n_group=1, topk_group=1, norm_topk_prob=True, routed_scaling_factor=1.0, scoring="sigmoid",
              balance_ranks: int = 0, log2phy: Optional[torch.Tensor] = None, logcnt: Optional[torch.Tensor] = None):
    """`balance_ranks`, `log2phy` / `logcnt` (int32 device tables [E, R] / [E]): see `reference.moe_route`."""
    planes = logits.shape[0] if logits.dim() == 3 else 1
    T, E = logits.shape[-2:]
    logits = logits.float().contiguous()
    idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    if log2phy is not None:
        assert log2phy.dtype == torch.int32 and logcnt.dtype == torch.int32 and log2phy.is_contiguous() and log2phy.shape[0] == E
    _ck(lib().ne_moe_route(_p(logits), _p(bias), _p(idx), _p(w), _c.c_int(T), _c.c_int(E), _c.c_int(top_k), _c.c_int(n_group), _c.c_int(topk_group),
                           _c.c_int(1 if norm_topk_prob else 0), _c.c_float(routed_scaling_factor), _c.c_int({"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}[scoring]),
                           _c.c_int(planes), _c.c_int(balance_ranks), _p(log2phy), _p(logcnt), _c.c_int(0 if log2phy is None else log2phy.shape[1]), _st()),
        "ne_moe_route")
    return idx, w


def moe_experts(x, topk_idx, topk_w, w13, w2, w13_scale=None, w2_scale=None, expert_offset: int = 0, add_in=None, act=None) -> torch.Tensor:
    """Local routed experts over an expert-major, 128-row-aligned layout: scatter (+fp8 quant) -> grouped GEMM ->
    SwiGLU (+requant) -> grouped GEMM -> weighted gather.  `add_in` (e.g. the shared-expert output) is summed in the gather."""
    T, H = x.shape
    E, I2, _ = w13.shape
    I = I2 // 2
    K = topk_idx.shape[1]
    dev = x.device
    fp8 = w13.dtype == FP8
    x = _as_bf16_2d(x)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    if T == 0:
        return out
    R = T * K + E * 127
    R = (R + 127) // 128 * 128
    meta = torch.empty(E + (E + 1) + 2 * T * K, dtype=torch.int32, device=dev)      # every entry is written by the dispatch kernels
    counts, row_start = meta[:E], meta[E:2 * E + 1]
    slot, pos = meta[2 * E + 1:2 * E + 1 + T * K], meta[2 * E + 1 + T * K:]
    idx = topk_idx.to(torch.int32).contiguous()
    w = topk_w.float().contiguous()
    if fp8:
        a_q = torch.empty(R, H, dtype=FP8, device=dev)
        a_s = torch.empty(H // 128, R, dtype=torch.float32, device=dev)
        a_b = None
    else:
        a_b = torch.empty(R, H, dtype=torch.bfloat16, device=dev)
        a_q = a_s = None
    _ck(lib().ne_moe_dispatch_local(_p(x), _p(idx), _p(counts), _p(slot), _p(row_start), _p(pos), _p(a_b), _p(a_q), _p(a_s), _c.c_int(R),
                                    _c.c_int(T), _c.c_int(K), _c.c_int(H), _c.c_int(expert_offset), _c.c_int(E), _c.c_int(R), _c.c_int(128), _st()),
        "ne_moe_dispatch_local")
    g = torch.empty(R, I2, dtype=torch.bfloat16, device=dev)
    y = torch.empty(R, H, dtype=torch.bfloat16, device=dev)
    if fp8:
        _gemm(a_q, H, 0, w13, g, I2, 0, R, I2, H, E, counts, row_start, True, a_s, R, 0, w13_scale, False)
        h_q = torch.empty(R, I, dtype=FP8, device=dev)
        h_s = torch.empty(I // 128, R, dtype=torch.float32, device=dev)
        _ck(lib().ne_act_mul(_p(g), _p(None), _p(h_q), _p(h_s), _c.c_int(R), _c.c_longlong(0), _p(counts), _p(row_start), _c.c_int(E), _c.c_int(R), _c.c_int(I),
                             *_act_args(act), _st()), "ne_act_mul")
        _gemm(h_q, I, 0, w2, y, H, 0, R, H, I, E, counts, row_start, True, h_s, R, 0, w2_scale, False)
    else:
        _gemm(a_b, H, 0, w13, g, I2, 0, R, I2, H, E, counts, row_start, False, None, 0, 0, None, False)
        h = torch.empty(R, I, dtype=torch.bfloat16, device=dev)
        _ck(lib().ne_act_mul(_p(g), _p(h), _p(None), _p(None), _c.c_int(0), _c.c_longlong(0), _p(counts), _p(row_start), _c.c_int(E), _c.c_int(R), _c.c_int(I),
                             *_act_args(act), _st()), "ne_act_mul")
        _gemm(h, I, 0, w2, y, H, 0, R, H, I, E, counts, row_start, False, None, 0, 0, None, False)
    if callable(add_in):
        add_in = add_in()          # produced on another stream: the callable joins that stream as late as possible
    _ck(lib().ne_moe_combine_local(_p(y), _p(pos), _p(w), _p(add_in), _p(out), _c.c_int(T), _c.c_int(K), _c.c_int(H), _st()), "ne_moe_combine_local")
    return out


# ---- NVFP4 -------------------------------------------------------------------------------------------------------
nvfp4_unpack, nvfp4_quant_weight = ref.nvfp4_unpack, ref.nvfp4_quant_weight


def _nvfp4_quant_raw(x, gscale, row_start, counts, groups):
    R, K = x.shape
    q = torch.empty(R, K // 2, dtype=torch.uint8, device=x.device)
    sf = torch.zeros(R, K // 16, dtype=FP8, device=x.device) if row_start is not None else torch.empty(R, K // 16, dtype=FP8, device=x.device)
    _ck(lib().ne_nvfp4_quant(_p(x), _c.c_longlong(x.stride(0)), _p(q), _p(sf), _p(gscale), _p(row_start), _p(counts), _c.c_int(groups), _c.c_int(R),
                             _c.c_int(K), _st()), "ne_nvfp4_quant")
    return q, sf


def nvfp4_quant(x: torch.Tensor, gscale: torch.Tensor, row_group: Optional[torch.Tensor] = None):
    """bf16 [R, K] -> (packed e2m1 [R, K/2], e4m3 scales [R, K/16]); see the reference body.  `row_group` must be sorted (rows of a
    group adjacent), as the grouped layouts are."""
    x = _as_bf16_2d(x)
    g = gscale.float().reshape(-1).contiguous()
    if row_group is None:
        return _nvfp4_quant_raw(x, g, None, None, 1)
    G = g.numel()
    counts = torch.bincount(row_group.long(), minlength=G).to(torch.int32)
    row_start = (counts.cumsum(0) - counts).to(torch.int32)
    return _nvfp4_quant_raw(x, g, row_start, counts, G)


def nvfp4_gemm(a_q, a_sf, b_q, b_sf, alpha, masked_m=None, row_start=None, out_fp32: bool = False) -> torch.Tensor:
    """NVFP4 grouped GEMM on the tensor cores (tcgen05.mma.kind::mxf4nvf4.block_scale); layouts as the reference body."""
    G, N, K2 = b_q.shape
    R = a_q.shape[0]
    assert a_q.shape[1] == K2 and a_q.is_contiguous() and b_q.is_contiguous() and a_sf.is_contiguous() and b_sf.is_contiguous()
    out = torch.zeros(R, N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=a_q.device)
    if G > 1:
        assert row_start is not None and masked_m is not None, "several groups: the contiguous grouped layout"
    al = None if alpha is None else alpha.float().reshape(-1).contiguous()
    _ck(lib().ne_gemm_nvfp4(_p(a_q), _p(b_q), _p(out), _c.c_longlong(N), _c.c_int(R), _c.c_int(N), _c.c_int(K2 * 2), _c.c_int(G),
                            _p(None if masked_m is None else masked_m.to(torch.int32)), _p(None if row_start is None else row_start.to(torch.int32)),
                            _p(a_sf), _p(b_sf), _p(al), _c.c_int(1 if out_fp32 else 0), _st()), "ne_gemm_nvfp4")
    return out


def moe_experts_nvfp4(x, topk_idx, topk_w, w13_q, w13_sf, alpha1, a1_gscale, w2_q, w2_sf, alpha2, a2_gscale, expert_offset: int = 0,
                      add_in=None, act=None) -> torch.Tensor:
    """Local routed experts, W4A4: dispatch into the contiguous grouped layout, quantise, NVFP4 GEMM, gated activation, quantise with
    the expert's own scale, NVFP4 GEMM, weighted combine."""
    T, H = x.shape
    E, I2 = w13_q.shape[0], w13_q.shape[1]
    I = I2 // 2
    K = topk_idx.shape[1]
    dev = x.device
    x = _as_bf16_2d(x)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    if T == 0:
        return out
    R = (T * K + E * 127 + 127) // 128 * 128
    meta = torch.empty(E + (E + 1) + 2 * T * K, dtype=torch.int32, device=dev)
    counts, row_start = meta[:E], meta[E:2 * E + 1]
    slot, pos = meta[2 * E + 1:2 * E + 1 + T * K], meta[2 * E + 1 + T * K:]
    idx = topk_idx.to(torch.int32).contiguous()
    w = topk_w.float().contiguous()
    a_b = torch.empty(R, H, dtype=torch.bfloat16, device=dev)
    _ck(lib().ne_moe_dispatch_local(_p(x), _p(idx), _p(counts), _p(slot), _p(row_start), _p(pos), _p(a_b), _p(None), _p(None), _c.c_int(R),
                                    _c.c_int(T), _c.c_int(K), _c.c_int(H), _c.c_int(expert_offset), _c.c_int(E), _c.c_int(R), _c.c_int(128), _st()),
        "ne_moe_dispatch_local")
    g1 = a1_gscale.float().reshape(-1)[:1].expand(E).contiguous()
    aq, asf = _nvfp4_quant_raw(a_b, g1, row_start, counts, E)
    g = nvfp4_gemm(aq, asf, w13_q, w13_sf, alpha1, counts, row_start)
    h = torch.empty(R, I, dtype=torch.bfloat16, device=dev)
    _ck(lib().ne_act_mul(_p(g), _p(h), _p(None), _p(None), _c.c_int(0), _c.c_longlong(0), _p(counts), _p(row_start), _c.c_int(E), _c.c_int(R), _c.c_int(I),
                         *_act_args(act), _st()), "ne_act_mul")
    hq, hsf = _nvfp4_quant_raw(h, a2_gscale.float().reshape(-1).contiguous(), row_start, counts, E)
    y = nvfp4_gemm(hq, hsf, w2_q, w2_sf, alpha2, counts, row_start)
    if callable(add_in):
        add_in = add_in()
    _ck(lib().ne_moe_combine_local(_p(y), _p(pos), _p(w), _p(add_in), _p(out), _c.c_int(T), _c.c_int(K), _c.c_int(H), _st()), "ne_moe_combine_local")
    return out


# ---- attention / sampling: filled in by the dedicated kernel modules ---------------------------------
def mla_attention_paged(q, cache, block_tables, cu_seqlens_q, context_lens, scale, kv_lora_rank, sparse_indices=None):
    from . import sm100_attn
    return sm100_attn.mla_attention_paged(q, cache, block_tables, cu_seqlens_q, context_lens, scale, kv_lora_rank, sparse_indices)


def attention_varlen(q, k, v, cu_seqlens, scale, causal: bool = False):
    from . import sm100_attn
    return sm100_attn.attention_varlen(q, k, v, cu_seqlens, scale, causal)


def mla_prefill_ragged(q: torch.Tensor, k_nope: torch.Tensor, k_rope: torch.Tensor, v: torch.Tensor, cu_seqlens, scale: float) -> torch.Tensor:
    """Non-absorbed MLA prefill attention on the tcgen05 kernel (128-query tiles per head, 64-key tiles fetched by token
    coordinate, the shared rotary key part through its own tensor map): head dims 128 + 64 / 128 only."""
    T, H, D = q.shape
    assert D == 192 and k_nope.shape == (T, H, 128) and v.shape == (T, H, 128) and k_rope.shape == (T, 64)
    for t in (q, k_nope, k_rope, v):
        assert t.dtype == torch.bfloat16 and t.stride(-1) == 1
    assert q.stride(1) == 192 and k_nope.is_contiguous() and v.is_contiguous() and q.data_ptr() % 16 == 0 and k_rope.data_ptr() % 16 == 0
    cu = cu_seqlens if isinstance(cu_seqlens, torch.Tensor) else torch.tensor(list(cu_seqlens), dtype=torch.int32)
    cu = cu.to(q.device, torch.int32)
    lens = (cu[1:] - cu[:-1]).contiguous()
    B = lens.numel()
    out = torch.empty(T, H, 128, dtype=torch.bfloat16, device=q.device)
    _ck(lib().ne_mla_prefill_bf16(_p(q), _c.c_longlong(q.stride(0)), _p(k_nope), _p(k_rope), _c.c_longlong(k_rope.stride(0)), _p(v), _p(cu), _p(lens),
                                  _c.c_int(B), _c.c_int(T), _c.c_int(H), _c.c_int(T // 128 + B), _c.c_float(scale), _p(out), _st()),
        "ne_mla_prefill_bf16")
    return out


def gelu(x: torch.Tensor, tanh: bool = True) -> torch.Tensor:
    """GELU (tanh approximation or exact) over a contiguous bf16 tensor."""
    x = x.contiguous()
    assert x.dtype == torch.bfloat16
    y = torch.empty_like(x)
    _ck(lib().ne_gelu(_p(x), _p(y), _c.c_longlong(x.numel()), _c.c_int(1 if tanh else 0), _st()), "ne_gelu")
    return y


def gqa_attention_paged(q, k_cache, v_cache, block_tables, cu_seqlens_q, context_lens, scale, window: int = 0):
    from . import sm100_attn
    return sm100_attn.gqa_attention_paged(q, k_cache, v_cache, block_tables, cu_seqlens_q, context_lens, scale, window)


def sample(logits, temperatures, generator=None, return_logprobs=False):
    from . import sm100_attn
    return sm100_attn.sample(logits, temperatures, generator, return_logprobs)


def dequant_fp8_block(q, s, block=128):
    return ref.dequant_fp8_block(q, s, block)


def quant_fp8_block(w, block=128, ue8m0=None):
    return ref.quant_fp8_block(w, block, ue8m0)


fp8_block_for_format = ref.fp8_block_for_format


def merge_attention_states(o1, lse1, o2, lse2):
    """o1, o2 [..., D] bf16 partial attention outputs with their log-sum-exp values [...]; one CTA per row."""
    D = o1.shape[-1]
    a = o1.reshape(-1, D).to(torch.bfloat16).contiguous()
    b = o2.reshape(-1, D).to(torch.bfloat16).contiguous()
    l1, l2 = lse1.reshape(-1).float().contiguous(), lse2.reshape(-1).float().contiguous()
    out = torch.empty_like(a)
    lse = torch.empty_like(l1)
    _ck(lib().ne_merge_states(_p(a), _p(l1), _p(b), _p(l2), _p(out), _p(lse), _c.c_longlong(a.shape[0]), _c.c_int(D), _st()), "ne_merge_states")
    return out.view(o1.shape).to(o1.dtype), lse.view(lse1.shape)


# ---- DSA lightning indexer --------------------------------------------------------------------------
hadamard = ref.hadamard                                     # building blocks of the oracle; the fused kernels below are what runs
quant_fp8_per_token_pow2 = ref.quant_fp8_per_token_pow2
indexer_logits = ref.indexer_logits
indexer_topk = ref.indexer_topk
logical_to_physical = ref.logical_to_physical
indexer_gather = ref.indexer_gather


def _i64(t):
    return t if t.dtype == torch.int64 else t.long()


def indexer_k_store(k, ln_w, ln_b, eps, positions, rope_cache, rope_dim, cache, slots) -> None:
    T, D = k.shape
    assert D == 128 and k.dtype == torch.bfloat16 and k.stride(1) == 1 and cache.dtype == torch.uint8 and cache.is_contiguous()
    bs = cache.shape[1] // (D + 4)
    _ck(lib().ne_indexer_prep(_p(k), _c.c_longlong(k.stride(0)), _c.c_int(T), _c.c_int(1), _p(ln_w), _p(ln_b), _c.c_float(eps), _p(_i64(positions)),
                              _p(rope_cache), _c.c_int(rope_dim), _p(None), _p(None), _p(cache), _p(_i64(slots)), _c.c_int(bs),
                              _c.c_longlong(cache.shape[1]), _st()), "ne_indexer_prep")


def indexer_q_prep(q, positions, rope_cache, rope_dim):
    T, Hi, D = q.shape
    assert D == 128
    q = q if (q.dtype == torch.bfloat16 and q.is_contiguous()) else q.to(torch.bfloat16).contiguous()
    q8 = torch.empty(T, Hi, D, dtype=torch.uint8, device=q.device)
    qs = torch.empty(T, Hi, dtype=torch.float32, device=q.device)
    _ck(lib().ne_indexer_prep(_p(q), _c.c_longlong(D), _c.c_int(T * Hi), _c.c_int(Hi), _p(None), _p(None), _c.c_float(0.0), _p(_i64(positions)),
                              _p(rope_cache), _c.c_int(rope_dim), _p(q8), _p(qs), _p(None), _p(None), _c.c_int(1), _c.c_longlong(0), _st()),
        "ne_indexer_prep")
    return q8.view(FP8), qs


INDEXER_LOGITS_BYTES = 1 << 30          # query tokens are processed in chunks whose logits fit this budget


def indexer_select(q8, q_scale, head_w, cache, block_tables, cu_seqlens_q, context_lens, topk: int, logical: bool = False) -> torch.Tensor:
    """fp8 logits on the tensor cores (one CTA per token and key split) followed by the radix top-k with page translation
    (`logical`: no translation, the list holds key positions)."""
    T, Hi, D = q8.shape
    dev = q8.device
    bs = cache.shape[1] // (D + 4)
    assert D == 128 and bs == 64 and Hi <= 64, "the indexer kernels take 128-wide heads, 64-key pages and at most 64 heads"
    cu = cu_seqlens_q if isinstance(cu_seqlens_q, torch.Tensor) else torch.tensor(list(cu_seqlens_q), dtype=torch.int32)
    cl = context_lens if isinstance(context_lens, torch.Tensor) else torch.tensor(list(context_lens), dtype=torch.int32)
    cu, cl = cu.to(dev, torch.int32), cl.to(dev, torch.int32)
    bt = block_tables.to(torch.int32).contiguous()
    B = cl.numel()
    ld = (bt.shape[1] * bs + 127) // 128 * 128
    out = torch.empty(T, topk, dtype=torch.int32, device=dev)
    w = head_w.float().contiguous()
    qs = q_scale.float().contiguous()
    q8c = q8.contiguous()
    chunk = max(1, min(T, INDEXER_LOGITS_BYTES // (ld * 4)))
    logits = torch.empty(chunk, ld, dtype=torch.float32, device=dev)
    l = lib()
    for t0 in range(0, T, chunk):
        n = min(chunk, T - t0)
        # the kernels find a token's sequence from cu_seqlens_q, so a chunk sees the table shifted by its first token
        cu_c = (cu - t0).clamp_(min=-(1 << 30))
        splits = max(1, min(16, 148 // max(n, 1)))
        _ck(l.ne_indexer_logits(_c.c_void_p(q8c.data_ptr() + t0 * Hi * D), _c.c_void_p(qs.data_ptr() + t0 * Hi * 4), _c.c_void_p(w.data_ptr() + t0 * Hi * 4),
                                _p(cache), _c.c_int(cache.shape[0]), _c.c_longlong(cache.shape[1]), _p(bt), _c.c_int(bt.stride(0)), _p(cu_c), _p(cl),
                                _c.c_int(B), _c.c_int(n), _c.c_int(Hi), _c.c_int(splits), _p(logits), _c.c_longlong(ld), _st()), "ne_indexer_logits")
        _ck(l.ne_indexer_topk(_p(logits), _c.c_longlong(ld), _p(cu_c), _p(cl), _c.c_int(B), _p(None if logical else bt), _c.c_int(bt.stride(0)), _c.c_int(bs),
                              _c.c_int(topk), _c.c_int(n), _c.c_void_p(out.data_ptr() + t0 * topk * 4), _st()), "ne_indexer_topk")
    return out
dequant_fp8_1x128 = ref.dequant_fp8_1x128


# ---- hot / cold tier of the sparse-attention cache ---------------------------------------------------------------------------
def hisparse_stage(L: dict, sel: torch.Tensor, slots: torch.Tensor, context_lens: torch.Tensor, block_tables: torch.Tensor):
    """One kernel, one CTA per sequence: stamps the resident positions, picks victims in ring order, copies the missing rows
    from the cold pages (pinned host memory, read through the unified address space) and emits hot row ids."""
    B, topk = sel.shape
    hot, cold = L["hot"], L["cold"]
    assert sel.dtype == torch.int32 and sel.is_contiguous() and hot.is_cuda and hot.is_contiguous() and cold.is_contiguous()
    assert cold.is_pinned() or cold.is_cuda, "the cold pages must be pinned host memory (or device memory)"
    bt = block_tables if (block_tables.dtype == torch.int32 and block_tables.stride(1) == 1) else block_tables.int().contiguous()
    out = torch.empty(B, topk, dtype=torch.int32, device=sel.device)
    new_slot = torch.empty(B, dtype=torch.int64, device=sel.device)
    _ck(lib().ne_hisparse_stage(_p(L["pos_to_hot"]), _p(L["hot_to_pos"]), _p(L["stamp"]), _p(L["cursor"]), _p(L["step"]), _c.c_void_p(cold.data_ptr()),
                                _p(hot), _p(sel), _c.c_int(topk), _p(_i32(slots)), _p(_i32(context_lens)), _p(bt), _c.c_int(bt.stride(0)), _p(out),
                                _p(new_slot), _c.c_int(L["pos_to_hot"].shape[1]), _c.c_int(L["hot_to_pos"].shape[1]), _c.c_int(hot.shape[1]),
                                _c.c_int(L["page_rows"]), _c.c_int(B), _st()), "ne_hisparse_stage")
    return out, new_slot


def hisparse_writeback(hot: torch.Tensor, cold: torch.Tensor, new_slot: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    _ck(lib().ne_hisparse_writeback(_p(hot), _c.c_void_p(cold.data_ptr()), _p(new_slot), _p(_i64c(slot_mapping)), _c.c_int(hot.shape[1]),
                                    _c.c_int(new_slot.numel()), _st()), "ne_hisparse_writeback")


# ---- gated delta-net linear attention ---------------------------------------------------------------
def _i32(t):
    return t if t.dtype == torch.int32 else t.int()


def gdn_conv(x: torch.Tensor, weight: torch.Tensor, conv_state: torch.Tensor, slots: torch.Tensor, cu_seqlens: torch.Tensor,
             fresh: torch.Tensor, uniform_one: bool = False) -> torch.Tensor:
    """Causal depthwise convolution + SiLU with the carried window updated in place.  `uniform_one`: every sequence
    contributes exactly one token, so the window shift is done by the same kernel."""
    T, C = x.shape
    K = weight.shape[1]
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
    assert conv_state.dtype == torch.bfloat16 and conv_state.is_contiguous() and conv_state.shape[1:] == (K - 1, C)
    y = torch.empty(T, C, dtype=torch.bfloat16, device=x.device)
    B = cu_seqlens.numel() - 1
    _ck(lib().ne_gdn_conv(_p(x), _c.c_longlong(x.stride(0)), _p(weight), _p(conv_state), _p(_i32(slots)), _p(_i32(cu_seqlens)), _p(_i32(fresh)),
                          _p(y), _c.c_longlong(C), _c.c_int(T), _c.c_int(B), _c.c_int(C), _c.c_int(K), _c.c_int(1 if uniform_one else 0), _st()),
        "ne_gdn_conv")
    if not uniform_one:
        LAUNCHES[0] += 1
    return y


def rmsnorm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
                  sigmoid: bool = False) -> torch.Tensor:
    """w * rmsnorm(x) * silu(z) per head; x [T, H, D] fp32, z [T, H, D] bf16 (rows may be strided).  `sigmoid`: the gate is
    sigmoid(z) and the whole product is taken in fp32 (the output norm of Kimi delta attention)."""
    T, H, D = x.shape
    x = x.float().contiguous()
    assert z.dtype == torch.bfloat16 and z.stride(2) == 1 and z.stride(1) == D and w.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(T, H, D, dtype=torch.bfloat16, device=x.device)
    assert out.stride(2) == 1 and out.stride(1) == D
    _ck(lib().ne_rmsnorm_gated(_p(x), _p(z), _c.c_longlong(z.stride(0)), _p(w), _c.c_float(eps), _p(out), _c.c_longlong(out.stride(0)),
                               _c.c_longlong(T), _c.c_int(H), _c.c_int(D), _c.c_int(1 if sigmoid else 0), _st()), "ne_rmsnorm_gated")
    return out


def gdn_recurrent(q, k, v, a, b, A_log, dt_bias, state, slots, cu_seqlens, fresh, z, norm_w, eps: float, max_q_len: int = 1,
                  cu_host=None) -> torch.Tensor:
    """Gated delta rule + gated RMSNorm.  Sequences shorter than `ref.GDN_CHUNK_MIN_TOKENS` new tokens (decode, verification,
    short chunks) run in the recurrent kernel that keeps the state in registers; longer ones take the chunked form, whose
    work is batched matrix products, and need the host copy of the sequence boundaries (`cu_host`)."""
    T, Hk, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    for t in (q, k, v, z):
        assert t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == t.shape[2]
    assert q.stride(0) == k.stride(0) and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(0) == b.stride(0)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (Hv, Dv, Dk)
    assert A_log.dtype == torch.float32 and dt_bias.dtype == torch.float32 and norm_w.dtype == torch.bfloat16
    out = torch.empty(T, Hv, Dv, dtype=torch.bfloat16, device=q.device)
    slots, cu, fresh = _i32(slots), _i32(cu_seqlens), _i32(fresh)
    skip = 1 << 30
    if max_q_len >= ref.GDN_CHUNK_MIN_TOKENS:
        assert cu_host is not None, "the chunked prefill form needs the sequence boundaries on the host"
        skip = ref.GDN_CHUNK_MIN_TOKENS
        rep = Hv // Hk
        g, beta = ref.gdn_gates(a, b, A_log, dt_bias)
        for i in range(len(cu_host) - 1):
            s, e = cu_host[i], cu_host[i + 1]
            if e - s < skip:
                continue
            qn = ref._l2norm(q[s:e].float()).repeat_interleave(rep, 1) * (Dk ** -0.5)
            kn = ref._l2norm(k[s:e].float()).repeat_interleave(rep, 1)
            sl = slots[i: i + 1].long()
            S0 = state.index_select(0, sl)[0] * (1 - fresh[i]).float()
            o, S = ref.gdn_chunked(qn, kn, v[s:e].float(), g[s:e], beta[s:e], S0)
            state.index_copy_(0, sl, S[None])
            rmsnorm_gated(o, z[s:e], norm_w, eps, out[s:e])
    raw = bool(lib().ne_gdn_step_raw_only(_c.c_int(Dk), _c.c_int(Dv)))     # large states: several CTAs per head, norm in its own kernel
    if raw and max_q_len >= ref.GDN_CHUNK_MIN_TOKENS:
        # rows of the long sequences were already normalised into `out`; the recurrent kernel's raw rows go to their own buffer
        dst = torch.zeros(T, Hv, Dv, dtype=torch.float32, device=q.device)
    else:
        dst = torch.empty(T, Hv, Dv, dtype=torch.float32, device=q.device) if raw else out
    _ck(lib().ne_gdn_step(_p(q), _p(k), _p(v), _c.c_longlong(q.stride(0)), _c.c_longlong(v.stride(0)), _p(a), _p(b), _c.c_longlong(a.stride(0)),
                          _p(A_log), _p(dt_bias), _p(state), _p(slots), _p(cu), _p(fresh), _p(z), _c.c_longlong(z.stride(0)), _p(norm_w),
                          _c.c_float(eps), _p(dst), _c.c_longlong(dst.stride(0)), _c.c_int(cu.numel() - 1), _c.c_int(Hk), _c.c_int(Hv), _c.c_int(Dk),
                          _c.c_int(Dv), _c.c_int(skip), _c.c_int(1 if raw else 0), _c.c_int(0), _c.c_float(0.0), _st()), "ne_gdn_step")
    if raw:
        if max_q_len >= ref.GDN_CHUNK_MIN_TOKENS:
            short = torch.ones(T, dtype=torch.bool, device=q.device)
            for i in range(len(cu_host) - 1):
                if cu_host[i + 1] - cu_host[i] >= skip:
                    short[cu_host[i]: cu_host[i + 1]] = False
            normed = rmsnorm_gated(dst, z, norm_w, eps)
            out[short] = normed[short]
        else:
            rmsnorm_gated(dst, z, norm_w, eps, out)
    return out.view(T, Hv * Dv)


def kda_recurrent(q, k, v, raw_g, b, A_log, dt_bias, lower_bound, state, slots, cu_seqlens, fresh, gate, norm_w, eps: float) -> torch.Tensor:
    """Kimi delta attention: the delta rule with a log-decay per key channel, then the sigmoid-gated RMSNorm.  Every sequence,
    prompt chunks included, runs token by token in the kernel that keeps the 128 x 128 state in registers."""
    T, H, Dk = q.shape
    Dv = v.shape[2]
    assert Dk == 128 and Dv == 128 and k.shape == q.shape and v.shape[1] == H, "the CUDA form covers 128 x 128 states"
    for t in (q, k, v, gate):
        assert t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == t.shape[2]
    raw_g = raw_g.reshape(T, H * Dk)
    assert q.stride(0) == k.stride(0) and raw_g.dtype == torch.bfloat16 and raw_g.is_contiguous() and b.dtype == torch.bfloat16 and b.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, Dv, Dk)
    assert A_log.dtype == torch.float32 and dt_bias.dtype == torch.float32 and dt_bias.numel() == H * Dk and norm_w.dtype == torch.bfloat16
    slots, cu, fresh = _i32(slots), _i32(cu_seqlens), _i32(fresh)
    raw = torch.empty(T, H, Dv, dtype=torch.float32, device=q.device)
    _ck(lib().ne_gdn_step(_p(q), _p(k), _p(v), _c.c_longlong(q.stride(0)), _c.c_longlong(v.stride(0)), _p(raw_g), _p(b), _c.c_longlong(b.stride(0)),
                          _p(A_log), _p(dt_bias), _p(state), _p(slots), _p(cu), _p(fresh), _p(gate), _c.c_longlong(gate.stride(0)), _p(norm_w),
                          _c.c_float(eps), _p(raw), _c.c_longlong(raw.stride(0)), _c.c_int(cu.numel() - 1), _c.c_int(H), _c.c_int(H), _c.c_int(Dk),
                          _c.c_int(Dv), _c.c_int(1 << 30), _c.c_int(1), _c.c_int(1), _c.c_float(float(lower_bound) if lower_bound is not None else 0.0),
                          _st()), "ne_gdn_step")
    w = norm_w.expand(Dv) if norm_w.numel() == Dv else norm_w
    return rmsnorm_gated(raw, gate, w.contiguous(), eps, sigmoid=True).view(T, H * Dv)


def sigmoid_mul(o: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """o * sigmoid(g) over rows [T, W]; g may have a row stride."""
    T, W = o.shape
    o = o.contiguous()
    assert o.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and g.shape == o.shape and g.stride(1) == 1
    out = torch.empty_like(o)
    _ck(lib().ne_sigmoid_mul(_p(o), _p(g), _c.c_longlong(g.stride(0)), _p(out), _c.c_longlong(T), _c.c_int(W), _st()), "ne_sigmoid_mul")
    return out


def attn_res_mix(prefix: torch.Tensor, bank: torch.Tensor, valid: int, w_score: torch.Tensor, w_out: torch.Tensor, eps: float,
                 write_row: int = -1) -> torch.Tensor:
    """Block attention residual: softmax mixture of the first `valid` bank rows and the running prefix, then RMSNorm; one
    kernel, one CTA per token.  `write_row` >= 0 also stores the prefix into that bank row."""
    T, D = prefix.shape
    assert prefix.dtype == torch.bfloat16 and bank.dtype == torch.bfloat16 and prefix.stride(1) == 1 and bank.stride(2) == 1
    assert bank.shape[0] >= T and bank.shape[2] == D and w_score.dtype == torch.float32 and w_score.is_contiguous() and w_out.dtype == torch.bfloat16
    out = torch.empty(T, D, dtype=torch.bfloat16, device=prefix.device)
    _ck(lib().ne_attn_res(_p(prefix), _c.c_longlong(prefix.stride(0)), _p(bank), _c.c_longlong(bank.stride(0)), _c.c_longlong(bank.stride(1)),
                          _c.c_int(valid), _p(w_score), _p(w_out), _c.c_float(eps), _p(out), _c.c_longlong(D), _c.c_int(T), _c.c_int(D),
                          _c.c_int(write_row), _st()), "ne_attn_res")
    return out


mhc_split_weights = ref.mhc_split_weights


def mhc_pre(x: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, iters: int, eps: float, fn_split=None):
    """Hyper-connection pre-mix: the coefficient product as a bf16 tensor-core GEMM against the head / remainder split of the
    fp32 matrix (`mhc_split_weights`, pass it in to avoid rebuilding it every call), then one kernel for the sum of squares,
    the sigmoid / softmax / Sinkhorn coefficients and the stream contraction."""
    T, h, D = x.shape
    x = x.contiguous()
    assert x.dtype == torch.bfloat16 and base.dtype == torch.float32 and scale.dtype == torch.float32 and D % 8 == 0
    if fn_split is None:
        fn_split = mhc_split_weights(fn)
    assert fn_split.dtype == torch.bfloat16 and fn_split.shape[1] == h * D and fn_split.shape[0] >= 2 * (2 + h) * h
    mixes = linear(x.view(T, h * D), fn_split, out_fp32=True)                    # [T, >= 2M] fp32
    y = torch.empty(T, D, dtype=torch.bfloat16, device=x.device)
    post = torch.empty(T, h, dtype=torch.bfloat16, device=x.device)
    comb = torch.empty(T, h, h, dtype=torch.bfloat16, device=x.device)
    _ck(lib().ne_mhc_mix(_p(x), _p(mixes), _c.c_int(mixes.stride(0)), _p(base), _p(scale), _p(y), _p(post), _p(comb), _c.c_int(T), _c.c_int(h),
                         _c.c_int(D), _c.c_int(iters), _c.c_float(eps), _st()), "ne_mhc_mix")
    return y, post, comb


def mhc_post(x: torch.Tensor, res: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """Hyper-connection post-mix: out[t, i] = post[t, i] x[t] + sum_j comb[t, j, i] res[t, j]."""
    T, h, D = res.shape
    res = res.contiguous()
    assert x.dtype == torch.bfloat16 and res.dtype == torch.bfloat16 and x.stride(1) == 1 and post.is_contiguous() and comb.is_contiguous()
    assert post.dtype == torch.bfloat16 and comb.dtype == torch.bfloat16
    out = torch.empty(T, h, D, dtype=torch.bfloat16, device=x.device)
    _ck(lib().ne_mhc_post(_p(x), _c.c_longlong(x.stride(0)), _p(res), _p(post), _p(comb), _p(out), _c.c_longlong(T), _c.c_int(h), _c.c_int(D), _st()),
        "ne_mhc_post")
    return out


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """o * sigmoid(gate) for o [T, heads, D] contiguous and gate a (possibly strided) view of the same shape."""
    T, Hh, D = o.shape
    o = o.contiguous()
    assert o.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16 and gate.stride(2) == 1 and D % 2 == 0
    out = torch.empty_like(o)
    _ck(lib().ne_sigmoid_gate(_p(o), _p(gate), _c.c_longlong(gate.stride(0)), _c.c_longlong(gate.stride(1)), _p(out), _c.c_longlong(T), _c.c_int(Hh),
                              _c.c_int(D), _st()), "ne_sigmoid_gate")
    return out


# ---- MTP draft verification --------------------------------------------------------------------------------
mtp_greedy_verify = ref.mtp_greedy_verify
mtp_rejection_sample = ref.mtp_rejection_sample


def mtp_verify(logits: torch.Tensor, drafts: torch.Tensor, temperatures: torch.Tensor, have: Optional[torch.Tensor] = None,
               coins: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None, force_accept: Optional[int] = None,
               want_logprob: bool = False, seed: Optional[int] = None, seed_buf: Optional[torch.Tensor] = None):
    """Two kernels, no host synchronisation (see csrc/kernels/mtp.cu); same contract as `reference.mtp_verify`.  The sampled
    rows draw from a counter-based hash of a seed: `seed_buf` (int64 [1] on the device, read at run time - what a captured
    CUDA graph uses, with the caller bumping it every step), else `seed`, else one taken from `generator`."""
    B, N1, V = logits.shape
    N = N1 - 1
    dev = logits.device
    logits = logits.float().contiguous()
    drafts = drafts.to(torch.int64).contiguous()
    temps = temperatures.float().contiguous()
    acc = torch.empty(B, dtype=torch.int32, device=dev)
    nxt = torch.empty(B, dtype=torch.int64, device=dev)
    bundle = torch.empty(B, N1, dtype=torch.int64, device=dev)
    ext = torch.empty(B, N1, dtype=torch.int64, device=dev)
    lp = torch.empty(B, dtype=torch.float32, device=dev) if want_logprob else None
    stats = torch.empty(B * N1 * 4, dtype=torch.int32, device=dev)
    if seed is None:
        seed = int(torch.randint(0, 2 ** 62, (1,), generator=generator).item()) if generator is not None and generator.device.type == "cpu" else 0x5eed
    hv = None if have is None else have.to(torch.int32).contiguous()
    cn = None if coins is None else coins.float().contiguous()
    _ck(lib().ne_mtp_verify(_p(logits), _p(drafts), _p(temps), _p(hv), _p(cn), _p(stats), _p(acc), _p(nxt), _p(bundle), _p(ext), _p(lp),
                            _c.c_int(B), _c.c_int(N), _c.c_int(V), _c.c_int(-1 if force_accept is None else int(force_accept)),
                            _c.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _p(seed_buf), _st()), "ne_mtp_verify")
    LAUNCHES[0] += 1
    return acc, nxt, bundle, ext, lp


def mtp_chain_meta(base_len: torch.Tensor, num_accepted: torch.Tensor, block_tables: torch.Tensor, block_size: int, k: int,
                   positions: torch.Tensor, slot_mapping: torch.Tensor, context_lens: torch.Tensor) -> None:
    """Positions, cache slots and context lengths of chain step `k` of the draft predictor, from the accepted counts on the device."""
    B = base_len.numel()
    assert base_len.dtype == torch.int32 and num_accepted.dtype == torch.int32 and block_tables.dtype == torch.int32
    assert positions.dtype == torch.int64 and slot_mapping.dtype == torch.int64 and context_lens.dtype == torch.int32
    _ck(lib().ne_mtp_chain_meta(_p(base_len), _p(num_accepted), _p(block_tables), _c.c_int(block_tables.stride(0)), _c.c_int(block_size), _c.c_int(k),
                                _c.c_int(B), _p(positions), _p(slot_mapping), _p(context_lens), _st()), "ne_mtp_chain_meta")
