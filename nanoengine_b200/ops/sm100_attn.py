"""CUDA bodies of attention and sampling.

MLA over an fp8 latent cache with the DeepSeek-V3 geometry (576-value rows, 64-token pages, <= 128 heads) runs on the
tcgen05 kernel, dense (paged) and DSA-sparse (listed rows gathered into the same pipeline) alike; every other shape and the
bf16 cache run on the shape-generic CUDA-core kernel.
"""
from __future__ import annotations

import ctypes as _c

import torch

from . import sm100 as _k

FP8 = torch.float8_e4m3fn
_NUM_SMS = None
_sample_calls = 0
SPARSE_TC_CALLS = [0]        # launches of the sparse tensor-core MLA kernel (tests check that the DSA path really takes it)


def _sms():
    global _NUM_SMS
    if _NUM_SMS is None:
        _NUM_SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _NUM_SMS


def _i32(t):
    return t if t.dtype == torch.int32 and t.is_contiguous() else t.to(torch.int32).contiguous()


def mla_splits(T: int, max_pages: int) -> int:
    """Key slices per token so that small batches still fill the GPU: each slice keeps at least 4 pages.  Slicing is only worth
    its price (every slice writes and the merge re-reads an fp32 [T, H, 512] partial result) when it raises the number of busy
    SMs: with 2 T CTAs covering more than ~60 % of them a second slice just adds a second, half-empty wave."""
    ctas = 2 * T
    if ctas * 5 >= _sms() * 3:
        return 1
    want = _sms() // ctas                       # the largest count that still fits one wave
    return max(1, min(want, max(1, max_pages // 4), 32))


def mla_partials(q, cache, block_tables, cu_seqlens_q, context_lens, scale, kv_lora_rank, splits: int):
    """Un-merged split-KV results of the fp8 tcgen05 kernel: part [splits, T, H, R] fp32 (each slice normalised on its own) and
    lse2 [splits, T, H] fp32 (log2-sum-exp of the slice, -inf where a slice saw no key).  `ne_attn_merge` folds any stack of
    such slices, including slices computed on other GPUs."""
    T, H, Dk = q.shape
    R = kv_lora_rank
    assert splits >= 2 and cache.dtype == FP8 and Dk == 576 and R == 512 and cache.shape[1] == 64 and H <= 128
    lib = _k.lib()
    bt, cu, cl = _i32(block_tables), _i32(cu_seqlens_q), _i32(context_lens)
    if q.dtype == FP8:
        q8 = q.contiguous()
    else:
        q = q if (q.dtype == torch.bfloat16 and q.is_contiguous()) else q.to(torch.bfloat16).contiguous()
        q8 = torch.empty(T * H, Dk, dtype=torch.uint8, device=q.device)
        _k._ck(lib.ne_cast_e4m3(_k._p(q), _k._p(q8), _c.c_longlong(T * H * Dk), _k._st()), "ne_cast_e4m3")
    part = torch.empty(splits, T, H, R, dtype=torch.float32, device=q.device)
    lse2 = torch.empty(splits, T, H, dtype=torch.float32, device=q.device)
    _k._ck(lib.ne_mla_fp8(_k._p(q8), _k._p(cache), _c.c_int(cache.shape[0]), _k._p(bt), _c.c_int(bt.stride(0)), _k._p(cu), _k._p(cl),
                          _c.c_int(cl.numel()), _c.c_int(T), _c.c_int(H), _c.c_int(splits), _c.c_float(scale), _k._p(None), _k._p(part), _k._p(lse2),
                          _k._st()), "ne_mla_fp8")
    return part, lse2


def mla_attention_paged(q, cache, block_tables, cu_seqlens_q, context_lens, scale, kv_lora_rank, sparse_indices=None, splits=None):
    T, H, Dk = q.shape
    R = kv_lora_rank
    lib = _k.lib()
    bt, cu, cl = _i32(block_tables), _i32(cu_seqlens_q), _i32(context_lens)
    B = cl.numel()
    out = torch.empty(T, H, R, dtype=torch.bfloat16, device=q.device)
    if T == 0:
        return out
    geom = cache.dtype == FP8 and Dk == 576 and R == 512 and cache.shape[1] == 64 and H <= 128
    fast = geom and sparse_indices is None
    if q.dtype == FP8:
        assert geom and q.is_contiguous(), "an e4m3 query is only produced for the fp8 tensor-core attention kernels"
    else:
        q = q if (q.dtype == torch.bfloat16 and q.is_contiguous()) else q.to(torch.bfloat16).contiguous()
    if geom and sparse_indices is not None:
        # DSA: the listed cache rows are gathered into the same tcgen05 pipeline (64 rows per tile)
        if q.dtype == FP8:
            q8 = q
        else:
            q8 = torch.empty(T * H, Dk, dtype=torch.uint8, device=q.device)
            _k._ck(lib.ne_cast_e4m3(_k._p(q), _k._p(q8), _c.c_longlong(T * H * Dk), _k._st()), "ne_cast_e4m3")
        sp = _i32(sparse_indices)
        topk = sp.shape[1]
        tiles = -(-topk // 64)
        S = splits if splits is not None else mla_splits(T, tiles)
        part = lse2 = None
        if S > 1:
            part = torch.empty(S, T, H, R, dtype=torch.float32, device=q.device)
            lse2 = torch.empty(S, T, H, dtype=torch.float32, device=q.device)
        _k._ck(lib.ne_mla_fp8_sparse(_k._p(q8), _k._p(cache), _c.c_int(cache.shape[0]), _k._p(sp), _c.c_int(topk), _c.c_int(T), _c.c_int(H),
                                     _c.c_int(S), _c.c_float(scale), _k._p(out), _k._p(part), _k._p(lse2), _k._st()), "ne_mla_fp8_sparse")
        SPARSE_TC_CALLS[0] += 1
        if S > 1:
            _k._ck(lib.ne_attn_merge(_k._p(part), _k._p(lse2), _k._p(out), _c.c_int(S), _c.c_longlong(T * H), _c.c_int(R), _c.c_int(R), _k._st()),
                   "ne_attn_merge")
        return out
    if fast:
        if q.dtype == FP8:
            q8 = q
        else:
            q8 = torch.empty(T * H, Dk, dtype=torch.uint8, device=q.device)
            _k._ck(lib.ne_cast_e4m3(_k._p(q), _k._p(q8), _c.c_longlong(T * H * Dk), _k._st()), "ne_cast_e4m3")
        S = splits if splits is not None else mla_splits(T, bt.shape[1])
        part = lse2 = None
        if S > 1:
            part = torch.empty(S, T, H, R, dtype=torch.float32, device=q.device)
            lse2 = torch.empty(S, T, H, dtype=torch.float32, device=q.device)
        _k._ck(lib.ne_mla_fp8(_k._p(q8), _k._p(cache), _c.c_int(cache.shape[0]), _k._p(bt), _c.c_int(bt.stride(0)), _k._p(cu), _k._p(cl),
                              _c.c_int(B), _c.c_int(T), _c.c_int(H), _c.c_int(S), _c.c_float(scale), _k._p(out), _k._p(part), _k._p(lse2), _k._st()),
               "ne_mla_fp8")
        if S > 1:
            _k._ck(lib.ne_attn_merge(_k._p(part), _k._p(lse2), _k._p(out), _c.c_int(S), _c.c_longlong(T * H), _c.c_int(R), _c.c_int(R), _k._st()),
                   "ne_attn_merge")
        return out
    fp8 = cache.dtype == FP8
    assert fp8 or cache.dtype == torch.bfloat16, "the CUDA attention kernels read bf16 or fp8 caches"
    sp = None if sparse_indices is None else _i32(sparse_indices)
    _k._ck(lib.ne_attn_generic(_k._p(q), _c.c_longlong(q.stride(0)), _c.c_int(q.stride(1)), _k._p(cache), _k._p(None),
                               _c.c_longlong(cache.shape[-1]), _c.c_int(0), _c.c_int(0), _k._p(bt), _c.c_int(bt.stride(0)), _c.c_int(cache.shape[1]),
                               _k._p(cu), _k._p(cl), _c.c_int(B), _k._p(sp), _c.c_int(0 if sp is None else sp.shape[1]), _k._p(out),
                               _c.c_longlong(H * R), _c.c_int(R), _k._p(None), _c.c_int(T), _c.c_int(H), _c.c_int(Dk), _c.c_int(R),
                               _c.c_float(scale), _c.c_int(1 if fp8 else 0), _c.c_int(0), _c.c_int(0), _k._st()), "ne_attn_generic")
    return out


def gqa_attention_paged(q, k_cache, v_cache, block_tables, cu_seqlens_q, context_lens, scale, window: int = 0):
    """`window` > 0: every query sees only its last `window` key positions (sliding-window layers); those layers and head
    dims other than 128 run on the generic kernel."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    lib = _k.lib()
    bt, cu, cl = _i32(block_tables), _i32(cu_seqlens_q), _i32(context_lens)
    q = q if (q.dtype == torch.bfloat16 and q.stride(-1) == 1) else q.to(torch.bfloat16).contiguous()
    out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    if T == 0:
        return out
    group = Hq // Hkv
    if (D == 128 and window <= 0 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16 and k_cache.shape[1] == 64 and Hq % Hkv == 0
            and group <= 128 and group & (group - 1) == 0 and k_cache.is_contiguous() and v_cache.is_contiguous()):
        # tcgen05 kernel: one CTA per (kv head, tile of 128 (token, head) rows, key slice)
        q = q.contiguous()
        tq = 128 // group
        B = cl.numel()
        max_tiles = min(T, T // tq + B)
        S = 1
        if max_tiles * Hkv < 74:                       # few CTAs (small decode batches): slice the keys
            S = max(1, min(148 // (max_tiles * Hkv), max(1, bt.shape[1] // 4), 16))
        part = lse2 = None
        if S > 1:
            part = torch.empty(S, T, Hq, D, dtype=torch.float32, device=q.device)
            lse2 = torch.empty(S, T, Hq, dtype=torch.float32, device=q.device)
        _k._ck(lib.ne_gqa_bf16(_k._p(q), _k._p(k_cache), _k._p(v_cache), _c.c_int(k_cache.shape[0]), _k._p(bt), _c.c_int(bt.stride(0)), _k._p(cu),
                               _k._p(cl), _c.c_int(B), _c.c_int(T), _c.c_int(Hq), _c.c_int(Hkv), _c.c_int(max_tiles), _c.c_int(S), _c.c_float(scale),
                               _k._p(out), _k._p(part), _k._p(lse2), _k._st()), "ne_gqa_bf16")
        if S > 1:
            _k._ck(lib.ne_attn_merge(_k._p(part), _k._p(lse2), _k._p(out), _c.c_int(S), _c.c_longlong(T * Hq), _c.c_int(D), _c.c_int(D), _k._st()),
                   "ne_attn_merge")
        return out
    assert group % 4 == 0 or group == 1 and Hq % 4 == 0 or Hkv == Hq, "query heads per kv head must be a multiple of 4"
    _k._ck(lib.ne_attn_generic(_k._p(q), _c.c_longlong(q.stride(0)), _c.c_int(q.stride(1)), _k._p(k_cache), _k._p(v_cache),
                               _c.c_longlong(Hkv * D), _c.c_int(D), _c.c_int(group), _k._p(bt), _c.c_int(bt.stride(0)), _c.c_int(k_cache.shape[1]),
                               _k._p(cu), _k._p(cl), _c.c_int(cl.numel()), _k._p(None), _c.c_int(0), _k._p(out), _c.c_longlong(Hq * D), _c.c_int(D),
                               _k._p(None), _c.c_int(T), _c.c_int(Hq), _c.c_int(D), _c.c_int(D), _c.c_float(scale), _c.c_int(0), _c.c_int(max(0, int(window))), _c.c_int(0), _k._st()),
           "ne_attn_generic")
    return out


def attention_varlen(q, k, v, cu_seqlens, scale, causal: bool = False):
    """Attention over ragged sequences without a paged cache: q, k, v [T, H, D] of the same tokens, sequence i owns rows
    [cu[i], cu[i+1]).  Runs on the generic kernel, which addresses k / v as a one-row-per-page cache through a table of row
    numbers (no copy); any head dim up to 640.  Used by the vision encoder (non-causal)."""
    T, H, D = q.shape
    q = q if (q.dtype == torch.bfloat16 and q.stride(-1) == 1) else q.to(torch.bfloat16).contiguous()
    k, v = k.to(torch.bfloat16).contiguous(), v.to(torch.bfloat16).contiguous()
    out = torch.empty(T, H, D, dtype=torch.bfloat16, device=q.device)
    if T == 0:
        return out
    cu = _i32(cu_seqlens)
    lens = (cu[1:] - cu[:-1])
    B = lens.numel()
    max_len = int(lens.max())
    bt = (cu[:-1, None] + torch.arange(max_len, device=q.device, dtype=torch.int32)[None, :]).clamp_(max=T - 1).contiguous()
    _k._ck(_k.lib().ne_attn_generic(_k._p(q), _c.c_longlong(q.stride(0)), _c.c_int(q.stride(1)), _k._p(k), _k._p(v), _c.c_longlong(H * D),
                                    _c.c_int(D), _c.c_int(1), _k._p(bt), _c.c_int(bt.stride(0)), _c.c_int(1), _k._p(cu), _k._p(lens.contiguous()),
                                    _c.c_int(B), _k._p(None), _c.c_int(0), _k._p(out), _c.c_longlong(H * D), _c.c_int(D), _k._p(None), _c.c_int(T),
                                    _c.c_int(H), _c.c_int(D), _c.c_int(D), _c.c_float(scale), _c.c_int(0), _c.c_int(0),
                                    _c.c_int(0 if causal else 1), _k._st()), "ne_attn_generic")
    return out


def sample(logits, temperatures, generator=None, return_logprobs=False):
    """Argmax / Gumbel-max on the device; the noise is a counter-based hash seeded from the generator's seed and a call counter."""
    global _sample_calls
    rows, V = logits.shape
    logits = logits if (logits.dtype == torch.float32 and logits.is_contiguous()) else logits.float().contiguous()
    temps = temperatures.float().contiguous()
    tok = torch.empty(rows, dtype=torch.int64, device=logits.device)
    lp = torch.empty(rows, dtype=torch.float32, device=logits.device) if return_logprobs else None
    _sample_calls += 1
    seed = ((generator.initial_seed() if generator is not None else 0) * 0x9E3779B97F4A7C15 + _sample_calls) & 0xFFFFFFFFFFFFFFFF
    _k._ck(_k.lib().ne_sample(_k._p(logits), _k._p(temps), _k._p(tok), _k._p(lp), _c.c_int(rows), _c.c_int(V), _c.c_ulonglong(seed), _k._st()),
           "ne_sample")
    return tok, lp
