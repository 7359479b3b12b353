"""Per-kernel timings at the shapes the DeepSeek-V3 decode and prefill steps use, with roofline fractions.

    python benchmarks/kernel_bench.py                       # all cases, table on stdout
    python benchmarks/kernel_bench.py --case moe_gemm1 --experts 8 --iters 3   # one small case (what the ncu captures run)
    python benchmarks/kernel_bench.py --case absorb_k_decode --graph           # short kernels: time a graph replay

Timing: CUDA events on the launching stream, 3 warm-up runs, a buffer larger than L2 is rewritten between timed
runs, the median of `--iters` runs is reported.  Fractions are against MEASURED_PEAKS.json (copy bandwidth and cuBLAS
bf16 throughput of the machine's B200s) when that file exists, otherwise against the documented fallback figures.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


from nanoengine_b200.ops import sm100, sm100_attn

FP8 = torch.float8_e4m3fn


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def timeit(fn, iters, graph=False):
    for _ in range(3):
        fn()
    if graph:
        # a kernel of a few microseconds is shorter than its own launch path: replay it from a CUDA graph, as the decode step does
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        fn = g.replay
        fn()
    ts = []
    for _ in range(iters):
        flush_l2()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    ts.sort()
    return ts[len(ts) // 2]


def rand_fp8(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(FP8)


def rand_scales(*shape):
    """Weight block scales in the process's scale format (powers of two under "ue8m0")."""
    if sm100.scale_format() == "ue8m0":
        return torch.exp2(torch.randint(-1, 2, shape, device="cuda").float())
    return torch.rand(*shape, device="cuda") + 0.5


def case_dense_fp8(M, N, K):
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w, s = rand_fp8(N, K), rand_scales((N + 127) // 128, K // 128)
    q = torch.empty(M, K, dtype=FP8, device="cuda")
    sc = torch.empty(K // 128, M, dtype=torch.float32, device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    q.copy_(rand_fp8(M, K)); sc.fill_(1.0)
    fn = lambda: sm100._gemm(q, K, 0, w, out, N, 0, M, N, K, 1, None, None, True, sc, M, 0, s, False)
    return fn, N * K + M * K + M * N * 2, 2.0 * M * N * K


def case_dense_bf16(M, N, K, out_fp32=False):
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    fn = lambda: sm100.linear(x, w, out_fp32=out_fp32)
    return fn, (N * K + M * K) * 2 + M * N * (4 if out_fp32 else 2), 2.0 * M * N * K


def case_moe_gemm(E, rows_per_expert, N, K):
    """Contiguous grouped fp8 GEMM as the local MoE path runs it (every expert gets the same number of rows)."""
    pad = (rows_per_expert + 127) // 128 * 128
    R = E * pad
    a = rand_fp8(R, K)
    sa = torch.ones(K // 128, R, device="cuda")
    w = rand_fp8(E, N, K)
    sb = rand_scales(E, (N + 127) // 128, K // 128)
    counts = torch.full((E,), rows_per_expert, dtype=torch.int32, device="cuda")
    row_start = (torch.arange(E + 1, device="cuda") * pad).to(torch.int32)
    out = torch.empty(R, N, dtype=torch.bfloat16, device="cuda")
    fn = lambda: sm100._gemm(a, K, 0, w, out, N, 0, R, N, K, E, counts, row_start, True, sa, R, 0, sb, False)
    return fn, E * N * K + E * rows_per_expert * (K + 2 * N), 2.0 * E * rows_per_expert * N * K


def case_moe_gemm_nvfp4(E, rows_per_expert, N, K):
    """The same grouped GEMM with NVFP4 operands (packed e2m1, e4m3 scale per 16 elements), W4A4."""
    pad = (rows_per_expert + 127) // 128 * 128
    R = E * pad
    a = torch.randint(0, 256, (R, K // 2), device="cuda", dtype=torch.int32).to(torch.uint8)
    b = torch.randint(0, 256, (E, N, K // 2), device="cuda", dtype=torch.int32).to(torch.uint8)
    sa = torch.ones(R, K // 16, device="cuda").to(FP8)
    sb = torch.ones(E, N, K // 16, device="cuda").to(FP8)
    alpha = torch.ones(E, device="cuda")
    counts = torch.full((E,), rows_per_expert, dtype=torch.int32, device="cuda")
    row_start = (torch.arange(E + 1, device="cuda") * pad).to(torch.int32)
    out = torch.empty(R, N, dtype=torch.bfloat16, device="cuda")
    lib = sm100.lib()
    import ctypes as _c
    p = sm100._p
    fn = lambda: sm100._ck(lib.ne_gemm_nvfp4(p(a), p(b), p(out), _c.c_longlong(N), _c.c_int(R), _c.c_int(N), _c.c_int(K), _c.c_int(E), p(counts),
                                             p(row_start), p(sa), p(sb), p(alpha), _c.c_int(0), sm100._st()), "ne_gemm_nvfp4")
    return fn, E * N * K // 2 + E * N * K // 16 + E * rows_per_expert * (K // 2 + K // 16 + 2 * N), 2.0 * E * rows_per_expert * N * K


def case_mla(B, ctx, H=128, q_len=1):
    bs = 64
    nb = (ctx + bs - 1) // bs
    cache = rand_fp8(B * nb + 1, bs, 576)
    bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    q = (torch.randn(B * q_len, H, 576, device="cuda") * 0.3).to(torch.bfloat16)
    cu = (torch.arange(B + 1, device="cuda") * q_len).to(torch.int32)
    cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    fn = lambda: sm100_attn.mla_attention_paged(q, cache, bt, cu, cl, 0.07, 512)
    return fn, B * ctx * 576 + B * q_len * H * (576 + 512) * 2, 2.0 * B * q_len * H * ctx * (576 + 512)


def case_mla_sparse(B, ctx, topk=2048, H=128):
    """DSA decode attention: every token attends `topk` rows of its own ~ctx-token context, picked at random."""
    bs = 64
    nb = (ctx + bs - 1) // bs
    cache = rand_fp8(B * nb + 1, bs, 576)
    q = (torch.randn(B, H, 576, device="cuda") * 0.3).to(torch.bfloat16)
    bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    cu = torch.arange(B + 1, device="cuda", dtype=torch.int32)
    cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    sp = torch.stack([torch.randperm(ctx, device="cuda")[:topk] + b * nb * bs for b in range(B)]).to(torch.int32)
    fn = lambda: sm100_attn.mla_attention_paged(q, cache, bt, cu, cl, 0.07, 512, sparse_indices=sp)
    return fn, B * topk * 576 + B * H * (576 + 512) * 2, 2.0 * B * H * topk * (576 + 512)


# ---- the same shapes through the libraries the reference calls on Blackwell (bars, not product paths) ----
def bar_mla_flashinfer(B, ctx, H=128):
    """flashinfer's TRTLLM-GEN MLA decode, the kernel the reference selects on sm_100 (layers/backends/mla/trtllm.py:45-204)."""
    from flashinfer.mla import trtllm_batch_decode_with_kv_cache_mla
    bs = 64
    nb = (ctx + bs - 1) // bs
    cache = rand_fp8(B * nb + 1, 1, bs, 576)
    bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    q = (torch.randn(B, 1, H, 576, device="cuda") * 0.3).to(FP8)
    sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device="cuda")
    fn = lambda: trtllm_batch_decode_with_kv_cache_mla(q, cache, ws, 128, 512, 64, bt, sl, ctx, bmm1_scale=0.07, bmm2_scale=1.0)
    return fn, B * ctx * 576 + B * H * (576 + 512) * 2, 2.0 * B * H * ctx * (576 + 512)


def bar_gqa_flashinfer(B, ctx, Hq, Hkv, D=128, bs=64):
    """flashinfer's TRTLLM-GEN GQA decode (reference layers/backends/attention/fa4.py:100-149)."""
    from flashinfer.decode import trtllm_batch_decode_with_kv_cache
    nb = (ctx + bs - 1) // bs
    kv = torch.randn(B * nb + 1, 2, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device="cuda")
    fn = lambda: trtllm_batch_decode_with_kv_cache(q, kv, ws, bt, sl, ctx, bmm1_scale=D ** -0.5, bmm2_scale=1.0, kv_layout="HND")
    return fn, B * ctx * Hkv * D * 4 + B * Hq * D * 4, 4.0 * B * Hq * ctx * D


def bar_matmul_bf16(M, N, K):
    """torch.matmul (cuBLAS) on bf16 operands of the same M, N, K."""
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    fn = lambda: torch.nn.functional.linear(x, w)
    return fn, N * K * 2 + M * (K + N) * 2, 2.0 * M * N * K


def case_silu_masked(E=32, rows=32, cap=512, I=2048):
    g = torch.randn(E, cap, 2 * I, device="cuda", dtype=torch.bfloat16)
    counts = torch.full((E,), rows, dtype=torch.int32, device="cuda")
    q = torch.empty(E, cap, I, dtype=FP8, device="cuda")
    sc = torch.empty(E, I // 128, cap, dtype=torch.float32, device="cuda")
    import ctypes as _c
    lib = sm100.lib()
    def fn():
        sm100._ck(lib.ne_silu_mul(sm100._p(g), sm100._p(None), sm100._p(q), sm100._p(sc), _c.c_int(cap), _c.c_longlong((I // 128) * cap),
                                  sm100._p(counts), sm100._p(None), _c.c_int(E), _c.c_int(cap), _c.c_int(I), sm100._st()), "ne_silu_mul")
    return fn, E * rows * I * 5, 0.0


def case_indexer(B, ctx, q_len=1, Hi=64, D=128, bs=64, topk=2048):
    """DSA indexer selection: fp8 logits of every visible key + top-2048 + page translation (decode: one token per sequence)."""
    nb = (ctx + bs - 1) // bs
    cache = torch.randint(0, 127, (B * nb + 1, bs * (D + 4)), device="cuda", dtype=torch.uint8)
    cache[:, bs * D:] = torch.ones(B * nb + 1, bs, device="cuda").view(torch.uint8).view(B * nb + 1, bs * 4)
    bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    T = B * q_len
    cu = (torch.arange(B + 1, device="cuda") * q_len).to(torch.int32)
    cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q8 = (torch.randn(T, Hi, D, device="cuda")).to(FP8)
    qs = torch.ones(T, Hi, device="cuda")
    w = torch.randn(T, Hi, device="cuda")
    fn = lambda: sm100.indexer_select(q8, qs, w, cache, bt, cu, cl, topk)
    return fn, B * ctx * (D + 4) + T * ctx * 4 * 2, 2.0 * T * Hi * ctx * D


def case_absorb(T, which, H=128, nope=128, rope=64, R=512, v=128):
    """The two per-head products around absorbed MLA: q_nope @ W_UK ([T, H, 128] -> [T, H, 512], read out of the q_b output) and
    the latent attention output @ W_UV ([T, H, 512] -> [T, H, 128]); one GEMM group per head."""
    if which == "k":
        q = torch.randn(T, H, nope + rope, device="cuda", dtype=torch.bfloat16)
        x, w = q[..., :nope], (torch.randn(H, nope, R, device="cuda") * 0.05).to(torch.bfloat16)
    else:
        x, w = torch.randn(T, H, R, device="cuda", dtype=torch.bfloat16), (torch.randn(H, R, v, device="cuda") * 0.05).to(torch.bfloat16)
    out = torch.empty(T, H, w.shape[2], device="cuda", dtype=torch.bfloat16)
    wt = sm100.kmajor(w)
    fn = lambda: sm100.bmm_absorb(x, w, out, wt=wt)
    return fn, w.numel() * 2 + T * H * (w.shape[1] + w.shape[2]) * 2, 2.0 * T * H * w.shape[1] * w.shape[2]


def case_gdn(B, q_len=1, Hk=16, Hv=32, Dk=128, Dv=128, K=4):
    """Gated delta-net layer core at the Qwen3.5-MoE shape: conv over [q|k|v] with window shift, then the recurrent step with the gated
    norm.  The floor is one read and one write of every sequence's fp32 state."""
    T = B * q_len
    C = 2 * Hk * Dk + Hv * Dv
    bf = dict(device="cuda", dtype=torch.bfloat16)
    proj = torch.randn(T, C + Hv * Dv, **bf)
    qkv, z = proj[:, :C], proj[:, C:].reshape(T, Hv, Dv)
    ab = torch.randn(T, 2 * Hv, **bf)
    w = (torch.randn(C, K, device="cuda") * 0.3).to(torch.bfloat16)
    conv = torch.zeros(B + 1, K - 1, C, **bf)
    state = torch.randn(B + 1, Hv, Dv, Dk, device="cuda") * 0.1
    slots = torch.arange(B, device="cuda", dtype=torch.int32)
    cu = (torch.arange(B + 1, device="cuda") * q_len).to(torch.int32)
    fresh = torch.zeros(B, dtype=torch.int32, device="cuda")
    A_log, dtb = torch.rand(Hv, device="cuda"), torch.randn(Hv, device="cuda")
    nw = torch.ones(Dv, **bf)

    def fn():
        y = sm100.gdn_conv(qkv, w, conv, slots, cu, fresh, q_len == 1)
        q = y[:, : Hk * Dk].view(T, Hk, Dk)
        k = y[:, Hk * Dk: 2 * Hk * Dk].view(T, Hk, Dk)
        v = y[:, 2 * Hk * Dk:].view(T, Hv, Dv)
        return sm100.gdn_recurrent(q, k, v, ab[:, :Hv], ab[:, Hv:], A_log, dtb, state, slots, cu, fresh, z, nw, 1e-6, q_len, None)

    nbytes = B * Hv * Dv * Dk * 4 * 2 + T * (C * 2 * 3 + Hv * Dv * 2 * 2) + B * (K - 1) * C * 2 * 2
    return fn, nbytes, 2.0 * T * Hv * Dv * Dk * 3


def case_gqa(B, ctx, q_len, Hq, Hkv, D=128, bs=64):
    nb = (ctx + bs - 1) // bs
    kc = torch.randn(B * nb + 1, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(B * nb + 1, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    T = B * q_len
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = (torch.arange(B + 1, device="cuda") * q_len).to(torch.int32)
    cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    fn = lambda: sm100_attn.gqa_attention_paged(q, kc, vc, bt, cu, cl, D ** -0.5)
    causal = ctx - (q_len - 1) / 2.0
    return fn, B * ctx * Hkv * D * 4 + T * Hq * D * 4, 4.0 * T * Hq * causal * D


def case_moe_layer(T, E, topk=8, H=7168, I=2048):
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w13, w2 = rand_fp8(E, 2 * I, H), rand_fp8(E, H, I)
    s13 = torch.rand(E, 2 * I // 128, H // 128, device="cuda") * 0.01
    s2 = torch.rand(E, H // 128, I // 128, device="cuda") * 0.01
    idx = torch.stack([torch.randperm(E, device="cuda")[:topk] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, topk, device="cuda")
    fn = lambda: sm100.moe_experts(x, idx, w, w13, w2, s13, s2, 0)
    return fn, E * 3 * I * H, 2.0 * T * topk * 3 * I * H


def case_small(kind, T=128, H=7168, E=32, K=8, I=2048):
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    if kind == "router":
        w = torch.randn(E, H, device="cuda")
        def fn():
            sm100.moe_route(sm100.router_logits(x, w), None, 8, 1, 1, True, 2.5, "sigmoid")
        return fn, E * H * 4 + T * H * 2, 2.0 * T * E * H
    if kind == "add_rmsnorm_quant":
        r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16); w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        return (lambda: sm100.add_rmsnorm(x, r, w, 1e-6, False, True)), T * H * (2 + 2 + 2 + 2 + 1), 0.0
    if kind == "rmsnorm_then_quant":
        r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16); w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        def fn():
            y, _ = sm100._rmsnorm(x, r, w, 1e-6, True, False)
            sm100.quant_fp8_1x128(y)
        return fn, T * H * (2 + 2 + 2 + 2 + 2 + 1), 0.0
    if kind == "moe_route":
        lg = torch.randn(T, 256, device="cuda"); b = torch.zeros(256, device="cuda")
        return (lambda: sm100.moe_route(lg, b, 8, 8, 4, True, 2.5, "sigmoid")), T * 256 * 4, 0.0
    if kind == "sample":
        lg = torch.randn(T, 129280, device="cuda"); tm = torch.zeros(T, device="cuda")
        return (lambda: sm100_attn.sample(lg, tm)), T * 129280 * 4, 0.0
    raise ValueError(kind)


def build_cases(args):
    E = args.experts
    c = {
        # decode, 128 tokens per GPU
        "qkv_a_decode": lambda: case_dense_fp8(128, 2112, 7168),
        "q_b_decode": lambda: case_dense_fp8(128, 24576, 1536),
        "o_proj_decode": lambda: case_dense_fp8(128, 7168, 16384),
        "shared_up_decode": lambda: case_dense_fp8(128, 4096, 7168),
        "shared_down_decode": lambda: case_dense_fp8(128, 7168, 2048),
        # same bytes and K steps as the fp8 cases above, without the per-K-block promotion (isolates the memory path)
        "qkv_a_like_bf16": lambda: case_dense_bf16(128, 2112, 3584),
        "o_proj_like_bf16": lambda: case_dense_bf16(128, 7168, 8192),
        "lm_head_decode": lambda: case_dense_bf16(128, 129280, 7168, True),
        "moe_gemm1": lambda: case_moe_gemm(E, args.rows, 4096, 7168),
        "moe_gemm2": lambda: case_moe_gemm(E, args.rows, 7168, 2048),
        "moe_layer_decode": lambda: case_moe_layer(128, E),
        "router": lambda: case_small("router"),
        "silu_masked": lambda: case_silu_masked(),
        "add_rmsnorm_quant": lambda: case_small("add_rmsnorm_quant"),
        "rmsnorm_then_quant": lambda: case_small("rmsnorm_then_quant"),
        "moe_route": lambda: case_small("moe_route"),
        "sample": lambda: case_small("sample"),
        "indexer_decode_16k": lambda: case_indexer(128, 16384),
        "indexer_decode_64k": lambda: case_indexer(32, 65536),
        "indexer_prefill_4k": lambda: case_indexer(1, 8192, q_len=4096),
        "gqa_decode_tp8": lambda: case_gqa(256, 4352, 1, 8, 1),          # Qwen3-235B per rank at TP8: 8 q heads, 1 kv head
        "gqa_decode_tp1": lambda: case_gqa(64, 4352, 1, 64, 4),
        "gqa_prefill_tp8": lambda: case_gqa(4, 4096, 4096, 8, 1),
        "absorb_k_decode": lambda: case_absorb(128, "k"),
        "absorb_v_decode": lambda: case_absorb(128, "v"),
        "gdn_decode": lambda: case_gdn(128),
        "gdn_verify2": lambda: case_gdn(128, q_len=2),
        "kda_decode_256": lambda: case_kda(256),
        "kda_prefill_2048": lambda: case_kda(8, q_len=2048),
        "attn_res_decode": lambda: case_attn_res(128),
        "attn_res_prefill": lambda: case_attn_res(16384),
        "mhc_decode": lambda: case_mhc(128),
        "mhc_prefill": lambda: case_mhc(8192),
        "mla_decode": lambda: case_mla(128, args.ctx),
        "mla_decode_small_batch": lambda: case_mla(8, 8192),
        "mla_sparse_decode_2048": lambda: case_mla_sparse(128, 8192),
        "mla_sparse_decode_64k": lambda: case_mla_sparse(64, 65536),
        # library bars at the same shapes (what the reference runs on this hardware); "unavailable" when the import or call fails
        "bar:mla_decode_flashinfer": lambda: bar_mla_flashinfer(128, args.ctx),
        "bar:gqa_decode_tp8_flashinfer": lambda: bar_gqa_flashinfer(256, 4352, 8, 1),
        "bar:qkv_a_like_bf16_cublas": lambda: bar_matmul_bf16(128, 2112, 3584),
        "bar:o_proj_like_bf16_cublas": lambda: bar_matmul_bf16(128, 7168, 8192),
        "bar:bf16_square_cublas": lambda: bar_matmul_bf16(8192, 8192, 8192),
        # prefill, 16384 tokens
        "qkv_a_prefill": lambda: case_dense_fp8(args.prefill_tokens, 2112, 7168),
        "o_proj_prefill": lambda: case_dense_fp8(args.prefill_tokens, 7168, 16384),
        "moe_gemm1_prefill": lambda: case_moe_gemm(E, args.prefill_tokens * 8 // 32, 4096, 7168),
        "moe_gemm2_prefill": lambda: case_moe_gemm(E, args.prefill_tokens * 8 // 32, 7168, 2048),
        "nvfp4_moe_gemm1_prefill": lambda: case_moe_gemm_nvfp4(E, args.prefill_tokens * 8 // 32, 4096, 7168),
        "nvfp4_moe_gemm2_prefill": lambda: case_moe_gemm_nvfp4(E, args.prefill_tokens * 8 // 32, 7168, 2048),
        "nvfp4_moe_gemm1": lambda: case_moe_gemm_nvfp4(E, args.rows, 4096, 7168),
        "nvfp4_moe_gemm2": lambda: case_moe_gemm_nvfp4(E, args.rows, 7168, 2048),
        "bf16_square": lambda: case_dense_bf16(8192, 8192, 8192),
    }
    return c


def case_kda(B, q_len=1, H=64, D=128, K=4):
    """Kimi delta attention layer core (convolution + recurrence with a decay per key channel + sigmoid-gated norm) at a 64-head
    128 x 128 shape.  The floor is one read and one write of every sequence's fp32 state."""
    T = B * q_len
    C = 3 * H * D
    bf = dict(device="cuda", dtype=torch.bfloat16)
    proj = torch.randn(T, C + H * D, **bf)
    qkv, gate = proj[:, :C], proj[:, C:].view(T, H, D)
    raw_g = torch.randn(T, H * D, **bf)
    b = torch.randn(T, H, **bf)
    w = (torch.randn(C, K, device="cuda") * 0.3).to(torch.bfloat16)
    conv = torch.zeros(B + 1, K - 1, C, **bf)
    state = torch.randn(B + 1, H, D, D, device="cuda") * 0.1
    slots = torch.arange(B, device="cuda", dtype=torch.int32)
    cu = (torch.arange(B + 1, device="cuda") * q_len).to(torch.int32)
    fresh = torch.zeros(B, dtype=torch.int32, device="cuda")
    A_log, dtb = torch.rand(H, device="cuda") - 0.5, torch.randn(H * D, device="cuda") * 0.3
    nw = torch.ones(D, **bf)

    def fn():
        y = sm100.gdn_conv(qkv, w, conv, slots, cu, fresh, q_len == 1)
        q, k, v = y[:, : H * D].view(T, H, D), y[:, H * D: 2 * H * D].view(T, H, D), y[:, 2 * H * D:].view(T, H, D)
        return sm100.kda_recurrent(q, k, v, raw_g, b, A_log, dtb, -5.0, state, slots, cu, fresh, gate, nw, 1e-6)

    nbytes = B * H * D * D * 4 * 2 + T * (C * 2 * 3 + H * D * 2 * 3) + B * (K - 1) * C * 2 * 2
    return fn, nbytes, 2.0 * T * H * D * D * 3


def case_attn_res(T, D=7168, valid=8):
    """Block attention residual of one layer: 9 candidate rows per token mixed and normalised."""
    bank = torch.randn(T, valid + 1, D, device="cuda", dtype=torch.bfloat16)
    prefix = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    ws = torch.randn(D, device="cuda") * 0.05
    wo = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    fn = lambda: sm100.attn_res_mix(prefix, bank, valid, ws, wo, 1e-6, -1)
    return fn, T * D * 2 * (valid + 2), 4.0 * T * D * (valid + 1)


def case_mhc(T, h=4, D=6144):
    """Hyper-connection pre-mix + post-mix around one sub-layer (4 streams)."""
    x = torch.randn(T, h, D, device="cuda", dtype=torch.bfloat16)
    fn_w = torch.randn((2 + h) * h, h * D, device="cuda") * 0.02
    base = torch.zeros((2 + h) * h, device="cuda")
    scale = torch.ones(3, device="cuda")
    sub = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    split = sm100.mhc_split_weights(fn_w)

    def fn():
        y, post, comb = sm100.mhc_pre(x, fn_w, base, scale, 3, 1e-6, split)
        return sm100.mhc_post(sub, x, post, comb)

    return fn, T * h * D * 2 * 3 + T * D * 2 * 2 + fn_w.numel() * 4, 2.0 * T * (2 + h) * h * h * D


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--rows", type=int, default=32, help="rows per expert for the grouped GEMM cases")
    ap.add_argument("--ctx", type=int, default=2560)
    ap.add_argument("--prefill-tokens", type=int, default=16384)
    ap.add_argument("--graph", action="store_true", help="time a CUDA-graph replay of the case (removes the host launch path from short kernels)")
    ap.add_argument("--scale-format", default="fp32", choices=["fp32", "ue8m0"],
                    help="ue8m0: power-of-two fp8 block scales, applied by the tensor cores (tcgen05 block-scaled MMA) instead of the CUDA cores")
    args = ap.parse_args()
    sm100.lib()
    sm100.set_scale_format(args.scale_format)
    bw, fl, src = peaks()
    cases = build_cases(args)
    names = list(cases) if args.case == "all" else args.case.split(",")
    print(f"{'case':26s} {'time_us':>10s} {'GB/s':>9s} {'frac_bw':>8s} {'TFLOP/s':>9s} {'frac_bf16':>9s}   (fractions of {src} peaks)")
    for n in names:
        if n.startswith("bar:"):
            try:
                fn, nbytes, flops = cases[n]()
                t = timeit(fn, args.iters, args.graph)
            except Exception as e:                 # a library that does not import or does not take this shape here
                print(f"{n:26s} unavailable: {type(e).__name__}: {str(e).splitlines()[0][:120] if str(e) else ''}")
                continue
            print(f"{n:26s} {t * 1e6:10.1f} {nbytes / t / 1e9:9.0f} {nbytes / t / bw:8.2f} {flops / t / 1e12:9.1f} {flops / t / fl:9.2f}")
            del fn
            torch.cuda.empty_cache()
            continue
        fn, nbytes, flops = cases[n]()
        t = timeit(fn, args.iters, args.graph)
        print(f"{n:26s} {t * 1e6:10.1f} {nbytes / t / 1e9:9.0f} {nbytes / t / bw:8.2f} {flops / t / 1e12:9.1f} {flops / t / fl:9.2f}")
        del fn
        torch.cuda.empty_cache()
    st = sm100.kernel_status()
    if st[0] != 0:
        print("kernel status:", st)


if __name__ == "__main__":
    main()
