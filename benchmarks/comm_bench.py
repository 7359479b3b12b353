"""Fused tensor-parallel collectives against NCCL on the GPUs of one box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 benchmarks/comm_bench.py

For every token count it times a CUDA-graph replay of each sequence (as the decode step runs them; --eager times plain
launches), with CUDA events on the launching stream (max over ranks, median of --iters, 3 warm-up runs, an L2-sized
buffer rewritten between runs):
  gemm_rs   row-parallel fp8 GEMM (K split over the group) + reduce-scatter: fused scatter epilogue vs GEMM then NCCL
  ag        all-gather of [T / world, H] bf16: peer-store push vs NCCL
  ar        all-reduce of [T, H] bf16: push + reduce + push vs NCCL
  ag_gemm   all-gather of [T / world, H] bf16 followed by a column-parallel bf16 GEMM: push + gated GEMM vs NCCL then GEMM
  cp        (--decode-cp) MLA decode of a few long sequences: all pages on one GPU vs pages dealt over the group, partials
            pushed to every peer and merged by log-sum-exp
  ep        (--ep) one expert-parallel MoE layer of the DeepSeek-V3 shape (fp8, 32 experts per GPU, top-8) through the fused
            dispatch / grouped GEMMs / combine, per token count per rank; there is no graph-capturable NCCL composition of it
            (the all-gather form sizes its buffers from a host read-back), so the column beside it is the layer on local experts
  kv_push   (--kv-push, 2 ranks) PD page push of rank 0 into rank 1's pool through a CUDA IPC mapping vs one contiguous
            device-to-device copy of the same bytes
and prints one table from rank 0.  Rooflines: a collective's floor is the bytes crossing NVLink per GPU over --link-gbs
(default 770 GB/s per direction, the peer-copy rate the kv_push case measures with `cudaMemcpyPeer`-style copies); a fused
GEMM + collective is held against max(GEMM FLOPs over --peak-tflops, bytes over the link).
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=9)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--k-total", type=int, default=16384, help="contraction size of the row-parallel GEMM before sharding")
    ap.add_argument("--tokens", default="128,512,2048,8192")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--decode-cp", action="store_true", help="also time context-parallel MLA decode")
    ap.add_argument("--cp-batch", type=int, default=8)
    ap.add_argument("--cp-ctx", type=int, default=65536)
    ap.add_argument("--ep", action="store_true", help="also time one fused expert-parallel MoE layer")
    ap.add_argument("--ep-tokens", default="128,2048")
    ap.add_argument("--kv-push", action="store_true", help="also time the PD page push (needs exactly 2 ranks)")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--peak-tflops", type=float, default=1631.1, help="bf16 GEMM peak for the roofline (fp8 counted at twice this)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from nanoengine_b200.ops import reference as ref, sm100
    from nanoengine_b200.parallel.fused_tp import FusedTP
    H, Kl = args.hidden, args.k_total // world
    toks = [int(t) for t in args.tokens.split(",")]
    be = FusedTP(dist.group.WORLD, "attn_tp", H, max_rows=max(toks))
    w = torch.randn(H, Kl, device="cuda") * 0.05
    wq, ws = ref.quant_fp8_block(w)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn):
        for _ in range(3):
            fn()
        if not args.eager:
            # the decode path replays these sequences from a CUDA graph: time the replay, not the host-side launches
            torch.cuda.synchronize(); dist.barrier()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            fn = gr.replay
            fn(); torch.cuda.synchronize(); dist.barrier()
        ts = []
        for _ in range(args.iters):
            flush.fill_(1)
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); e1.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        ts.sort()
        return ts[len(ts) // 2] * 1e3           # us

    rows = []
    for T in toks:
        x = torch.randn(T, Kl, device="cuda").to(torch.bfloat16)
        rpr = -(-T // world)
        out_rs = torch.empty(rpr, H, dtype=torch.bfloat16, device="cuda")

        def nccl_gemm_rs():
            y = sm100.linear(x, wq, ws)
            dist.reduce_scatter_tensor(out_rs, y[: rpr * world].contiguous() if y.shape[0] == rpr * world else torch.nn.functional.pad(y, (0, 0, 0, rpr * world - T)))

        t_f = timeit(lambda: be.gemm_reduce_scatter(x, wq, ws))
        t_n = timeit(nccl_gemm_rs)
        t_g = timeit(lambda: sm100.linear(x, wq, ws))
        link_us = (world - 1) * rpr * H * 2 / (args.link_gbs * 1e3)                     # partial rows leaving this GPU
        flop_us = 2.0 * T * H * Kl / (2 * args.peak_tflops * 1e6)                        # fp8 operands
        floor = max(link_us, flop_us)
        rows.append(("gemm_rs", T, t_f, t_n, f"GEMM alone {t_g:7.1f}; floor max(link {link_us:.1f}, flops {flop_us:.1f}) -> {floor / t_f:4.2f} of roofline"))
        sl = torch.randn(rpr, H, device="cuda").to(torch.bfloat16)
        full = torch.empty(rpr * world, H, dtype=torch.bfloat16, device="cuda")
        t_f = timeit(lambda: be.all_gather(sl))
        t_n = timeit(lambda: dist.all_gather_into_tensor(full, sl))
        nbytes = rpr * (world - 1) * H * 2
        rows.append(("ag", T, t_f, t_n, f"link floor {nbytes / 770e9 * 1e6:6.1f}"))
        wcol = (torch.randn(2048, H, device="cuda") * 0.05).to(torch.bfloat16)
        t_f = timeit(lambda: be.all_gather_gemm(sl, wcol))

        def nccl_ag_gemm():
            dist.all_gather_into_tensor(full, sl)
            return sm100.linear(full, wcol)

        t_n = timeit(nccl_ag_gemm)
        flop_us = 2.0 * rpr * world * H * 2048 / (args.peak_tflops * 1e6)
        rows.append(("ag_gemm", T, t_f, t_n, f"floor max(link {nbytes / (args.link_gbs * 1e3):.1f}, flops {flop_us:.1f}) -> "
                                               f"{max(nbytes / (args.link_gbs * 1e3), flop_us) / t_f:4.2f} of roofline"))
        y = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        t_f = timeit(lambda: be.all_reduce(y))
        t_n = timeit(lambda: dist.all_reduce(y.clone()))
        rows.append(("ar", T, t_f, t_n, f"link floor {2 * nbytes / 770e9 * 1e6:6.1f}"))
    if args.decode_cp:
        from nanoengine_b200.ops import sm100_attn
        from nanoengine_b200.parallel.decode_cp import DecodeCP, shard_pages
        B, ctx, Hh, bs = args.cp_batch, args.cp_ctx, 128, 64
        npg = -(-ctx // bs)
        cache = (torch.randn(B * npg + 1, bs, 576, device="cuda") * 0.5).to(torch.float8_e4m3fn)
        tables = [list(range(b * npg, (b + 1) * npg)) for b in range(B)]
        bt_full = torch.tensor(tables, dtype=torch.int32, device="cuda")
        cl_full = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        loc = [shard_pages(t, ctx, bs, world, rank) for t in tables]
        lw = max(len(p) for p, _ in loc)
        bt_loc = torch.tensor([p + [0] * (lw - len(p)) for p, _ in loc], dtype=torch.int32, device="cuda")
        cl_loc = torch.tensor([n for _, n in loc], dtype=torch.int32, device="cuda")
        cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        q = torch.randn(B, Hh, 576, device="cuda").to(torch.bfloat16)
        cp = DecodeCP(dist.group.WORLD, Hh, 512, max_tokens=B, local_splits=max(2, 16 // world))
        sc = 576 ** -0.5
        t_full = timeit(lambda: sm100_attn.mla_attention_paged(q, cache, bt_full, cu, cl_full, sc, 512))
        t_cp = timeit(lambda: cp.attention(q, cache, bt_loc, cu, cl_loc, sc))
        rows.append(("cp", B, t_cp, t_full, f"ctx {ctx}; 'nccl' column = all pages on one GPU"))
    if args.ep:
        from nanoengine_b200.models.layers import RoutedExperts
        from nanoengine_b200.parallel.dist import ParallelSpec, init_dist_context
        from nanoengine_b200.parallel.fused_moe import FusedEP
        d = init_dist_context(ParallelSpec(attention_dp=world, ffn_ep=world), rank, world, f"cuda:{torch.cuda.current_device()}")
        Hm, I, El, K = 7168, 2048, 32, 8
        E = El * world
        ex = RoutedExperts(E, Hm, I, torch.bfloat16, "cuda", "fp8")
        # weights only need the right size and a sane scale for timing
        ex.gate_up_proj.view(torch.uint8).random_(0, 120); ex.down_proj.view(torch.uint8).random_(0, 120)
        ex.gate_up_scale.fill_(1e-3); ex.down_scale.fill_(1e-3)
        ep_toks = [int(t) for t in args.ep_tokens.split(",")]
        fe = FusedEP(d.group("ffn_ep"), d.ep_rank, world, E, Hm, I, K, max_tokens=max(ep_toks), fp8=True)
        g = torch.Generator(device="cuda").manual_seed(5 + rank)
        for T in ep_toks:
            xt = torch.randn(T, Hm, device="cuda", generator=g).to(torch.bfloat16)
            idx = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(T)]).to(torch.int32)
            wt = torch.rand(T, K, device="cuda", generator=g)
            t_f = timeit(lambda: fe.forward(ex, xt, idx, wt))
            lidx = (idx % El + rank * El).to(torch.int32)               # the same load on local experts only: no NVLink traffic
            t_l = timeit(lambda: ex(xt, lidx, wt))
            out_b = T * K * (world - 1) / world * (Hm + Hm // 128 * 4 + 8)            # fp8 rows + scales + info leaving this GPU
            back_b = T * K * (world - 1) / world * Hm * 2                               # bf16 rows coming back
            link_us = max(out_b, back_b) / (args.link_gbs * 1e3)
            flop_us = 2.0 * T * K * Hm * 3 * I / (2 * args.peak_tflops * 1e6)
            wbytes_us = El * 3 * I * Hm / 6456.8e3                                      # every local expert's weights read once
            floor = max(link_us, flop_us, wbytes_us)
            rows.append(("ep", T, t_f, t_l, f"'nccl' column = same layer on local experts; per rank {out_b / 1e6:.1f} MB out + {back_b / 1e6:.1f} MB back; "
                                              f"floor max(link {link_us:.1f}, flops {flop_us:.1f}, weights {wbytes_us:.1f}) -> {floor / t_f:4.2f} of roofline"))
    if args.kv_push and world == 2:
        import ctypes as _c
        from nanoengine_b200.parallel.kv_transfer import export_tensor, open_tensor
        L, pages, page_bytes = 61, 256, 64 * 576                                         # 256 pages = 16K tokens of fp8 MLA rows
        pool = torch.zeros(L, pages + 1, page_bytes, dtype=torch.uint8, device="cuda")
        flags = torch.zeros(64, dtype=torch.int32, device="cuda")
        desc = [export_tensor(pool.view(-1), False), export_tensor(flags, False)] if rank == 1 else [None, None]
        dist.broadcast_object_list(desc, src=1)
        if rank == 0:
            rpool, rflags = open_tensor(desc[0]), open_tensor(desc[1])
            sb = torch.randperm(pages, device="cuda").to(torch.int32)
            db = torch.randperm(pages, device="cuda").to(torch.int32)
            fi = torch.zeros(1, dtype=torch.int32, device="cuda")
            ctr = torch.zeros(1, dtype=torch.int32, device="cuda")
            stride = (pages + 1) * page_bytes

            def push():
                sm100._ck(sm100.lib().ne_kv_push(sm100._p(pool), _c.c_void_p(rpool.data_ptr()), _c.c_longlong(stride), _c.c_longlong(stride),
                                                 _c.c_int(page_bytes), sm100._p(sb), sm100._p(db), _c.c_int(pages), _c.c_int(L),
                                                 _c.c_void_p(rflags.data_ptr()), sm100._p(fi), _c.c_int(1), _c.c_int(1), sm100._p(ctr), sm100._st()), "ne_kv_push")

            def copy():
                rpool[: L * pages * page_bytes].copy_(pool.view(-1)[: L * pages * page_bytes], non_blocking=True)
        else:
            push = copy = (lambda: None)
        saved, args.eager = args.eager, True                                             # one-sided: nothing to capture on the idle rank
        t_p, t_c = timeit(push), timeit(copy)
        args.eager = saved
        nb = L * pages * page_bytes
        rows.append(("kv_push", pages, t_p, t_c, f"{nb / 1e6:.0f} MB ({L} layers x {pages} scattered pages): push {nb / t_p / 1e3:.0f} GB/s, "
                                                  f"contiguous peer copy {nb / t_c / 1e3:.0f} GB/s ('nccl' column)"))
    if rank == 0:
        print(f"world={world} hidden={H} K/rank={Kl}; times in us (max over ranks)")
        print(f"{'op':8s} {'tokens':>7s} {'fused':>9s} {'nccl':>9s} {'speedup':>8s}   note")
        for op, T, a, b, note in rows:
            print(f"{op:8s} {T:7d} {a:9.1f} {b:9.1f} {b / a:8.2f}   {note}")
        st = sm100.kernel_status()
        if st[0]:
            print("kernel status:", st)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
