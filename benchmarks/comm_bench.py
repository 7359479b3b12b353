"""Fused tensor-parallel collectives against NCCL on the GPUs of one box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 benchmarks/comm_bench.py

For every token count it times a CUDA-graph replay of each sequence (as the decode step runs them; --eager times plain
launches), with CUDA events on the launching stream (max over ranks, median of --iters, 3 warm-up runs, an L2-sized
buffer rewritten between runs):
  gemm_rs   row-parallel fp8 GEMM (K split over the group) + reduce-scatter: fused scatter epilogue vs GEMM then NCCL
  ag        all-gather of [T / world, H] bf16: peer-store push vs NCCL
  ar        all-reduce of [T, H] bf16: push + reduce + push vs NCCL
  cp        (--decode-cp) MLA decode of a few long sequences: all pages on one GPU vs pages dealt over the group, partials
            pushed to every peer and merged by log-sum-exp
and prints one table from rank 0.  The roofline for the collectives is bytes crossing NVLink per GPU / 770 GB/s.
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
        rows.append(("gemm_rs", T, t_f, t_n, f"GEMM alone {t_g:7.1f}"))
        sl = torch.randn(rpr, H, device="cuda").to(torch.bfloat16)
        full = torch.empty(rpr * world, H, dtype=torch.bfloat16, device="cuda")
        t_f = timeit(lambda: be.all_gather(sl))
        t_n = timeit(lambda: dist.all_gather_into_tensor(full, sl))
        nbytes = rpr * (world - 1) * H * 2
        rows.append(("ag", T, t_f, t_n, f"link floor {nbytes / 770e9 * 1e6:6.1f}"))
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
