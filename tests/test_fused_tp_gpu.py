"""Fused tensor-parallel collectives (GEMM -> reduce-scatter through the scatter epilogue, all-gather push, all-reduce)
against NCCL on 2 GPUs of one box: eagerly with changing sizes, and from a captured CUDA graph."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, fp8, q):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        from nanoengine_b200.ops import reference as ref, sm100
        from nanoengine_b200.parallel.fused_tp import FusedTP
        H, Kl = 1024, 512                                   # output width, this rank's share of the contraction
        be = FusedTP(dist.group.WORLD, "attn_tp", H, max_rows=256)
        g = torch.Generator(device=f"cuda:{rank}").manual_seed(7 + rank)
        w = torch.randn(H, Kl, device="cuda", generator=g) * 0.05
        if fp8:
            wq, ws = ref.quant_fp8_block(w)
        else:
            wq, ws = w.to(torch.bfloat16), None
        worst = 0.0

        def rel(a, b):
            return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()

        for T in [128, 7, 256, 1]:
            x = torch.randn(T, Kl, device="cuda", generator=g).to(torch.bfloat16)
            # oracle: local partial product, NCCL all-reduce, own slice
            part = ref.linear(x, wq, ws).float()
            dist.all_reduce(part)
            rpr = -(-T // world)
            want = torch.zeros(rpr, H, device="cuda")
            lo, hi = rank * rpr, min(T, (rank + 1) * rpr)
            if hi > lo:
                want[: hi - lo] = part[lo:hi]
            got = be.gemm_reduce_scatter(x, wq, ws)
            torch.cuda.synchronize()
            assert got.shape == (rpr, H)
            worst = max(worst, rel(got[: max(hi - lo, 0)], want[: max(hi - lo, 0)]) if hi > lo else 0.0)
            # all-gather of the slices gives every rank the full sum
            full = be.all_gather(got)
            torch.cuda.synchronize()
            worst = max(worst, rel(full[:T], part[:T]))
            # all-gather -> GEMM with the gated operand (bf16 weights): every rank multiplies the gathered slices
            if not fp8:
                wcol = (torch.randn(384, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
                prod = be.all_gather_gemm(got, wcol)
                torch.cuda.synchronize()
                worst = max(worst, rel(prod[:T], part[:T].to(torch.bfloat16).float() @ wcol.float().t()))
            # stand-alone all-reduce
            y = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
            wanty = y.float().clone()
            dist.all_reduce(wanty)
            worst = max(worst, rel(be.all_reduce(y), wanty))
        # graph capture: GEMM -> reduce-scatter -> all-gather, replayed with fresh inputs
        T = 64
        xs = torch.randn(T, Kl, device="cuda", generator=g).to(torch.bfloat16)
        be.all_gather(be.gemm_reduce_scatter(xs, wq, ws))
        torch.cuda.synchronize(); dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            yg = be.all_gather(be.gemm_reduce_scatter(xs, wq, ws)).clone()
        for rep in range(3):
            xs.copy_(torch.randn(T, Kl, device="cuda", generator=g).to(torch.bfloat16))
            part = ref.linear(xs, wq, ws).float()
            dist.all_reduce(part)
            gr.replay()
            torch.cuda.synchronize()
            worst = max(worst, rel(yg[:T], part))
        # an ODD number of collectives per graph, replayed an even and an odd number of times, with eager calls in between:
        # the receive buffers alternate per call on the device, so nothing the host fixed at capture may depend on the parity
        if not fp8:
            wcol = (torch.randn(256, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
            warm = be.gemm_reduce_scatter(xs, wq, ws)
            be.all_gather_gemm(warm, wcol)
            be.all_gather(warm)
            torch.cuda.synchronize(); dist.barrier()
            g3 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g3):
                mine = be.gemm_reduce_scatter(xs, wq, ws)              # 1
                y3 = be.all_gather_gemm(mine, wcol)                     # 2
                z3 = be.all_gather(mine)                                # 3
            for rep in range(5):
                xs.copy_(torch.randn(T, Kl, device="cuda", generator=g).to(torch.bfloat16))
                part = ref.linear(xs, wq, ws).float()
                dist.all_reduce(part)
                g3.replay()
                torch.cuda.synchronize()
                worst = max(worst, rel(z3[:T], part), rel(y3[:T], part.to(torch.bfloat16).float() @ wcol.float().t()))
                if rep % 2 == 0:                                        # an eager collective between replays shifts the parity again
                    e = be.all_gather(mine.clone())
                    torch.cuda.synchronize()
                    worst = max(worst, rel(e[:T], part))
        st = sm100.kernel_status()
        dist.barrier()
        q.put((rank, worst, st[0]))
        dist.destroy_process_group()
    except Exception as e:  # surface the failure to the parent instead of hanging it
        import traceback
        q.put((rank, f"{e}\n{traceback.format_exc()}", -1))


@pytest.mark.parametrize("fp8", [True, False])
def test_fused_tp_matches_nccl(fp8):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, fp8, q), daemon=True) for r in range(2)]
    for p in ps:
        p.start()
    res = [q.get(timeout=300) for _ in ps]
    for p in ps:                           # a rank left waiting for a failed peer must not outlive the test
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    for rank, worst, status in res:
        assert status == 0, f"rank {rank}: {worst}"
        assert worst < 2e-2, f"rank {rank}: relative error {worst}"
