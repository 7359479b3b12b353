"""In-switch (multimem) all-reduce / reduce-scatter / all-gather against NCCL on 2 GPUs, eagerly and from a CUDA graph.
The ranks opt in to the multicast binding (NE_NVLS=1); where the fabric offers no multicast object the case reports that
and passes without running the kernels.  Both ranks stay alive until both are done, so no multicast object is torn down
under a peer."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NE_NVLS="1")
        os.environ.pop("TORCH_SYMM_MEM_DISABLE_MULTICAST", None)
        torch.cuda.set_device(rank)
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        from nanoengine_b200.ops import sm100
        from nanoengine_b200.parallel.fused_tp import NvlsCollectives
        H = 1024
        nv = NvlsCollectives(dist.group.WORLD, H, max_rows=512)
        if not nv.available:
            dist.barrier()
            q.put((rank, "no multicast object on this fabric", 0))
            dist.destroy_process_group()
            return
        g = torch.Generator(device=f"cuda:{rank}").manual_seed(3 + rank)
        worst = 0.0

        def rel(a, b):
            return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()

        for T in (128, 7, 512, 2):
            x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
            want = x.float().clone()
            dist.all_reduce(want)
            worst = max(worst, rel(nv.all_reduce(x), want))
            if T % world == 0:
                got = nv.reduce_scatter(x)
                per = T // world
                worst = max(worst, rel(got, want[rank * per:(rank + 1) * per]))
            if T * world <= 512:
                full = torch.empty(T * world, H, dtype=torch.bfloat16, device="cuda")
                dist.all_gather_into_tensor(full, x)
                worst = max(worst, rel(nv.all_gather(x), full))
            torch.cuda.synchronize()
        x = torch.randn(64, H, device="cuda", generator=g).to(torch.bfloat16)
        nv.all_reduce(x)
        torch.cuda.synchronize(); dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            y = nv.all_gather(nv.reduce_scatter(nv.all_reduce(x)))
        for _ in range(3):
            x.copy_(torch.randn(64, H, device="cuda", generator=g).to(torch.bfloat16))
            want = x.float().clone()
            dist.all_reduce(want)                       # sum over ranks ...
            want2 = want.to(torch.bfloat16).float().clone()
            dist.all_reduce(want2)                      # ... and the reduce-scatter sums the (identical) results once more
            gr.replay()
            torch.cuda.synchronize()
            worst = max(worst, rel(y, want2))
        st = sm100.kernel_status()
        dist.barrier()
        q.put((rank, worst, st[0]))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        import traceback
        q.put((rank, f"{e}\n{traceback.format_exc()}", -1))


def test_multimem_collectives_match_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in ps:
        p.start()
    try:
        res = [q.get(timeout=240) for _ in ps]
    finally:
        for p in ps:
            p.join(timeout=60)
            if p.is_alive():
                p.terminate()
    for rank, worst, status in res:
        assert status == 0, f"rank {rank}: {worst}"
        if isinstance(worst, str):
            print(f"rank {rank}: {worst}")
        else:
            assert worst < 2e-2, f"rank {rank}: relative error {worst}"
