"""Context-parallel MLA decode on 2 GPUs: pages dealt round-robin, local split-KV partials, peer-store gather, one merge -
against the same attention computed over all pages on one GPU."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q_out):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        from nanoengine_b200.ops import reference as ref, sm100, sm100_attn
        from nanoengine_b200.parallel.decode_cp import DecodeCP, shard_pages
        H, R, bs = 16, 512, 64
        ctx_lens = [1000, 30, 64, 129, 4000]
        B = len(ctx_lens)
        g = torch.Generator(device="cuda").manual_seed(11)           # the same data on every rank
        n_pages = [-(-c // bs) for c in ctx_lens]
        cache = (torch.randn(sum(n_pages) + 1, bs, 576, device="cuda", generator=g) * 0.5).to(torch.float8_e4m3fn)
        tables, nxt = [], 0
        for n in n_pages:
            tables.append(list(range(nxt, nxt + n))); nxt += n
        width = max(n_pages)
        bt_full = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32, device="cuda")
        cl_full = torch.tensor(ctx_lens, dtype=torch.int32, device="cuda")
        local = [shard_pages(t, c, bs, world, rank) for t, c in zip(tables, ctx_lens)]
        assert sum(shard_pages(tables[0], ctx_lens[0], bs, world, r)[1] for r in range(world)) == ctx_lens[0]
        lw = max(1, max(len(p) for p, _ in local))
        bt_loc = torch.tensor([p + [0] * (lw - len(p)) for p, _ in local], dtype=torch.int32, device="cuda")
        cl_loc = torch.tensor([n for _, n in local], dtype=torch.int32, device="cuda")
        cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        cp = DecodeCP(dist.group.WORLD, H, R, max_tokens=8, local_splits=2)
        scale = 576 ** -0.5
        worst = 0.0
        for it in range(3):                                           # three rounds: both parities of the gather buffers
            q = torch.randn(B, H, 576, device="cuda", generator=g).to(torch.bfloat16)
            want = sm100_attn.mla_attention_paged(q, cache, bt_full, cu, cl_full, scale, R)
            got = cp.attention(q, cache, bt_loc, cu, cl_loc, scale)
            torch.cuda.synchronize()
            worst = max(worst, ((got.float() - want.float()).norm() / want.float().norm()).item())
            if it == 0:                                               # and against the plain fp32 statement
                oracle = ref.mla_attention_paged(q.cpu(), cache.cpu(), bt_full.cpu(), cu.cpu(), cl_full.cpu(), scale, R)
                worst = max(worst, ((got.float().cpu() - oracle.float()).norm() / oracle.float().norm()).item())
        st = sm100.kernel_status()
        dist.barrier()
        q_out.put((rank, worst, st[0]))
        dist.destroy_process_group()
    except Exception as e:
        import traceback
        q_out.put((rank, f"{e}\n{traceback.format_exc()}", -1))


def test_context_parallel_decode_matches_single_gpu():
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
    res = [q.get(timeout=300) for _ in ps]
    for p in ps:                           # a rank left waiting for a failed peer must not outlive the test
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    for rank, worst, status in res:
        assert status == 0, f"rank {rank}: {worst}"
        assert worst < 3e-2, f"rank {rank}: relative error {worst}"
