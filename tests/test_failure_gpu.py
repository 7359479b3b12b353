"""Failure detection on GPUs, without faulting one: two ranks (child processes, one GPU each, NVLS off, peer-memory kernels
on plain loads and stores) decode through the fused expert-parallel path; rank 1 leaves BETWEEN steps with nothing in flight.
Rank 0 must stop at its next per-step host rendezvous with an error, launch nothing after that, and keep a usable context.
A device wait that runs out is covered separately: a flag nobody raises, a one-second limit, a status word the host reads."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    try:
        from nanoengine_b200 import Config, LLM, SamplingParams
        from nanoengine_b200.engine.executor import ExecutorError
        from nanoengine_b200.ops import sm100
        cfg = Config(model="tiny-deepseek-v3", dtype="bfloat16", device="cuda", kvcache_block_size=64, max_num_seqs=4, num_kvcache_blocks=32,
                     attention_dp=world, ffn_ep=world, executor_backend="spmd", peer_timeout_s=10.0, seed=rank, kernel_status_every=1)
        llm = LLM(cfg)
        g = torch.Generator().manual_seed(rank)
        llm.add_request(torch.randint(0, 1024, (20,), generator=g).tolist(), SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True))
        steps = 0
        try:
            while steps < 30:
                llm.step()
                steps += 1
                if rank == 1 and steps == 3:
                    torch.cuda.synchronize()
                    llm.shutdown()                      # between steps: announce and leave
                    q.put((rank, "left", steps, 0))
                    return
            q.put((rank, "finished", steps, 0))
        except ExecutorError:
            torch.cuda.synchronize()
            alive = float((torch.ones(1024, device="cuda") * 2).sum())          # the context still works
            q.put((rank, "peer-lost", steps, alive, sm100.kernel_status()[0]))
    except Exception as e:
        import traceback
        q.put((rank, "error", f"{e}\n{traceback.format_exc()}", 0))


def test_rank_leaving_between_steps_is_detected_before_the_next_launch():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in ps:
        p.start()
    res = {r[0]: r for r in (q.get(timeout=300) for _ in ps)}
    for p in ps:                           # a rank left waiting for a failed peer must not outlive the test
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    assert res[1][1] == "left", res
    assert res[0][1] == "peer-lost", res
    assert 3 <= res[0][2] <= 5 and res[0][3] == 2048.0 and res[0][4] == 0, res


def test_device_wait_runs_out_and_reports():
    """A peer flag nobody raises: the wait kernel gives up after its (short) limit, the status word says so, the context lives."""
    if torch.cuda.device_count() < 1:
        pytest.skip("needs a GPU")
    import ctypes as c
    from nanoengine_b200.ops import sm100
    lib = sm100.lib()
    sm100.clear_kernel_status()
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    flags[2] = 5                                                    # one producer did finish
    idx = torch.tensor([2, 3], dtype=torch.int32, device="cuda")
    out = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    rc = lib.ne_kv_wait(c.c_void_p(flags.data_ptr()), c.c_void_p(idx.data_ptr()), c.c_int(2), c.c_int(5), c.c_void_p(out.data_ptr()),
                        c.c_int(1 << 16), sm100._st())
    torch.cuda.synchronize()
    st = sm100.kernel_status()
    assert rc == 0 and out.tolist() == [1, 0] and st[0] != 0, (out.tolist(), st)
    sm100.clear_kernel_status()
    assert float(torch.ones(8, device="cuda").sum()) == 8.0
