"""Prefill -> decode KV push between two GPUs of one box, as two processes: the decode process publishes its page pool, flag
words and MTP hand-off table as CUDA IPC handles, the prefill process maps them and pushes the pages of finished prompts
with peer stores (`ne_kv_push`), the decode process admits each request once its completion flag has arrived.  The decoded
tokens must equal those of a hybrid engine on one GPU.  A request whose push is never issued is failed alone by the bounded
wait; nothing on either GPU faults.  NVLS stays off and no multicast object is created."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(mode, **kw):
    from nanoengine_b200 import Config
    from nanoengine_b200.models.config import tiny_deepseek_v3
    mc = tiny_deepseek_v3(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024, q_lora_rank=256, kv_lora_rank=512,
                          qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_attention_heads=16, quant="fp8")
    base = dict(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kv_cache_dtype="fp8",
                kvcache_block_size=64, num_kvcache_blocks=48, max_num_seqs=8, mode=mode, seed=0)
    base.update(kw)
    return Config(**base)


def _prompts():
    g = torch.Generator().manual_seed(33)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (150, 70, 129)]


def _recv(conn, timeout=180.0):
    """A peer that failed never answers: give up instead of waiting for the test's own limit."""
    if not conn.poll(timeout):
        raise TimeoutError("the other PD process stopped answering")
    return conn.recv()


def _prefill_proc(conn, q):
    # both GPUs stay visible: mapping the decode GPU's memory needs that device in this process too
    os.environ.update(CUDA_VISIBLE_DEVICES="0,1", LOCAL_RANK="0", NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    try:
        torch.cuda.set_device(0)
        from nanoengine_b200 import LLM, SamplingParams
        llm = LLM(_cfg("prefill", engine_id="p0"))
        runner = llm.engine.executor.runner
        pools, dinfo = _recv(conn)
        assert runner.pd_open_pool("d0", pools) == 1
        conn.send(llm.engine.engine_info())
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
        for round_ in range(2):
            blobs = llm.generate(_prompts(), sp, return_serialized=True)
            conn.send(blobs)
            while True:
                msg = _recv(conn)
                if msg[0] == "push":
                    reqs = msg[1]
                    drop = msg[2]                                   # host-side fault injection: requests the producer never runs
                    sizes = runner.pd_push("d0", [r for i, r in enumerate(reqs) if i not in drop])
                    it = iter(sizes)
                    conn.send([0 if i in drop else next(it) for i in range(len(reqs))])
                elif msg[0] == "free":
                    llm.free_to_be_migrated_ids(msg[1])
                    break
        torch.cuda.synchronize()
        from nanoengine_b200.ops import sm100
        q.put(("prefill", "ok", sm100.kernel_status()[0]))
    except Exception as e:
        import traceback
        q.put(("prefill", f"{e}\n{traceback.format_exc()}", -1))


def _decode_proc(conn, q):
    os.environ.update(CUDA_VISIBLE_DEVICES="0,1", NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    try:
        torch.cuda.set_device(1)
        os.environ["LOCAL_RANK"] = "1"
        from nanoengine_b200 import LLM, RequestMigrate, SamplingParams
        from nanoengine_b200.ops import sm100
        from nanoengine_b200.parallel.kv_transfer import KVMigrator, PeerPushTransport
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
        hyb = LLM(_cfg("hybrid"))
        want = {o["seq_id"]: o["token_ids"] for o in hyb.generate(_prompts(), sp)}
        del hyb
        torch.cuda.empty_cache()
        llm = LLM(_cfg("decode", engine_id="d0"))
        runner = llm.engine.executor.runner
        conn.send(([runner.pd_export_pool(direct=False)], llm.engine.engine_info()))
        pinfo = _recv(conn)
        drop = set()

        def pusher(reqs):
            conn.send(("push", reqs, drop))
            return _recv(conn)

        def waiter(dst_dp, flags, epochs):
            return runner.pd_wait(dst_dp, flags, epochs, spin_limit=1 << 21)

        llm.engine.migrator = KVMigrator(PeerPushTransport(pusher, waiter), llm.engine.engine_info(), pinfo)
        results = []
        for round_ in range(2):
            drop.clear()
            if round_ == 1:
                drop.add(1)                                         # the second request of this round is never pushed
            firsts = {}
            for b in _recv(conn):
                sid, first = RequestMigrate.from_bytes(b).metadata
                firsts[sid] = first
                llm.add_request_payload(b)
            outs = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in llm.generate()}
            conn.send(("free", list(firsts)))
            results.append(outs)
        free = llm.engine.scheduler.num_free_blocks()
        q.put(("decode", (want, results, free), sm100.kernel_status()[0]))
    except Exception as e:
        import traceback
        q.put(("decode", f"{e}\n{traceback.format_exc()}", -1))


def test_prefill_gpu_pushes_pages_into_the_decode_gpus_pool():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    a, b = ctx.Pipe()
    q = ctx.Queue()
    ps = [ctx.Process(target=_prefill_proc, args=(a, q), daemon=True), ctx.Process(target=_decode_proc, args=(b, q), daemon=True)]
    for p in ps:
        p.start()
    try:
        res = dict((r[0], r) for r in (q.get(timeout=420) for _ in ps))
    finally:
        for p in ps:                       # a child still blocked on its pipe must not keep the test process alive
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    assert res["prefill"][2] == 0 and res["decode"][2] == 0, f"prefill: {res['prefill'][1]}\ndecode: {res['decode'][1]}"
    want, results, free = res["decode"][1]
    ids = sorted(want)
    # first pass: every request decodes to the hybrid engine's tokens (sequence ids differ between engines, order does not)
    got0 = results[0]
    assert [got0[k] for k in sorted(got0)] == [want[k] for k in ids]
    # second pass: the request whose push never ran is dropped, the others still match; its pages went back to the pool
    got1 = results[1]
    assert len(got1) == 2
    assert [got1[k] for k in sorted(got1)] == [want[ids[0]], want[ids[2]]]
    assert free == 48


def test_pd_between_serving_processes_named_by_pd_peers():
    """The deployment form: a prefill engine process with a fixed ZMQ endpoint, a decode engine process whose `pd_peers` names it
    (it publishes its pools to the prefill engine when it starts), each behind the HTTP app.  A request prefilled through one app
    and continued through the other, the way the gateway forwards it, reads the same tokens as a hybrid engine."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import tempfile
    from starlette.testclient import TestClient
    from nanoengine_b200.server.engine_server import EngineClient, spawn_backend
    from nanoengine_b200.server.openai_server import create_app
    from nanoengine_b200.server.tokenizer import ByteTokenizer
    os.environ.update(NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    ep_p = f"ipc://{tempfile.gettempdir()}/ne-test-pd-p0-{os.getpid()}.sock"
    procs, clients = [], []

    def start(cfg, mode, local_rank, endpoint=None):
        old = os.environ.get("LOCAL_RANK")
        os.environ["LOCAL_RANK"] = str(local_rank)
        try:
            proc, ep = spawn_backend(cfg, endpoint=endpoint)
        finally:
            if old is None:
                os.environ.pop("LOCAL_RANK", None)
            else:
                os.environ["LOCAL_RANK"] = old
        cli = EngineClient(ep, proc)
        procs.append(proc); clients.append(cli)
        return create_app(cli, ByteTokenizer(1024), "m", mode=mode)

    try:
        app_h = start(_cfg("hybrid", engine_id="h0"), "hybrid", 0)
        app_p = start(_cfg("prefill", engine_id="p0", engine_endpoint=ep_p), "prefill", 0, ep_p)
        app_d = start(_cfg("decode", engine_id="d0", pd_peers={"p0": ep_p}), "decode", 1)
        prompt = _prompts()[0]
        base = {"prompt": prompt, "max_tokens": 6, "temperature": 0.0, "ignore_eos": True, "logprobs": True}
        with TestClient(app_h) as th, TestClient(app_p) as tp, TestClient(app_d) as td:
            want = th.post("/v1/completions", json=base).json()["choices"][0]
            r = tp.post("/v1/completions", json=dict(base, kv_transfer_params={"do_remote_decode": True})).json()
            kv = r["kv_transfer_params"]
            assert kv["migration"] and kv["first_token"] is not None and kv["engine_id"] == "p0"
            got = td.post("/v1/completions", json=dict(base, kv_transfer_params={"migration": kv["migration"], "first_token": kv["first_token"]}))
            assert got.status_code == 200, got.text
            got = got.json()["choices"][0]
            assert tp.post("/pd/free", json={"seq_ids": [kv["seq_id"]]}).json()["freed"] == 1
        assert got["text"] == want["text"]
        assert len(got["logprobs"]["tokens"]) >= 5 and got["logprobs"]["tokens"][-5:] == want["logprobs"]["tokens"][-5:]
    finally:
        for c in clients:
            c.destroy()
        for p in procs:
            if p.is_alive():
                p.terminate()
            p.join(timeout=20)
