"""Two GPUs, engines under CUDA graphs with collectives inside the graphs: Qwen3-MoE with tensor-parallel attention (an odd
number of collectives per forward pass) interleaving prefills and decode steps, and DeepSeek-style DP2 + EP2 where the two
ranks hold different numbers of requests (so they replay different batch-size buckets, and one of them runs out of requests
and continues on dummy batches).  Every rank must produce the tokens of the same engine run eagerly."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(rank, world, port, case, eager, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    try:
        from nanoengine_b200 import Config, LLM, SamplingParams
        from nanoengine_b200.models.config import PRESETS
        from nanoengine_b200.ops import sm100
        if case in ("qwen3_tp2", "qwen3_tp2_ffn_tp2", "qwen3_dense_tp2_ffn_tp2"):
            ffn_tp = case != "qwen3_tp2"                                # experts / dense MLP split by intermediate columns, vocab-parallel head
            mc = PRESETS["qwen3-235b-a22b"](num_hidden_layers=3, hidden_size=1024, num_attention_heads=16, num_key_value_heads=4, head_dim=128,
                                            n_routed_experts=8, moe_intermediate_size=256, num_experts_per_tok=2, vocab_size=2048,
                                            max_position_embeddings=4096)
            if case == "qwen3_dense_tp2_ffn_tp2":
                mc.n_routed_experts, mc.intermediate_size = 0, 2048
            cfg = Config(model="qwen3-235b-a22b", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kvcache_block_size=64,
                         num_kvcache_blocks=64, max_num_seqs=8, attention_tp=world, ffn_ep=1 if ffn_tp else world, ffn_tp=world if ffn_tp else 1,
                         executor_backend="spmd", seed=0,
                         enforce_eager=eager, peer_timeout_s=60.0)
            prompts = [torch.randint(0, 2048, (n,), generator=torch.Generator().manual_seed(5 + i)).tolist() for i, n in enumerate((40, 70, 9))]
            late = [torch.randint(0, 2048, (33,), generator=torch.Generator().manual_seed(99)).tolist()]
            max_tokens = 10
        else:
            cfg = Config(model="tiny-deepseek-v3", dtype="bfloat16", device="cuda", kvcache_block_size=64, max_num_seqs=8, num_kvcache_blocks=64,
                         attention_dp=world, ffn_ep=world, executor_backend="spmd", seed=0, enforce_eager=eager, peer_timeout_s=60.0)
            n_req = 5 if rank == 0 else 1                          # unequal loads: buckets 8 and 1, then rank 1 idles on dummy batches
            prompts = [torch.randint(0, 1024, (20 + 7 * i,), generator=torch.Generator().manual_seed(rank * 50 + i)).tolist() for i in range(n_req)]
            late = []
            max_tokens = 10 if rank == 0 else 6
        llm = LLM(cfg)
        sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
        ids = [llm.add_request(p, sp) for p in prompts]
        out = {}
        for step in range(40):                                      # the same number of steps on every rank: each one is a host rendezvous
            for so in llm.step():
                out.setdefault(so.seq_id, []).extend(so.token_ids)
            if late and step == 4:                                  # a prefill arriving between decode steps
                ids.append(llm.add_request(late.pop(), sp))
        assert llm.engine.is_finished()
        if not eager:
            assert llm.engine.executor.runner.graphs is not None and llm.engine.executor.runner.graphs.graphs
        torch.cuda.synchronize()
        q.put((rank, [out[i] for i in ids], sm100.kernel_status()[0]))
        llm.shutdown()
    except Exception as e:
        import traceback
        q.put((rank, f"{e}\n{traceback.format_exc()}", -1))


def _launch(case, eager):
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_run, args=(r, 2, port, case, eager, q), daemon=True) for r in range(2)]
    for p in ps:
        p.start()
    try:
        res = [q.get(timeout=300) for _ in ps]
    finally:
        for p in ps:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    for rank, toks, status in res:
        assert status == 0, f"rank {rank} ({'eager' if eager else 'graphs'}): {toks}"
    return {rank: toks for rank, toks, _ in res}


@pytest.mark.parametrize("case", ["qwen3_tp2", "qwen3_tp2_ffn_tp2", "qwen3_dense_tp2_ffn_tp2", "deepseek_dp2_ep2_unequal"])
def test_graphs_with_collectives_match_eager(case):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    eager, graph = _launch(case, True), _launch(case, False)
    for rank in (0, 1):
        a_all, b_all = eager[rank], graph[rank]
        assert len(a_all) == len(b_all) and all(len(a) == len(b) for a, b in zip(a_all, b_all))
        same = sum(a == b for a, b in zip(a_all, b_all))
        assert same >= len(a_all) - 1 and all(a[:3] == b[:3] for a, b in zip(a_all, b_all)), (rank, a_all, b_all)
    if case.startswith("qwen3"):
        assert graph[0] == graph[1]                                     # TP ranks serve the same requests
