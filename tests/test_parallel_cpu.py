"""Multi-rank layouts on CPU (gloo) ranks: the outputs must equal the single-rank run.

* attention-DP 2 + expert-parallel 2 (DeepSeek-V3 style): the all-gather EP oracle path, dummy batches for the idle rank
* attention-TP 2 + expert-parallel 2 (Qwen3-MoE style): token-sliced residual stream, head-sharded qkv, reduce-scatter
* a worker that dies is noticed by the executor instead of hanging the controller
"""
import pytest
import torch

from nanoengine_b200 import Config, LLM, SamplingParams
from nanoengine_b200.models.config import ModelConfig


def _prompts(n, length, seed, vocab):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _run(cfg, prompts, sp):
    llm = LLM(cfg)
    try:
        return {o["seq_id"]: o["token_ids"] for o in llm.generate(prompts, sp)}
    finally:
        llm.shutdown()


def test_dp2_ep2_matches_single_rank():
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64)
    prompts = _prompts(3, 24, 1, 1024)       # odd count: one DP rank runs a dummy batch on some steps
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    want = _run(Config(**base), prompts, sp)
    got = _run(Config(**base, attention_dp=2, ffn_ep=2), prompts, sp)
    assert got == want


def test_dp2_ep2_nvfp4_experts_match_single_rank():
    """NVFP4 routed experts under attention-DP + EP: every rank holds half of the experts in the packed form, the GEMM-1 activation
    scale is agreed on with a MAX over the EP group when the experts are first used, and the tokens equal the single-rank run."""
    from nanoengine_b200.models.config import tiny_deepseek_v3
    mc = tiny_deepseek_v3(moe_intermediate_size=256, intermediate_size=512, quant="nvfp4")
    base = dict(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=16,
                max_num_seqs=8, num_kvcache_blocks=64)
    prompts = _prompts(3, 24, 4, 1024)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = _run(Config(**base), prompts, sp)
    got = _run(Config(**base, attention_dp=2, ffn_ep=2), prompts, sp)
    assert got == want


def test_dp2_ep2_hybrid_delta_net_moe_matches_single_rank():
    """The hybrid family under attention-DP + EP: every rank keeps its own recurrent-state pool; a rank without work runs a dummy
    batch on the scratch state slot."""
    from nanoengine_b200.models.config import tiny_qwen3_5
    base = dict(model="tiny-qwen3.5", model_config=tiny_qwen3_5(moe=True), dummy_weight=True, dtype="float32", device="cpu",
                kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64)
    prompts = _prompts(3, 40, 2, 512)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = _run(Config(**base), prompts, sp)
    got = _run(Config(**base, attention_dp=2, ffn_ep=2), prompts, sp)
    assert got == want


def test_dp2_ep2_deepseek_v4_matches_single_rank():
    """DeepSeek-V4 under attention-DP + EP: every rank keeps its own window / pooled-row pages and compressor carries; hash-routed
    and score-routed layers both dispatch over the EP group; an idle rank's dummy batch uses the spare state slot."""
    from nanoengine_b200.models.config import tiny_deepseek_v4
    base = dict(model="tiny-dsv4", model_config=tiny_deepseek_v4(head_dim=80), dummy_weight=True, dtype="float32", device="cpu",
                kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64)
    prompts = _prompts(3, 40, 5, 512)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = _run(Config(**base), prompts, sp)
    got = _run(Config(**base, attention_dp=2, ffn_ep=2), prompts, sp)
    assert got == want


def _qwen_cfg():
    return ModelConfig(architecture="Qwen3MoeForCausalLM", vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=8,
                       num_key_value_heads=2, head_dim=16, rope_theta=1e6, max_position_embeddings=1024, intermediate_size=256,
                       n_routed_experts=8, n_shared_experts=0, num_experts_per_tok=2, moe_intermediate_size=64, first_k_dense_replace=0,
                       n_group=1, topk_group=1, scoring_func="softmax", qk_norm=True, q_lora_rank=None, routed_scaling_factor=1.0)


def test_tp2_ep2_qwen3_moe_matches_single_rank():
    base = dict(model="qwen3-tiny", dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64)
    prompts = _prompts(3, 21, 2, 512)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = _run(Config(**base, model_config=_qwen_cfg()), prompts, sp)
    got = _run(Config(**base, model_config=_qwen_cfg(), attention_tp=2, ffn_ep=2), prompts, sp)
    assert got == want


@pytest.mark.parametrize("moe", [False, True])
def test_tp2_ffn_tp2_with_vocab_parallel_head_matches_single_rank(moe):
    """Attention-TP 2 with the FFN split by intermediate columns over the same two ranks (dense MLP: all-gather -> GEMM and
    GEMM -> reduce-scatter; experts: every rank holds half of every expert) and the embedding table / output projection split by
    vocabulary rows (509 rows: the last shard is padded)."""
    mc = _qwen_cfg()
    mc.vocab_size = 509
    if not moe:
        mc.n_routed_experts = 0
    base = dict(model="qwen3-tiny", dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64)
    prompts = _prompts(3, 21, 2, 509)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = _run(Config(**base, model_config=mc), prompts, sp)
    got = _run(Config(**base, model_config=mc, attention_tp=2, ffn_tp=2), prompts, sp)
    assert got == want


def test_dead_worker_is_reported():
    from nanoengine_b200.engine.executor import ExecutorError, MultiprocExecutor
    cfg = Config(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, num_kvcache_blocks=32, attention_dp=2, ffn_ep=2)
    ex = MultiprocExecutor(cfg, timeout_s=30)
    try:
        ex.procs[1].terminate()
        ex.procs[1].join(timeout=10)
        with pytest.raises(ExecutorError):
            ex.collective_rpc("get_step_timing")
    finally:
        ex.shutdown()


def test_pp2_prefill_pipeline_matches_single_stage():
    """Static prefill pipeline over 2 stages (prefill mode): same first tokens as the single-stage prefill engine."""
    from nanoengine_b200 import RequestMigrate
    from nanoengine_b200.models.pp import pp_layer_partition, split_batch
    assert pp_layer_partition(61, 8)[0] == (0, 8) and pp_layer_partition(61, 8)[-1] == (54, 61)
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64, mode="prefill")
    prompts = _prompts(5, 19, 7, 1024)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)

    def firsts(cfg):
        llm = LLM(cfg)
        try:
            blobs = llm.generate(prompts, sp, return_serialized=True)
            return sorted(RequestMigrate.from_bytes(b).metadata for b in blobs)
        finally:
            llm.shutdown()

    assert firsts(Config(**base, pp=2)) == firsts(Config(**base))


def _spmd_peer(rank, world, port, mode, q):
    """One SPMD rank on CPU (gloo).  Rank 1 leaves after two steps: politely (mode 'leave') or by dying ('die')."""
    import os
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        from nanoengine_b200.engine.executor import ExecutorError
        cfg = Config(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=4, num_kvcache_blocks=64,
                     attention_dp=world, ffn_ep=world, executor_backend="spmd", peer_timeout_s=8.0, seed=rank)
        llm = LLM(cfg)
        llm.add_request(_prompts(1, 12, 5 + rank, 1024)[0], SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True))
        steps = 0
        try:
            while steps < 40:
                llm.step()
                steps += 1
                if rank == 1 and steps == 2:
                    if mode == "die":
                        os._exit(0)                   # no goodbye: the peer has to notice by itself
                    llm.shutdown()                    # between steps, nothing in flight: announce and go
                    q.put((rank, "left", steps))
                    return
            q.put((rank, "finished", steps))
        except ExecutorError as e:
            q.put((rank, "peer-lost", steps, str(e)))
    except Exception as e:
        import traceback
        q.put((rank, "error", f"{e}\n{traceback.format_exc()}"))


@pytest.mark.parametrize("mode", ["leave", "die"])
def test_spmd_rank_loss_is_detected_on_the_host(mode):
    """Failure detection without touching a GPU: the surviving rank must stop with an error at its next per-step
    rendezvous (announced departure: at once; silent death: connection error or the rendezvous timeout), never hang."""
    import socket
    import time
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_spmd_peer, args=(r, 2, port, mode, q)) for r in range(2)]
    t0 = time.time()
    for p in ps:
        p.start()
    want = 2 if mode == "leave" else 1
    res = [q.get(timeout=120) for _ in range(want)]
    for p in ps:
        p.join(timeout=60)
    by_rank = {r[0]: r for r in res}
    assert by_rank[0][1] == "peer-lost", by_rank
    assert 2 <= by_rank[0][2] <= 4                       # it noticed within a step or two
    assert time.time() - t0 < 100
