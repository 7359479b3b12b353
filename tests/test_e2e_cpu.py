"""The CPU plumbing run: a tiny DeepSeek-V3-style model through the offline LLM API with continuous batching,
checked against a dense PyTorch reference (logits within 1e-4, identical greedy tokens)."""
import torch

from nanoengine_b200 import Config, LLM, RequestIn, SamplingParams
from nanoengine_b200.models.weights import random_hf_weights

from dense_reference import dense_forward


def _prompts(n=4, length=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length,), generator=g).tolist() for _ in range(n)]


def _make(**kw):
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8,
                num_kvcache_blocks=64, seed=0)
    base.update(kw)
    return LLM(Config(**base))


def test_tiny_deepseek_matches_dense_reference():
    llm = _make()
    cfg = llm.config.model_config
    W = dict(random_hf_weights(cfg, seed=0))
    prompts = _prompts()
    captured = {}
    runner = llm.engine.executor.runner
    orig = runner.model.compute_logits

    def spy(h):
        out = orig(h)
        captured.setdefault("logits", []).append(out.clone())
        return out

    runner.model.compute_logits = spy
    for i, p in enumerate(prompts):
        llm.add_request_payload(RequestIn(i + 1, p, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)).to_bytes())
    outs = {o["seq_id"]: o["token_ids"] for o in llm.generate()}
    assert sorted(outs) == [1, 2, 3, 4] and all(len(v) == 16 for v in outs.values())
    # reference: greedy decode each prompt on its own with the dense model
    for i, p in enumerate(prompts):
        toks = list(p)
        for step in range(16):
            logits = dense_forward(cfg, W, toks)[-1]
            eng = captured["logits"][step][i]      # prefill step holds all four sequences, then one decode step each
            assert torch.allclose(logits, eng, atol=1e-4, rtol=1e-4), (i, step, (logits - eng).abs().max())
            toks.append(int(logits.argmax()))
        assert toks[len(p):] == outs[i + 1]


def test_chunked_prefill_prefix_cache_and_preemption_keep_tokens_identical():
    prompts = _prompts(4, 40, seed=3)
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    base = _make()
    want = {o["seq_id"]: o["token_ids"] for o in base.generate(prompts, sp)}
    # chunked prefill with a small token budget
    a = _make(max_num_batched_tokens=24)
    assert {o["seq_id"]: o["token_ids"] for o in a.generate(prompts, sp)} == want
    # a pool so small that decode growth must preempt and recompute
    b = _make(num_kvcache_blocks=10, enable_prefix_caching=False)
    assert {o["seq_id"]: o["token_ids"] for o in b.generate(prompts, sp)} == want
    # same prompts again on the first engine: prefix-cache hits, same tokens
    again = {o["seq_id"] - 4: o["token_ids"] for o in base.generate(prompts, sp)}
    assert again == want
    assert "dlengine_prefix_cache_hit_rate" in base.metrics()


def test_group_limited_routing_and_no_q_lora_variant():
    llm = _make(hf_overrides=dict(n_group=4, topk_group=2, q_lora_rank=None, routed_scaling_factor=2.5))
    cfg = llm.config.model_config
    W = dict(random_hf_weights(cfg, seed=0))
    p = _prompts(1, 20, seed=5)[0]
    out = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))[0]["token_ids"]
    toks = list(p)
    for _ in range(4):
        toks.append(int(dense_forward(cfg, W, toks)[-1].argmax()))
    assert toks[len(p):] == out


def test_sampling_temperature_is_seeded_and_logprobs_are_returned():
    p = _prompts(1, 16, seed=7)[0]
    sp = SamplingParams(temperature=0.8, max_tokens=6, ignore_eos=True, return_completion_logprobs=True)
    a = _make().generate([p], sp)[0]
    b = _make().generate([p], sp)[0]
    assert a["token_ids"] == b["token_ids"] and len(a["logprobs"]) == 6 and all(x <= 0 for x in a["logprobs"])


def test_weights_pulled_from_a_peer_engine_replace_the_local_ones():
    """Live weight update from a serving replica: after the pull the engine generates what the peer generates, its prefix
    cache is empty, and a shape mismatch is refused before anything is copied."""
    import torch
    from nanoengine_b200 import Config, LLM, SamplingParams
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=4, num_kvcache_blocks=32)
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (18, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a, b = LLM(Config(**base, seed=0)), LLM(Config(**base, seed=7))
    want = [o["token_ids"] for o in a.generate(prompts, sp)]
    before = [o["token_ids"] for o in b.generate(prompts, sp)]
    assert before != want
    n = b.pull_weights(a.export_weights(direct=True))
    assert n > 20 and b.engine.scheduler.num_cached_blocks(0) == 0
    assert [o["token_ids"] for o in b.generate(prompts, sp)] == want
    bad = a.export_weights(direct=True)
    bad[0] = {k: (v[:1] if k.endswith("lm_head.weight") else v) for k, v in bad[0].items()}
    import pytest
    with pytest.raises(ValueError):
        b.pull_weights(bad)
