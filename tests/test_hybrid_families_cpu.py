"""GLM5-next and Kimi-K3 families on CPU: the delta-attention recurrence with a gate per key channel, hyper-connections, block
attention residuals, gated activations, packed MXFP4 expert tensors, and the models end to end through the engine."""
import pytest
import torch

from nanoengine_b200 import LLM, Config, SamplingParams
from nanoengine_b200.models.config import ModelConfig, tiny_glm5_next, tiny_kimi_k3
from nanoengine_b200.ops import reference as ref


def test_kda_step_matches_the_written_out_recurrence():
    """One sequence, token by token, against the formula of a single decode step: S *= exp(g) per key channel,
    v' = beta (v - S k), S += v' k^T, o = S q."""
    torch.manual_seed(0)
    T, H, Dk, Dv = 7, 2, 8, 4
    q, k, v = torch.randn(T, H, Dk), torch.randn(T, H, Dk), torch.randn(T, H, Dv)
    raw_g, b = torch.randn(T, H, Dk), torch.randn(T, H)
    A_log, dtb = torch.randn(H) * 0.3, torch.randn(H * Dk) * 0.3
    gate, nw = torch.randn(T, H, Dv), torch.rand(Dv) + 0.5
    for lb in (-5.0, None):
        state = torch.zeros(2, H, Dv, Dk)
        out = ref.kda_recurrent(q, k, v, raw_g, b, A_log, dtb, lb, state, torch.tensor([1]), torch.tensor([0, T]), torch.tensor([1]), gate, nw, 1e-6)
        S = torch.zeros(H, Dv, Dk)
        rows = []
        for t in range(T):
            qn = q[t] / torch.sqrt((q[t] ** 2).sum(-1, keepdim=True) + 1e-6) * Dk ** -0.5
            kn = k[t] / torch.sqrt((k[t] ** 2).sum(-1, keepdim=True) + 1e-6)
            x = raw_g[t] + dtb.view(H, Dk)
            g = lb * torch.sigmoid(A_log.exp()[:, None] * x) if lb else -A_log.exp()[:, None] * torch.nn.functional.softplus(x)
            S = S * g.exp()[:, None, :]
            vp = torch.sigmoid(b[t])[:, None] * (v[t] - torch.einsum("hvk,hk->hv", S, kn))
            S = S + vp[:, :, None] * kn[:, None, :]
            o = torch.einsum("hvk,hk->hv", S, qn)
            rows.append(o * torch.rsqrt((o ** 2).mean(-1, keepdim=True) + 1e-6) * nw * torch.sigmoid(gate[t]))
        assert (out.view(T, H, Dv) - torch.stack(rows)).abs().max() < 1e-5
        assert (state[1] - S).abs().max() < 1e-5 and state[0].abs().max() == 0


def test_kda_state_continues_across_calls():
    torch.manual_seed(1)
    T, H, Dk, Dv = 12, 2, 8, 8
    a = [torch.randn(T, H, Dk), torch.randn(T, H, Dk), torch.randn(T, H, Dv), torch.randn(T, H, Dk), torch.randn(T, H)]
    A_log, dtb, gate, nw = torch.zeros(H), torch.zeros(H * Dk), torch.randn(T, H, Dv), torch.ones(Dv)

    def run(bounds):
        st = torch.zeros(1, H, Dv, Dk)
        outs = [ref.kda_recurrent(*[t[s:e] for t in a], A_log, dtb, -5.0, st, torch.tensor([0]), torch.tensor([0, e - s]),
                                  torch.tensor([1 if i == 0 else 0]), gate[s:e], nw, 1e-6) for i, (s, e) in enumerate(bounds)]
        return torch.cat(outs), st
    whole, s1 = run([(0, T)])
    parts, s2 = run([(0, 5), (5, 11), (11, 12)])
    assert (whole - parts).abs().max() < 1e-5 and (s1 - s2).abs().max() < 1e-5


def test_hyper_connection_mix_is_doubly_normalised_and_post_matches_einsum():
    torch.manual_seed(2)
    T, h, D = 5, 4, 32
    x = torch.randn(T, h, D)
    fn, base, scale = torch.randn((2 + h) * h, h * D) * 0.1, torch.randn((2 + h) * h) * 0.1, torch.tensor([1.0, 0.9, 1.1])
    y, post, comb = ref.mhc_pre(x, fn, base, scale, 8, 1e-6)
    assert y.shape == (T, D) and post.shape == (T, h) and comb.shape == (T, h, h)
    assert (comb.sum(-2) - 1).abs().max() < 1e-3 and (comb.sum(-1) - 1).abs().max() < 2e-2      # columns exact, rows after 8 rounds
    assert (post > 0).all() and (post < 2).all()
    sub = torch.randn(T, D)
    out = ref.mhc_post(sub, x, post, comb)
    want = post[:, :, None] * sub[:, None, :] + torch.einsum("tij,tjd->tid", comb.transpose(1, 2), x)
    assert (out - want).abs().max() < 1e-5


def test_attention_residual_mixture_matches_the_softmax_statement():
    torch.manual_seed(3)
    T, D, rows, valid = 3, 64, 6, 4
    prefix, bank = torch.randn(T, D), torch.randn(T, rows, D)
    ws, wo = torch.randn(D), torch.rand(D) + 0.5
    keep = bank.clone()
    out = ref.attn_res_mix(prefix, bank, valid, ws, wo, 1e-6, write_row=valid)
    cand = torch.cat([keep[:, :valid], prefix[:, None]], 1)
    sc = (cand * ws).sum(-1) * torch.rsqrt(cand.square().mean(-1) + 1e-6)
    mix = (sc.softmax(-1)[..., None] * cand).sum(1)
    want = mix * torch.rsqrt(mix.square().mean(-1, keepdim=True) + 1e-6) * wo
    assert (out - want).abs().max() < 1e-5
    assert torch.equal(bank[:, valid], prefix) and torch.equal(bank[:, :valid], keep[:, :valid])


def test_gated_activations():
    torch.manual_seed(4)
    x = torch.randn(6, 32) * 8
    a, b = x.chunk(2, -1)
    assert torch.allclose(ref.silu_and_mul(x), torch.nn.functional.silu(a) * b)
    assert torch.allclose(ref.silu_and_mul(x, act=("clamp", 3.0)), torch.nn.functional.silu(a.clamp(max=3.0)) * b.clamp(-3.0, 3.0))
    situ = 4.0 * torch.tanh(a / 4.0) * torch.sigmoid(a) * (25.0 * torch.tanh(b / 25.0))
    assert torch.allclose(ref.silu_and_mul(x, act=("situ", 4.0, 25.0)), situ)
    assert torch.allclose(ref.silu_and_mul(x, act=("situ", 4.0, None)), 4.0 * torch.tanh(a / 4.0) * torch.sigmoid(a) * b)


def test_mxfp4_round_trip():
    torch.manual_seed(5)
    w = torch.randn(8, 64) * 3
    p, s = ref.mxfp4_quant(w)
    assert p.shape == (8, 32) and s.shape == (8, 2) and p.dtype == torch.uint8
    back = ref.mxfp4_dequant(p, s)
    assert (back - w).abs().max() <= w.abs().amax() / 6.0 + 1e-6            # at most one e2m1 step of the block's scale
    p2, s2 = ref.mxfp4_quant(back)                                          # representable values survive unchanged
    assert torch.equal(ref.mxfp4_dequant(p2, s2), back)


def test_hf_configs_of_the_two_families():
    k3 = ModelConfig.from_dict({"architectures": ["KimiK3ForConditionalGeneration"], "hidden_size": 64, "num_hidden_layers": 4,
                                "num_attention_heads": 4, "num_experts": 8, "num_experts_per_token": 2, "num_shared_experts": 1,
                                "routed_expert_hidden_size": 32, "attn_res_block_size": 2, "moe_intermediate_size": 32, "vocab_size": 100,
                                "layer_types": ["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                                "linear_attn_config": {"num_heads": 2, "head_dim": 16, "short_conv_kernel_size": 4}})
    assert k3.is_mla and k3.is_hybrid_gdn and k3.linear_kind == "kda" and k3.n_routed_experts == 8 and k3.num_experts_per_tok == 2
    assert k3.glu_act == ("situ", 4.0, 25.0) and k3.mla_skip_rope and k3.mla_output_gate and k3.kda_gate_lower_bound == -5.0
    assert k3.scoring_func == "sigmoid" and k3.norm_topk_prob and k3.num_layers_of("full_attention") == 1
    glm = ModelConfig.from_dict({"architectures": ["Glm5NextForConditionalGeneration"], "hidden_size": 64, "num_hidden_layers": 2,
                                 "layer_types": ["linear_attention", "sparse_attention"], "mlp_layer_types": ["dense", "sparse"],
                                 "hc_mult": 4, "hc_sinkhorn_iters": 3, "linear_attn_config": {"num_heads": 2, "head_dim": 16, "short_conv_kernel_size": 4}})
    assert glm.glu_act == ("clamp", 10.0) and glm.layer_type(1) == "full_attention" and not glm.is_moe_layer(0) and glm.is_moe_layer(1)
    from nanoengine_b200.runtime.cache import make_cache_plan
    plan = make_cache_plan(k3, "bfloat16", 64, state_slots=4)
    assert plan.mla and plan.gdn and plan.num_layers == 1 and plan.gdn_layers == 3 and plan.gdn_dk == 16


def _llm(mc, **kw):
    base = dict(model="tiny", model_config=mc, dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=64,
                num_kvcache_blocks=32, max_num_seqs=8)
    base.update(kw)
    if mc is None:
        base.pop("model_config"); base.pop("dummy_weight")
    return LLM(Config(**base))


@pytest.mark.parametrize("make", [tiny_glm5_next, tiny_kimi_k3])
def test_family_prefill_chunks_and_decode_agree(make):
    mc = make()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    ref_out = [o["token_ids"] for o in _llm(mc).generate(prompts, sp)]
    assert all(len(o) == 6 for o in ref_out)
    chunked = [o["token_ids"] for o in _llm(mc, max_num_batched_tokens=32, enable_chunked_prefill=True).generate(prompts, sp)]
    assert chunked == ref_out
    forced = _llm(mc).generate([p + o[:5] for p, o in zip(prompts, ref_out)], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    assert [o["token_ids"][0] for o in forced] == [o[5] for o in ref_out]


def test_kimi_k3_without_residual_blocks_is_a_plain_residual_stream():
    mc = tiny_kimi_k3(attn_res_block_size=0, routed_expert_hidden_size=0)
    out = _llm(mc).generate([list(range(3, 30))], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert len(out[0]["token_ids"]) == 4


@pytest.mark.parametrize("make", [tiny_glm5_next, tiny_kimi_k3])
def test_family_checkpoint_round_trip(tmp_path, make):
    from nanoengine_b200.models.weights import random_hf_weights, save_hf_checkpoint
    mc = make()
    save_hf_checkpoint(str(tmp_path), mc, random_hf_weights(mc, seed=3))
    from_disk = _llm(None, model=str(tmp_path))
    direct = _llm(mc)
    # the checkpoint stores bf16: feed the directly loaded model the same rounded values
    direct.engine.executor.runner.load_weights((n, t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=3))
    prompts = [list(range(5, 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    assert from_disk.generate(prompts, sp)[0]["token_ids"] == direct.generate(prompts, sp)[0]["token_ids"]


def test_kimi_k3_reads_packed_mxfp4_experts():
    """Expert tensors that arrive as packed e2m1 nibbles + e8m0 scales load as their dequantised values."""
    from nanoengine_b200.models.weights import random_hf_weights
    mc = tiny_kimi_k3()
    plain, packed = [], []
    for name, t in random_hf_weights(mc, seed=7):
        if ".mlp.experts." in name:
            p, s = ref.mxfp4_quant(t)
            packed += [(name.replace(".weight", ".weight_packed"), p), (name.replace(".weight", ".weight_scale"), s)]
            plain.append((name, ref.mxfp4_dequant(p, s)))
        else:
            plain.append((name, t)); packed.append((name, t))
    a, b = _llm(mc), _llm(mc)
    a.engine.executor.runner.load_weights(iter(plain))
    b.engine.executor.runner.load_weights(iter(packed))
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    assert a.generate([list(range(9, 40))], sp)[0]["token_ids"] == b.generate([list(range(9, 40))], sp)[0]["token_ids"]


# ---- Gemma4 -----------------------------------------------------------------------------------------------------------------
def test_sliding_window_attention_oracle():
    """A window of w keeps exactly the last w key positions: equal to dense attention over a cache truncated to them."""
    torch.manual_seed(7)
    Hq, Hkv, D, bs, n, w = 4, 2, 16, 8, 29, 5
    kc, vc = torch.randn(8, bs, Hkv, D), torch.randn(8, bs, Hkv, D)
    bt = torch.arange(8, dtype=torch.int32).view(1, 8)
    q = torch.randn(1, Hq, D)
    got = ref.gqa_attention_paged(q, kc, vc, bt, torch.tensor([0, 1]), torch.tensor([n]), 1.0, window=w)
    k = kc.view(-1, Hkv, D)[n - w: n].repeat_interleave(2, 1)
    v = vc.view(-1, Hkv, D)[n - w: n].repeat_interleave(2, 1)
    want = torch.einsum("hn,nhd->hd", torch.softmax(torch.einsum("hd,nhd->hn", q[0], k), -1), v)
    assert (got[0] - want).abs().max() < 1e-5


def test_gemma4_config_and_cache_layers():
    from nanoengine_b200.models.config import tiny_gemma4
    from nanoengine_b200.runtime.cache import KVCache, make_cache_plan
    mc = tiny_gemma4()
    assert [mc.kv_source_layer(i) for i in range(6)] == [0, 1, 2, 3, 3, 2]         # layer 4 (sliding) reads layer 3, layer 5 (global) layer 2
    assert mc.attn_head_dim(0) == 32 and mc.attn_head_dim(2) == 64 and mc.glu_act == ("gelu_tanh",)
    plan = make_cache_plan(mc, "float32", 16)
    assert plan.num_layers == 4 and plan.layer_dims == [32, 32, 64, 32] and plan.row_dim == 64
    cache = KVCache(plan, 4, "cpu")
    assert cache.layers[0][0].shape == (5, 16, 2, 32) and cache.layers[2][1].shape == (5, 16, 2, 64) and cache.layers[0][0].is_contiguous()
    d = ModelConfig.from_dict({"architectures": ["Gemma4ForConditionalGeneration"],
                               "text_config": {"hidden_size": 64, "num_hidden_layers": 2, "layer_types": ["sliding_attention", "full_attention"],
                                               "sliding_window": 8, "head_dim": 16, "global_head_dim": 32, "num_attention_heads": 4,
                                               "num_key_value_heads": 2, "vocab_size": 100, "intermediate_size": 64,
                                               "rope_parameters": {"sliding_attention": {"rope_theta": 1e4}, "full_attention": {"rope_theta": 1e6}}}})
    assert d.attn_layer_type(0) == "sliding_attention" and d.rope_parameters_by_type["full_attention"]["rope_theta"] == 1e6 and d.tie_word_embeddings


def test_gemma4_prefill_chunks_and_decode_agree():
    from nanoengine_b200.models.config import tiny_gemma4
    mc = tiny_gemma4()
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    kw = dict(kvcache_block_size=16, num_kvcache_blocks=64)
    ref_out = [o["token_ids"] for o in _llm(mc, **kw).generate(prompts, sp)]
    chunked = [o["token_ids"] for o in _llm(mc, max_num_batched_tokens=32, enable_chunked_prefill=True, **kw).generate(prompts, sp)]
    assert chunked == ref_out
    forced = _llm(mc, **kw).generate([p + o[:5] for p, o in zip(prompts, ref_out)], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    assert [o["token_ids"][0] for o in forced] == [o[5] for o in ref_out]
    # the window matters: the same weights with a window that covers everything give other tokens for the long prompt
    wide = [o["token_ids"] for o in _llm(tiny_gemma4(sliding_window=4096), **kw).generate(prompts, sp)]
    assert wide[1] == ref_out[1] and wide[0] != ref_out[0]


def test_gemma4_checkpoint_round_trip(tmp_path):
    from nanoengine_b200.models.config import tiny_gemma4
    from nanoengine_b200.models.weights import random_hf_weights, save_hf_checkpoint
    mc = tiny_gemma4()
    save_hf_checkpoint(str(tmp_path), mc, random_hf_weights(mc, seed=3))
    kw = dict(kvcache_block_size=16, num_kvcache_blocks=64)
    from_disk = _llm(None, model=str(tmp_path), **kw)
    direct = _llm(mc, **kw)
    direct.engine.executor.runner.load_weights((n, t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=3))
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    assert from_disk.generate([list(range(5, 40))], sp)[0]["token_ids"] == direct.generate([list(range(5, 40))], sp)[0]["token_ids"]
