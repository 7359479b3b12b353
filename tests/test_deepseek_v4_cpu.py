"""DeepSeek-V4 on CPU: the KV compressor (whole prompt, chunks, one token at a time, batched decode), the window + pooled-row
attention with a sink, sqrt-softplus and hash routing, the config spellings, the cache plan, and the model through the engine."""
import pytest
import torch

from nanoengine_b200 import LLM, Config, SamplingParams
from nanoengine_b200.models.config import ModelConfig, tiny_deepseek_v4
from nanoengine_b200.ops import reference as ref


def _whole_prompt_pooling(kv, score, ape, ratio, d):
    """The whole-prompt statement: blocks of `ratio` rows; with overlap (two halves per row) a block pools the second halves
    of its rows together with the first halves of the previous block's rows (nothing before the first block)."""
    n = kv.shape[0] - kv.shape[0] % ratio
    k = kv[:n].view(-1, ratio, kv.shape[1])
    s = score[:n].view(-1, ratio, kv.shape[1]) + ape
    if kv.shape[1] == 2 * d:
        nb = k.shape[0]
        k2, s2 = torch.zeros(nb, 2 * ratio, d), torch.full((nb, 2 * ratio, d), float("-inf"))
        k2[:, ratio:], s2[:, ratio:] = k[:, :, d:], s[:, :, d:]
        k2[1:, :ratio], s2[1:, :ratio] = k[:-1, :, :d], s[:-1, :, :d]
        k, s = k2, s2
    return (k * s.softmax(1)).sum(1)


@pytest.mark.parametrize("ratio", [4, 8])
def test_compressor_chunks_and_single_tokens_equal_the_whole_prompt(ratio):
    torch.manual_seed(0)
    d, n = 16, 45
    c = 2 if ratio == 4 else 1
    kv, sc, ape = torch.randn(n, c * d), torch.randn(n, c * d), torch.randn(ratio, c * d)
    want = _whole_prompt_pooling(kv, sc, ape, ratio, d)
    pos = torch.arange(n)
    for bounds in ([0, n], [0, 3, 4, 11, 30, 31, n], list(range(n + 1))):
        ks, ss = torch.zeros(c * ratio, c * d), torch.full((c * ratio, c * d), float("-inf"))
        got = [ref.dsv4_compress_extend(kv[a:b], sc[a:b] + ape[pos[a:b] % ratio], ks, ss, a, ratio, d) for a, b in zip(bounds, bounds[1:])]
        got = torch.cat(got)
        assert got.shape == want.shape and (got - want).abs().max() < 1e-5


@pytest.mark.parametrize("ratio", [4, 8])
def test_batched_decode_compressor_equals_the_sequential_one(ratio):
    torch.manual_seed(1)
    d, B, steps = 8, 3, 20
    c = 2 if ratio == 4 else 1
    ape = torch.randn(ratio, c * d)
    start = [5, 0, 11]                    # every sequence is somewhere else in its block
    pool_k, pool_s = torch.zeros(B + 1, c * ratio, c * d), torch.full((B + 1, c * ratio, c * d), float("-inf"))
    seq_k = [torch.zeros(c * ratio, c * d) for _ in range(B)]
    seq_s = [torch.full((c * ratio, c * d), float("-inf")) for _ in range(B)]
    for b in range(B):                    # bring both forms to the start position with the same prefix
        pk, ps = torch.randn(start[b], c * d), torch.randn(start[b], c * d)
        if start[b]:
            for ks, ss in ((pool_k[b], pool_s[b]), (seq_k[b], seq_s[b])):
                ref.dsv4_compress_extend(pk, ps + ape[torch.arange(start[b]) % ratio], ks, ss, 0, ratio, d)
    slots = torch.arange(B)
    for t in range(steps):
        pos = torch.tensor(start) + t
        kv, sc = torch.randn(B, c * d), torch.randn(B, c * d)
        pooled, done = ref.dsv4_compress_decode(kv, sc + ape[pos % ratio], pool_k, pool_s, slots, pos, ratio, d)
        for b in range(B):
            one = ref.dsv4_compress_extend(kv[b: b + 1], sc[b: b + 1] + ape[pos[b: b + 1] % ratio], seq_k[b], seq_s[b], int(pos[b]), ratio, d)
            assert bool(done[b]) == (one.shape[0] == 1)
            if one.shape[0]:
                assert (pooled[b] - one[0]).abs().max() < 1e-5
            else:
                assert pooled[b].abs().max() == 0
            assert torch.equal(pool_s[b].isinf(), seq_s[b].isinf()) and (pool_k[b] - seq_k[b]).abs().max() < 1e-6
    assert pool_k[B].abs().max() == 0                       # the spare slot was never touched


def test_sink_attention_matches_a_softmax_with_one_extra_logit():
    torch.manual_seed(2)
    T, H, D, L = 5, 3, 8, 11
    q, kv, sink = torch.randn(T, H, D), torch.randn(T, L, D), torch.randn(H)
    mask = torch.rand(T, L) > 0.3
    mask[2] = False                                          # a row that sees nothing
    got = ref.sink_attention(q, kv, mask, sink, 0.5)
    s = torch.einsum("thd,tld->thl", q, kv) * 0.5
    s = s.masked_fill(~mask.unsqueeze(1), float("-inf"))
    p = torch.cat([s, sink.view(1, H, 1).expand(T, H, 1)], -1).softmax(-1)[..., :L]
    want = torch.einsum("thl,tld->thd", p, kv)
    assert (got - want).abs().max() < 1e-5 and got[2].abs().max() == 0
    shared = ref.sink_attention(q, kv[0], mask, sink, 0.5)
    assert (shared[0] - got[0]).abs().max() < 1e-5


def test_fp8_round_trip_uses_power_of_two_scales_per_64():
    torch.manual_seed(3)
    x = torch.randn(4, 128) * torch.tensor([0.01, 1.0, 50.0, 3000.0]).view(4, 1)
    y = ref.fp8_qdq_pow2(x.clone(), 64)
    assert ((y - x).abs() <= x.abs().view(4, 2, 64).amax(-1, keepdim=True).expand(4, 2, 64).reshape(4, 128) * 2 ** -3).all()
    v = x.view(4, 2, 64)
    s = torch.exp2(torch.ceil(torch.log2(v.abs().amax(-1, keepdim=True).clamp(min=1e-4) / 448.0)))
    assert torch.equal(y.view(4, 2, 64), (v / s).to(torch.float8_e4m3fn).float() * s)


def test_packed_cache_rows_keep_quantised_rows_exactly():
    torch.manual_seed(5)
    d, rd = 192, 64
    kv = (torch.randn(9, d) * torch.logspace(-3, 2, 9).view(9, 1)).to(torch.bfloat16)
    kv[:, :-rd] = ref.fp8_qdq_pow2(kv[:, :-rd], 64)
    rows = ref.dsv4_pack_rows(kv, rd)
    assert rows.dtype == torch.uint8 and rows.shape == (9, 128 + 128 + 8) and (rows[:, -6:] == 0).all()
    assert torch.equal(ref.dsv4_unpack_rows(rows, d, rd, torch.bfloat16), kv)
    assert torch.equal(ref.dsv4_unpack_rows(rows.view(3, 3, -1), d, rd, torch.bfloat16), kv.view(3, 3, d))


def test_model_with_packed_fp8_cache_equals_the_plain_cache():
    """In bf16 the packed rows hold exactly what the plain cache holds, so the tokens are the same."""
    mc = tiny_deepseek_v4(head_dim=80)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (41, 12)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    plain = _llm(mc, dtype="bfloat16")
    packed = _llm(mc, dtype="bfloat16", kv_cache_dtype="fp8")
    assert packed.engine.executor.runner.cache.kv.dtype == torch.uint8 and packed.engine.executor.runner.cache.kv.shape[-1] == 64 + 32 + 8
    assert [o["token_ids"] for o in packed.generate(prompts, sp)] == [o["token_ids"] for o in plain.generate(prompts, sp)]


def test_sqrt_softplus_routing():
    torch.manual_seed(4)
    logits, bias = torch.randn(6, 16) * 3, torch.randn(16) * 0.1
    idx, w = ref.moe_route(logits, bias, 4, 1, 1, True, 1.5, "sqrtsoftplus")
    s = torch.nn.functional.softplus(logits).sqrt()
    want = (s + bias).topk(4, -1).indices
    assert torch.equal(idx.long().sort(-1).values, want.sort(-1).values)
    ww = s.gather(1, idx.long())
    assert (w - 1.5 * ww / ww.sum(-1, keepdim=True)).abs().max() < 1e-6


def test_config_reads_the_release_spellings_and_the_cache_plan_counts_pooled_rows():
    mc = ModelConfig.from_dict({"architectures": ["DeepseekV4ForCausalLM"], "dim": 256, "n_layers": 3, "n_heads": 4, "head_dim": 128,
                                "rope_head_dim": 64, "q_lora_rank": 64, "moe_inter_dim": 128, "n_routed_experts": 8, "n_activated_experts": 2,
                                "norm_eps": 1e-5, "n_hash_layers": 1, "compress_ratios": [0, 4, 128], "vocab_size": 1000, "swiglu_limit": 10.0,
                                "route_scale": 1.5, "max_seq_len": 8192})
    assert mc.is_dsv4 and not mc.is_mla and mc.hidden_size == 256 and mc.num_hidden_layers == 3 and mc.qk_rope_head_dim == 64
    assert mc.scoring_func == "sqrtsoftplus" and mc.hc_mult == 4 and mc.hc_sinkhorn_iters == 20 and mc.window_size == 128 and mc.o_groups == 8
    assert mc.glu_act == ("clamp", 10.0) and mc.num_hash_layers == 1 and mc.routed_scaling_factor == 1.5 and mc.max_position_embeddings == 8192
    assert [mc.compress_ratio(i) for i in range(4)] == [0, 4, 128, 0] and mc.is_moe_layer(0)
    from nanoengine_b200.runtime.cache import KVCache, make_cache_plan
    plan = make_cache_plan(mc, "bfloat16", 64, state_slots=4)
    assert plan.dsv4 and plan.mla and plan.needs_state_slots and plan.kv_dtype == torch.bfloat16 and plan.row_dim == 128
    # 3 layers x 64 raw rows + 16 rows pooled over 4 + 1 row pooled over 128, two bytes each
    assert plan.block_bytes == (3 * 64 + 16 + 1) * 128 * 2
    packed = make_cache_plan(mc, "fp8", 64, state_slots=4)          # 64 e4m3 + 64 bf16 + 8 scale bytes per row
    assert packed.kv_dtype == torch.uint8 and packed.row_dim == 200 and packed.block_bytes == (3 * 64 + 16 + 1) * 200
    assert packed.state_slot_bytes == plan.state_slot_bytes and ref.dsv4_row_bytes(512, 64) == 584
    assert plan.state_slot_bytes == 2 * 4 * (4 * 4 * 128 + 128 * 128)
    from nanoengine_b200._native import _core as C
    assert plan.plan_bits() == C.PLAN_HCA | C.PLAN_CSA
    kv = KVCache(plan, 5, "cpu")
    assert kv.comp[0] is None and kv.comp[1].shape == (6, 16, 128) and kv.comp[2].shape == (6, 1, 128)
    assert kv.comp_kv_state[1].shape == (5, 8, 256) and kv.comp_score_state[2].shape == (5, 128, 128) and kv.comp_score_state[2].isinf().all()
    names = [f["name"] for f in kv.page_families()]
    assert names == ["mla_kv", "dsv4_pooled_1", "dsv4_pooled_2"] and len(kv.slot_families()) == 4
    assert sum(v.numel() * v.element_size() for v in kv.block_views(2)) == plan.block_bytes
    with pytest.raises(ValueError):
        Config(model="x", model_config=mc, dummy_weight=True, device="cpu", num_speculative_tokens=1)


def _llm(mc, **kw):
    base = dict(model="tiny", model_config=mc, dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=16,
                num_kvcache_blocks=48, max_num_seqs=8)
    base.update(kw)
    if mc is None:
        base.pop("model_config"); base.pop("dummy_weight")
    return LLM(Config(**base))


def test_model_prefill_chunks_decode_and_forced_prefill_agree():
    """Greedy tokens are the same whether the prompt arrives whole or in chunks that cut compression blocks, and each generated
    token equals the one a fresh prefill of prompt + earlier tokens gives (so the decode path - batched compressor, window /
    pooled-row gather - states the same function as the prefill path)."""
    mc = tiny_deepseek_v4(head_dim=80)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    whole = [o["token_ids"] for o in _llm(mc).generate(prompts, sp)]
    assert all(len(o) == 10 for o in whole)
    chunked = [o["token_ids"] for o in _llm(mc, max_num_batched_tokens=21, enable_chunked_prefill=True).generate(prompts, sp)]
    assert chunked == whole
    one = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    for k in (3, 9):
        forced = _llm(mc).generate([p + o[:k] for p, o in zip(prompts, whole)], one)
        assert [o["token_ids"][0] for o in forced] == [o[k] for o in whole]


def test_window_and_pooled_rows_are_what_the_layer_attends():
    """One compressing layer against a written-out statement over the whole sequence: token t sees raw rows t-W+1..t and
    pooled rows of blocks that ended at or before t."""
    from nanoengine_b200.models.deepseek_v4 import DeepseekV4ForCausalLM
    from nanoengine_b200.models.weights import random_hf_weights
    from nanoengine_b200.runtime.cache import KVCache, make_cache_plan
    from nanoengine_b200.runtime.context import ForwardContext
    mc = tiny_deepseek_v4(head_dim=80, num_hidden_layers=2, compress_ratios=[0, 4], num_hash_layers=0)
    torch.manual_seed(0)
    model = DeepseekV4ForCausalLM(mc, dtype=torch.float32)
    model.load_weights(random_hf_weights(mc, seed=1))
    A = model.model.layers["1"].self_attn
    n, bs = 37, 16
    kvc = KVCache(make_cache_plan(mc, "float32", bs, state_slots=2), 8, "cpu")
    x = torch.randn(n, mc.hidden_size)
    pos = torch.arange(n)
    ctx = ForwardContext(is_prefill=True, num_seqs=1, num_tokens=n, cu_seqlens_q=torch.tensor([0, n], dtype=torch.int32),
                         context_lens=torch.tensor([n], dtype=torch.int32), slot_mapping=torch.arange(n) + 2 * bs,
                         block_tables=torch.tensor([[2, 3, 4, 5]], dtype=torch.int32), max_seqlen_q=n, max_seqlen_k=n, kv_caches=kvc.layers,
                         cu_seqlens_q_host=[0, n], context_lens_host=[n], state_slots=torch.tensor([1], dtype=torch.int32),
                         comp_caches=kvc.comp, comp_kv_states=kvc.comp_kv_state, comp_score_states=kvc.comp_score_state)
    ctx.extras.update(state_slots_host=[1], fresh_host=[1])
    got = A(x, pos, ctx, model.rope_compress)
    # the statement
    from nanoengine_b200.models.deepseek_v4 import rotate_tail
    H, D, rd, W, r = mc.num_attention_heads, mc.head_dim, mc.qk_rope_head_dim, mc.window_size, 4
    kv = rotate_tail(A.kv_norm(A.wkv(x)).contiguous(), pos, model.rope_compress, rd)
    kv[:, :-rd] = ref.fp8_qdq_pow2(kv[:, :-rd], 64)
    q = A.wq_b(A.q_norm(A.wq_a(x))).view(n, H, D)
    q = rotate_tail(q * torch.rsqrt(q.square().mean(-1, keepdim=True) + mc.rms_norm_eps), pos, model.rope_compress, rd)
    C = A.compressor
    proj = x @ C.wkv_gate.t()
    pooled = _whole_prompt_pooling(proj[:, : 2 * D], proj[:, 2 * D:], C.ape, r, D)
    rows = rotate_tail(C.norm(pooled), torch.arange(pooled.shape[0]) * r, model.rope_compress, rd)
    rows[:, :-rd] = ref.fp8_qdq_pow2(rows[:, :-rd], 64)
    assert (kvc.comp[1][torch.tensor([2, 2, 2, 2, 3, 3, 3, 3, 4]), torch.tensor([0, 1, 2, 3, 0, 1, 2, 3, 0])] - rows).abs().max() < 1e-5
    outs = []
    for t in range(n):
        cand = torch.cat([kv[max(0, t - W + 1): t + 1], rows[: (t + 1) // r]])
        s = torch.einsum("hd,ld->hl", q[t], cand) * D ** -0.5
        p = torch.cat([s, A.attn_sink.view(H, 1)], -1).softmax(-1)[:, :-1]
        outs.append(p @ cand)
    o = rotate_tail(torch.stack(outs), pos, model.rope_compress, rd, inverse=True)
    want = A.wo_b(torch.einsum("tgd,grd->tgr", o.reshape(n, A.G, -1), A.wo_a).reshape(n, -1))
    assert (got - want).abs().max() < 1e-4
    # rotating back undoes the rotation
    z = torch.randn(5, 3, D)
    assert (rotate_tail(rotate_tail(z.clone(), pos[:5], model.rope_window, rd), pos[:5], model.rope_window, rd, inverse=True) - z).abs().max() < 1e-5


def test_checkpoint_names_fp8_scales_and_packed_experts():
    """A checkpoint under the release's names with fp8 attention weights (`.scale`) and packed 4-bit experts loads to the same
    model as its expanded values."""
    from nanoengine_b200.models.weights import random_hf_weights
    mc = tiny_deepseek_v4(head_dim=80, hidden_size=128, q_lora_rank=128, o_lora_rank=64)
    plain, packed = [], []
    for name, t in random_hf_weights(mc, seed=7):
        if ".ffn.experts." in name:
            p, s = ref.mxfp4_quant(t)
            packed += [(name, p.view(torch.int8)), (name.replace(".weight", ".scale"), s)]
            plain.append((name, ref.mxfp4_dequant(p, s)))
        elif name.endswith(("wq_a.weight", "wo_b.weight", "wo_a.weight")):
            q, s = ref.quant_fp8_block(t, ue8m0=True)
            packed += [(name.replace(".weight", ".scale"), s.to(torch.float8_e8m0fnu)), (name, q)]      # the scale may come first
            plain.append((name, ref.dequant_fp8_block(q, s)))
        else:
            plain.append((name, t)); packed.append((name, t))
    a, b = _llm(mc), _llm(mc)
    na = a.engine.executor.runner.load_weights(iter(plain))
    nb = b.engine.executor.runner.load_weights(iter(packed))
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    assert a.generate([list(range(9, 40))], sp)[0]["token_ids"] == b.generate([list(range(9, 40))], sp)[0]["token_ids"]
    with pytest.raises(ValueError):
        _llm(mc).engine.executor.runner.load_weights(iter([(n, t) for n, t in packed if not n.endswith("wq_a.scale")]))


def test_checkpoint_round_trip_and_preemption(tmp_path):
    from nanoengine_b200.models.weights import random_hf_weights, save_hf_checkpoint
    mc = tiny_deepseek_v4(head_dim=80)
    save_hf_checkpoint(str(tmp_path), mc, random_hf_weights(mc, seed=3))
    from_disk = _llm(None, model=str(tmp_path))
    direct = _llm(mc)
    direct.engine.executor.runner.load_weights((n, t if t.dtype == torch.int32 else t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=3))
    prompts = [list(range(5, 40)), list(range(100, 160)), list(range(7, 29))]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    want = [o["token_ids"] for o in direct.generate(prompts, sp)]
    assert [o["token_ids"] for o in from_disk.generate(prompts, sp)] == want
    # a pool so small that sequences are preempted and prefilled again: same tokens
    tight = _llm(mc, num_kvcache_blocks=9)
    tight.engine.executor.runner.load_weights((n, t if t.dtype == torch.int32 else t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=3))
    assert [o["token_ids"] for o in tight.generate(prompts, sp)] == want
    # the same pool with a host tier: preempted sequences swap their raw and pooled-row pages out and keep their state slot
    swapping = _llm(mc, num_kvcache_blocks=9, num_host_kvcache_blocks=16)
    swapping.engine.executor.runner.load_weights((n, t if t.dtype == torch.int32 else t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=3))
    assert set(swapping.engine.executor.runner.cache.host_families) == {"mla_kv", "dsv4_pooled_1", "dsv4_pooled_2"}
    assert [o["token_ids"] for o in swapping.generate(prompts, sp)] == want
