"""Attention and sampling kernels against the plain PyTorch statements."""
import pytest
import torch

from nanoengine_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def k():
    from nanoengine_b200.ops import sm100, sm100_attn
    sm100.lib()
    sm100.clear_kernel_status()
    yield sm100_attn
    assert sm100.kernel_status()[0] == 0, f"a kernel reported a timed-out wait: {sm100.kernel_status()}"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _paged_case(q_lens, ctx_lens, H, Dk, R, bs, fp8, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    B = len(q_lens)
    nb_per = [(c + bs - 1) // bs for c in ctx_lens]
    total = sum(nb_per) + 3
    perm = torch.randperm(total, device="cuda", generator=g).to(torch.int32)
    bt = torch.zeros(B, max(nb_per) + 2, dtype=torch.int32, device="cuda")
    o = 0
    for i, n in enumerate(nb_per):
        bt[i, :n] = perm[o:o + n]; o += n
    cache = torch.randn(total, bs, Dk, device="cuda", generator=g) * 0.5
    cache = cache.clamp(-448, 448).to(FP8) if fp8 else cache.to(torch.bfloat16)
    T = sum(q_lens)
    q = (torch.randn(T, H, Dk, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device="cuda")
    return q, cache, bt, cu, cl


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("H,Dk,R,bs", [(8, 80, 64, 16), (16, 576, 512, 64)])
def test_generic_mla_attention(k, H, Dk, R, bs, fp8):
    q, cache, bt, cu, cl = _paged_case([1, 5, 1, 17], [33, 70, 1, 17], H, Dk, R, bs, fp8)
    # force the generic kernel even for the tensor-core geometry by passing a dense "sparse" list? no: use bf16 / small dims
    if fp8 and Dk == 576:
        pytest.skip("covered by the tcgen05 test")
    got = k.mla_attention_paged(q, cache, bt, cu, cl, 0.11, R)
    want = ref.mla_attention_paged(q, cache, bt, cu, cl, 0.11, R)
    assert _rel(got, want) < 1e-2


def test_generic_sparse_indices(k):
    q, cache, bt, cu, cl = _paged_case([1, 1, 1], [200, 130, 64], 16, 576, 512, 64, True, seed=2)
    topk = 48
    sp = torch.full((3, topk), -1, dtype=torch.int32, device="cuda")
    for i, n in enumerate([200, 130, 64]):
        pick = torch.randperm(n, device="cuda")[: min(topk, n) - (i == 1) * 5]
        sp[i, : pick.numel()] = ref.logical_to_physical(pick.to(torch.int32).unsqueeze(0), bt[i:i + 1], 64)[0]
    got = k.mla_attention_paged(q, cache, bt, cu, cl, 0.07, 512, sparse_indices=sp)
    want = ref.mla_attention_paged(q, cache, bt, cu, cl, 0.07, 512, sparse_indices=sp)
    assert _rel(got, want) < 6e-2            # the fp8 geometry runs the tensor-core kernel, which rounds P to e4m3
    # the same lists through the CUDA-core kernel (bf16 cache): exact softmax weights
    got16 = k.mla_attention_paged(q, cache.float().to(torch.bfloat16), bt, cu, cl, 0.07, 512, sparse_indices=sp)
    assert _rel(got16, want) < 1.5e-2


@pytest.mark.parametrize("H", [128, 16])
@pytest.mark.parametrize("topk,splits", [(64, 1), (200, 1), (2048, 1), (2048, 4), (320, 3)])
def test_sparse_mla_fp8_tcgen05(k, H, topk, splits):
    """DSA decode / verify rows on the tensor cores: every token attends its own list of cache rows; ids are scattered over
    the pool, some are -1 (in the middle of a list as well as at its end), lists need not be a multiple of the 64-row tile."""
    ctxs = [3000, 700, 65, 2500]
    q_lens = [1, 2, 1, 3]
    q, cache, bt, cu, cl = _paged_case(q_lens, ctxs, H, 576, 512, 64, True, seed=4)
    T = sum(q_lens)
    g = torch.Generator(device="cuda").manual_seed(9)
    sp = torch.full((T, topk), -1, dtype=torch.int32, device="cuda")
    t = 0
    for i, (ql, n) in enumerate(zip(q_lens, ctxs)):
        for j in range(ql):
            vis = n - ql + j + 1                                  # keys this row may see
            pick = torch.randperm(vis, device="cuda", generator=g)[: min(topk, vis)]
            phys = ref.logical_to_physical(pick.to(torch.int32).unsqueeze(0), bt[i:i + 1], 64)[0]
            sp[t, : phys.numel()] = phys
            if phys.numel() > 8:
                sp[t, torch.randperm(phys.numel(), device="cuda", generator=g)[:5]] = -1     # holes inside the list
            t += 1
    got = k.mla_attention_paged(q, cache, bt, cu, cl, 0.0722, 512, sparse_indices=sp, splits=splits)
    want = ref.mla_attention_paged(q, cache, bt, cu, cl, 0.0722, 512, sparse_indices=sp)
    assert _rel(got, want) < 6e-2, _rel(got, want)
    assert torch.isfinite(got.float()).all()


@pytest.mark.parametrize("H", [128, 16])
@pytest.mark.parametrize("q_lens,ctx_lens", [([1], [64]), ([1, 1, 1], [1, 65, 700]), ([2, 2], [130, 257]), ([40, 9], [40, 200])])
@pytest.mark.parametrize("splits", [1, 3])
def test_mla_fp8_tcgen05(k, H, q_lens, ctx_lens, splits):
    q, cache, bt, cu, cl = _paged_case(q_lens, ctx_lens, H, 576, 512, 64, True, seed=1)
    got = k.mla_attention_paged(q, cache, bt, cu, cl, 0.0722, 512, splits=splits)
    want = ref.mla_attention_paged(q, cache, bt, cu, cl, 0.0722, 512)
    # P is rounded to e4m3 before P V, as in every fp8 attention kernel: a few percent relative error
    assert _rel(got, want) < 6e-2, _rel(got, want)


def test_gqa_attention(k):
    g = torch.Generator(device="cuda").manual_seed(3)
    Hq, Hkv, D, bs = 16, 4, 128, 16
    q_lens, ctx = [3, 1], [35, 50]
    kc = (torch.randn(12, bs, Hkv, D, device="cuda", generator=g)).to(torch.bfloat16)
    vc = (torch.randn(12, bs, Hkv, D, device="cuda", generator=g)).to(torch.bfloat16)
    bt = torch.tensor([[3, 1, 7, 0], [2, 9, 4, 5]], dtype=torch.int32, device="cuda")
    q = torch.randn(4, Hq, D, device="cuda", generator=g).to(torch.bfloat16)
    cu = torch.tensor([0, 3, 4], dtype=torch.int32, device="cuda"); cl = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    got = k.gqa_attention_paged(q, kc, vc, bt, cu, cl, D ** -0.5)
    want = ref.gqa_attention_paged(q, kc, vc, bt, cu, cl, D ** -0.5)
    assert _rel(got, want) < 1e-2


@pytest.mark.parametrize("Hq,Hkv", [(16, 1), (8, 1), (64, 4), (4, 4), (32, 2)])
@pytest.mark.parametrize("q_lens,ctx_lens", [([1], [64]), ([1, 1, 1], [1, 65, 700]), ([2, 3], [130, 257]), ([40, 9, 1], [40, 200, 64]), ([300], [420]), ([1], [2000]), ([1, 2], [3000, 1500])])
def test_gqa_bf16_tcgen05(k, Hq, Hkv, q_lens, ctx_lens):
    """The tensor-core GQA kernel (64-token pages, head dim 128) against the fp32 statement: decode, multi-token verify,
    prefill and chunked prefill, tiles that span several tokens of a sequence, per-row causal limits."""
    g = torch.Generator(device="cuda").manual_seed(11)
    D, bs = 128, 64
    B = len(q_lens)
    nb = [(c + bs - 1) // bs for c in ctx_lens]
    nblk = sum(nb) + 2
    kc = torch.randn(nblk, bs, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn(nblk, bs, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    perm = (torch.randperm(nblk - 1, device="cuda", generator=g)[: sum(nb)] + 1).to(torch.int32)
    bt = torch.zeros(B, max(nb), dtype=torch.int32, device="cuda")
    o = 0
    for i, n in enumerate(nb):
        bt[i, :n] = perm[o:o + n]; o += n
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device="cuda", generator=g).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device="cuda")
    got = k.gqa_attention_paged(q, kc, vc, bt, cu, cl, D ** -0.5)
    want = ref.gqa_attention_paged(q, kc, vc, bt, cu, cl, D ** -0.5)
    assert _rel(got, want) < 1.5e-2, _rel(got, want)


def test_sampler(k):
    torch.manual_seed(0)
    logits = torch.randn(6, 129280, device="cuda")
    temps = torch.tensor([0.0, 0.0, 1.0, 1.0, 0.7, 0.0], device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(5)
    tok, lp = k.sample(logits, temps, gen, True)
    assert torch.equal(tok[[0, 1, 5]], logits.argmax(-1)[[0, 1, 5]])
    want_lp = torch.log_softmax(logits, -1).gather(1, tok.unsqueeze(1)).squeeze(1)
    assert torch.allclose(lp, want_lp, atol=1e-3)
    # Gumbel-max follows softmax(logits / T): empirical frequencies over a small vocabulary
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device="cuda").repeat(4096, 1)
    t2, _ = k.sample(small, torch.ones(4096, device="cuda"), gen, False)
    freq = torch.bincount(t2, minlength=4).float() / 4096
    assert torch.allclose(freq, torch.softmax(small[0], -1), atol=0.03)


def test_dsa_model_end_to_end_takes_the_sparse_tensor_core_path():
    """A small DeepSeek-V3.2-style model (lightning indexer in every layer, top-64 of a ~200-token context, fp8 latent cache
    of the 576-byte geometry): prefill and decode select keys with the indexer kernels and attend them through the sparse
    tcgen05 kernel; CUDA-graph replay and eager execution give the same tokens."""
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models.config import tiny_deepseek_v3
    from nanoengine_b200.ops import sm100, sm100_attn
    mc = tiny_deepseek_v3(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024, q_lora_rank=256, kv_lora_rank=512,
                          qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_attention_heads=16, quant="fp8",
                          index_topk=64, index_n_heads=8, index_head_dim=128)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (200, 150, 90)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        before = sm100_attn.SPARSE_TC_CALLS[0]
        llm = LLM(Config(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kv_cache_dtype="fp8",
                         kvcache_block_size=64, num_kvcache_blocks=64, max_num_seqs=8, enforce_eager=eager, seed=0))
        outs[eager] = [o["token_ids"] for o in llm.generate(prompts, sp)]
        if eager:
            assert sm100_attn.SPARSE_TC_CALLS[0] > before, "the DSA layers did not reach the sparse tensor-core kernel"
        del llm
        torch.cuda.empty_cache()
    assert all(len(t) == 8 for t in outs[True])
    same = sum(a == b for a, b in zip(outs[True], outs[False]))
    assert same >= 2 and all(a[:3] == b[:3] for a, b in zip(outs[True], outs[False])), outs
    assert sm100.kernel_status()[0] == 0


@pytest.mark.parametrize("H,lens", [(4, [300, 1, 64, 129]), (16, [2048]), (2, [128, 128, 5])])
def test_mla_prefill_ragged_tcgen05(k, H, lens):
    """Non-absorbed MLA prefill (192-wide queries / keys with a rotary key part shared by the heads, 128-wide values) against the
    fp32 statement; q and the rotary keys are strided views, as the model passes them."""
    torch.manual_seed(11)
    T = sum(lens)
    q = (torch.randn(T, H * 192 + 64, device="cuda") * 0.5).to(torch.bfloat16)[:, : H * 192].view(T, H, 192)
    kn = (torch.randn(T, H, 128, device="cuda") * 0.5).to(torch.bfloat16)
    kr = (torch.randn(T, 576, device="cuda") * 0.5).to(torch.bfloat16)[:, 512:]
    v = torch.randn(T, H, 128, device="cuda").to(torch.bfloat16)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    want = ref.mla_prefill_ragged(q.float(), kn.float(), kr.float(), v.float(), cu, 192 ** -0.5)
    from nanoengine_b200.ops import sm100
    got = sm100.mla_prefill_ragged(q, kn, kr, v, cu, 192 ** -0.5)
    assert _rel(got, want) < 1e-2


def test_nonabsorbed_prefill_gives_the_absorbed_form_s_logits():
    """The same prompts through the absorbed (576 / 512-wide, paged) and the non-absorbed (192 / 128-wide, ragged) prefill: the
    logits of the first generated token agree, and so do the tokens that follow (the cache both leave is the same)."""
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models import deepseek
    from nanoengine_b200.models.config import tiny_deepseek_v3
    mc = tiny_deepseek_v3(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024, q_lora_rank=256, kv_lora_rank=512,
                          qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_attention_heads=16)
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (300, 70, 129)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = {}
    for flag in (True, False):
        deepseek.NONABSORBED_PREFILL = flag
        try:
            llm = LLM(Config(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kvcache_block_size=64,
                             num_kvcache_blocks=64, max_num_seqs=4, enforce_eager=True, seed=0, enable_prefix_caching=False))
            outs[flag] = [o["token_ids"] for o in llm.generate(prompts, sp)]
        finally:
            deepseek.NONABSORBED_PREFILL = True
        del llm
        torch.cuda.empty_cache()
    same = sum(a == b for a, b in zip(outs[True], outs[False]))
    assert same >= 2 and all(a[:2] == b[:2] for a, b in zip(outs[True], outs[False])), outs
