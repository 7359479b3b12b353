"""The fp8 GEMM whose block scales are applied by the tensor cores ("ue8m0" scale format: powers of two handed to
tcgen05.mma.kind::mxf8f6f4.block_scale through TMEM) against the fp32 statement of the same quantised product."""
import pytest
import torch

from nanoengine_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


@pytest.fixture()
def k():
    from nanoengine_b200.ops import sm100
    sm100.lib()
    sm100.clear_kernel_status()
    sm100.set_scale_format("ue8m0")
    try:
        yield sm100
        assert sm100.kernel_status()[0] == 0, f"a kernel reported a timed-out wait: {sm100.kernel_status()}"
    finally:
        sm100.set_scale_format(None)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _ragged_magnitudes(M, K, N, seed):
    """Activations and weights whose magnitude changes from row to row, from one 128-wide group of K to the next and from one
    weight block to the next by factors of up to 2^12: every (row, K block) and (weight block, K block) has its own scale
    exponent, so a scale byte read from the wrong TMEM lane, column or byte shows as an error of a power of two."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g)
    x = x * torch.exp2(torch.randint(-6, 7, (M, 1), device="cuda", generator=g).float())
    x = (x.view(M, K // 128, 128) * torch.exp2(torch.randint(-3, 4, (1, K // 128, 1), device="cuda", generator=g).float())).view(M, K)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    nb, kb = (N + 127) // 128, K // 128
    blk = torch.exp2(torch.randint(-6, 7, (nb, kb), device="cuda", generator=g).float())
    w = w * blk.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)
    return x.to(torch.bfloat16), w


def test_quantisers_round_scales_up_to_powers_of_two(k):
    torch.manual_seed(0)
    x = torch.randn(77, 1024, device="cuda", dtype=torch.bfloat16) * 3
    q, s = k.quant_fp8_1x128(x)
    rq, rs = ref.quant_fp8_1x128(x, ue8m0=True)
    assert torch.equal(s.contiguous(), rs)                                   # bit-exact scales
    assert bool(((s.contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())
    assert (q.view(torch.uint8) != rq.view(torch.uint8)).float().mean() < 0.02   # rounding-mode ties only
    # the norm and gated-activation producers follow the same setting
    w = torch.randn(1024, device="cuda", dtype=torch.bfloat16)
    qa = k.rmsnorm(x, w, 1e-6, quant=True)
    assert bool(((qa.scales.contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())
    ra = ref.rmsnorm(x, w, 1e-6, quant=True)
    assert _rel(k.dense(qa), ref.dense(ra)) < 2e-2
    h = torch.randn(33, 512, device="cuda", dtype=torch.bfloat16)
    qh = k.silu_and_mul(h, quant=True)
    assert bool(((qh.scales.contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (33, 2112, 7168), (128, 4096, 7168), (500, 7168, 2048), (2048, 2048, 2048),
                                   (300, 384, 640),        # five K blocks: the last scale chunk is partial
                                   (129, 1536, 4096),      # 8 chunks per tile: the scale-factor ring wraps twice
                                   (70, 192, 1024),        # N = 128 + 64: the last tile holds half a weight block
                                   (4096, 4096, 1024),     # the wide (224-column) tile is chosen; 4096 = 18 x 224 + 64
                                   (1000, 7168, 640)])     # 7168 = 32 x 224
def test_gemm_fp8_hw_scaled(k, M, N, K):
    x, w = _ragged_magnitudes(M, K, N, 2)
    wq, ws = ref.quant_fp8_block(w)
    assert bool(((ws.contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())
    got = k.linear(x, wq, ws)
    want = ref.linear(x, wq, ws)          # same quantisation recipe (power-of-two scales) in fp32
    assert _rel(got, want) < 5e-3
    # row by row: a misplaced scale byte hits single rows, which a norm over the whole matrix can hide
    row_err = (got.float() - want.float()).norm(dim=1) / want.float().norm(dim=1).clamp_min(1e-12)
    assert row_err.max().item() < 2e-2, row_err.argmax().item()
    assert _rel(got, x.float() @ w.t()) < 7e-2


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 4096), (1000, 7168, 4224), (640, 7168, 4096), (2047, 4256, 5120)])
def test_gemm_fp8_cta_pairs_equal_single_ctas(k, M, N, K):
    """256-row tiles worked on by two CTAs (tcgen05.mma.cta_group::2, each CTA half of B's rows) against the same GEMM on single
    CTAs and against the fp32 statement; row counts that leave the second CTA of the last pair partly or wholly without rows."""
    x, w = _ragged_magnitudes(M, K, N, 11)
    wq, ws = ref.quant_fp8_block(w)
    want = ref.linear(x, wq, ws)
    xq, xs = k.quant_fp8_1x128_raw(x)
    lib = k.lib()

    def run():
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        k._gemm(xq, K, 0, wq, out, N, 0, M, N, K, 1, None, None, True, xs, M, 0, ws, False, bn=224)
        return out

    pair = run()
    was = lib.ne_gemm_set_pair(0)
    try:
        single = run()
    finally:
        lib.ne_gemm_set_pair(was)
    assert _rel(pair, want) < 5e-3 and _rel(single, want) < 5e-3
    row_err = (pair.float() - want.float()).norm(dim=1) / want.float().norm(dim=1).clamp_min(1e-12)
    assert row_err.max().item() < 2e-2, row_err.argmax().item()
    assert torch.equal(pair, single)          # the same products summed in the same order


def test_grouped_gemm_fp8_cta_pairs(k):
    """Contiguous grouped layout with groups of 0, 130, 600 and 1000 rows: pair tiles that end inside the next group's rows store only
    their own."""
    gen = torch.Generator(device="cuda").manual_seed(12)
    E, N, K = 4, 4480, 4096
    counts = torch.tensor([600, 130, 0, 1000], dtype=torch.int32, device="cuda")
    starts = torch.tensor([0, 640, 896, 896, 1920], dtype=torch.int32, device="cuda")
    R = 2048
    x = (torch.randn(R, K, device="cuda", generator=gen) * torch.exp2(torch.randint(-4, 5, (R, 1), device="cuda", generator=gen).float())).to(torch.bfloat16)
    w = torch.randn(E, N, K, device="cuda", generator=gen) * 0.05
    wq, ws = ref.quant_fp8_block(w)
    xq, xs = k.quant_fp8_1x128_raw(x)
    out = torch.full((R, N), 7.0, device="cuda", dtype=torch.bfloat16)
    k._gemm(xq, K, 0, wq, out, N, 0, R, N, K, E, counts, starts, True, xs, R, 0, ws, False, bn=224)
    for e in range(E):
        lo, n = int(starts[e]), int(counts[e])
        if n:
            assert _rel(out[lo:lo + n], ref.linear(x[lo:lo + n], wq[e], ws[e])) < 5e-3, e
    assert bool((out[600:640] == 7.0).all()) and bool((out[770:896] == 7.0).all())          # rows between the groups stay untouched


@pytest.mark.parametrize("bn", [32, 64, 128, 224])      # 224: tiles straddle up to three weight blocks, B's scale factors are per column
def test_gemm_fp8_hw_scaled_every_tile_width(k, bn):
    M, N, K = 200, 768, 1536
    x, w = _ragged_magnitudes(M, K, N, 5)
    wq, ws = ref.quant_fp8_block(w)
    xq, xs = k.quant_fp8_1x128_raw(x)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    k._gemm(xq, K, 0, wq, out, N, 0, M, N, K, 1, None, None, True, xs, M, 0, ws, False, bn=bn)
    want = ref.linear(x, wq, ws)
    row_err = (out.float() - want.float()).norm(dim=1) / want.float().norm(dim=1).clamp_min(1e-12)
    assert row_err.max().item() < 2e-2


@pytest.mark.parametrize("M,N,K", [(128, 2112, 7168), (5, 4096, 7168), (77, 7168, 2048), (16, 520, 1024)])
def test_small_m_gemms_keep_the_promotion_path_and_its_split_k(k, M, N, K):
    """At most 128 rows: one wave of tiles bound by the weight stream, where the library keeps the CUDA-core promotion kernel (it
    takes any scales, powers of two included) and its split-K form."""
    x, w = _ragged_magnitudes(M, K, N, 7)
    wq, ws = ref.quant_fp8_block(w)
    want = ref.linear(x, wq, ws)
    lib = k.lib()
    was = lib.ne_gemm_set_split_k(0)
    try:
        single = k.linear(x, wq, ws)
    finally:
        lib.ne_gemm_set_split_k(was)
    split = k.linear(x, wq, ws)
    assert _rel(split, want) < 5e-3 and _rel(single, want) < 5e-3
    assert _rel(split, single) < 4e-3


@pytest.mark.parametrize("T,E,topk", [(1, 8, 2), (64, 32, 8), (700, 16, 4)])
def test_moe_experts_hw_scaled(k, T, E, topk):
    torch.manual_seed(10)
    H, I = 512, 256
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16) * torch.exp2(torch.randint(-4, 5, (T, 1), device="cuda").float()).to(torch.bfloat16)
    w13 = torch.randn(E, 2 * I, H, device="cuda") * 0.05 * torch.exp2(torch.randint(-3, 4, (E, 1, 1), device="cuda").float())
    w2 = torch.randn(E, H, I, device="cuda") * 0.05
    logits = torch.randn(T, E, device="cuda")
    idx, w = ref.moe_route(logits, None, topk, 1, 1, True, 1.0, "softmax")
    w13q, s13 = ref.quant_fp8_block(w13)
    w2q, s2 = ref.quant_fp8_block(w2)
    got = k.moe_experts(x, idx, w, w13q, w2q, s13, s2, 0)
    want = ref.moe_experts(x, idx, w, w13q, w2q, s13, s2, 0)
    assert _rel(got, want) < 2e-2
    row_err = (got.float() - want.float()).norm(dim=1) / want.float().norm(dim=1).clamp_min(1e-12)
    assert row_err.max().item() < 6e-2


def test_checkpoint_scales_are_requantised_for_the_format(k):
    torch.manual_seed(4)
    w = torch.randn(256, 512, device="cuda") * 0.05
    wq, ws = ref.quant_fp8_block(w, ue8m0=False)
    q2, s2 = ref.fp8_block_for_format(wq, ws)
    assert bool(((s2.contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())
    assert _rel(ref.dequant_fp8_block(q2, s2), ref.dequant_fp8_block(wq, ws)) < 4e-2
    q3, s3 = ref.fp8_block_for_format(q2, s2)          # already powers of two: untouched
    assert torch.equal(q3.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s3, s2)


def test_engine_under_ue8m0_reaches_the_tensor_core_scaled_gemm():
    """A small fp8 DeepSeek-style model served with power-of-two scales: the prefill GEMMs (more than 128 rows) take the
    tensor-core-scaled kernel, decode replays from CUDA graphs, and eager and graph execution give the same tokens."""
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models.config import tiny_deepseek_v3
    from nanoengine_b200.ops import sm100
    mc = tiny_deepseek_v3(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024, q_lora_rank=256, kv_lora_rank=512,
                          qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_attention_heads=16, quant="fp8", scale_fmt="ue8m0")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (300, 150, 9)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    try:
        for eager in (True, False):
            before = sm100.TC_SCALED_GEMMS[0]
            llm = LLM(Config(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kv_cache_dtype="fp8",
                             kvcache_block_size=64, num_kvcache_blocks=64, max_num_seqs=8, enforce_eager=eager, seed=0))
            assert sm100.scale_format() == "ue8m0"
            lin = next(m for m in llm.engine.executor.runner.model.modules() if getattr(m, "weight_scale_inv", None) is not None)
            assert bool(((lin.weight_scale_inv.float().contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())
            outs[eager] = [o["token_ids"] for o in llm.generate(prompts, sp)]
            assert sm100.TC_SCALED_GEMMS[0] > before
            del llm
            torch.cuda.empty_cache()
    finally:
        sm100.set_scale_format(None)
    assert all(len(t) == 8 for t in outs[True])
    same = sum(a == b for a, b in zip(outs[True], outs[False]))
    assert same >= 2 and all(a[:3] == b[:3] for a, b in zip(outs[True], outs[False])), outs
    assert sm100.kernel_status()[0] == 0
