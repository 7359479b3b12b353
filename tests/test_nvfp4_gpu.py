"""NVFP4 (packed e2m1, one e4m3 scale per 16 elements) on the tensor cores: quantiser, grouped GEMM (tcgen05.mma.kind::mxf4nvf4 with the
scale factors in TMEM) and the W4A4 routed-expert path, against the fp32 statement of the same quantised product."""
import pytest
import torch

from nanoengine_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def k():
    from nanoengine_b200.ops import sm100
    sm100.lib()
    sm100.clear_kernel_status()
    yield sm100
    assert sm100.kernel_status()[0] == 0, f"a kernel reported a timed-out wait: {sm100.kernel_status()}"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _random_operand(rows, K, gen, lead=()):
    """Full-entropy operand: random nibbles and random positive e4m3 scales spanning 2^-4 .. 2^3, so that a scale byte read from the
    wrong lane, column or byte of TMEM shows."""
    q = torch.randint(0, 256, (*lead, rows, K // 2), device="cuda", generator=gen, dtype=torch.int32).to(torch.uint8)
    sf = (torch.exp2(torch.randint(-4, 4, (*lead, rows, K // 16), device="cuda", generator=gen).float())
          * (1 + torch.randint(0, 8, (*lead, rows, K // 16), device="cuda", generator=gen).float() / 8)).to(FP8)
    return q, sf


@pytest.mark.parametrize("R,K", [(1, 256), (77, 1024), (300, 7168)])
def test_quantiser_matches_reference(k, R, K):
    torch.manual_seed(0)
    x = (torch.randn(R, K, device="cuda") * torch.exp2(torch.randint(-3, 4, (R, 1), device="cuda").float())).to(torch.bfloat16)
    g = torch.tensor([37.0], device="cuda")
    q, sf = k.nvfp4_quant(x, g)
    rq, rsf = ref.nvfp4_quant(x, g)
    assert (sf.view(torch.uint8) != rsf.view(torch.uint8)).float().mean() < 0.01        # reciprocal rounding at e4m3 ties
    assert _rel(ref.nvfp4_unpack(q, sf), ref.nvfp4_unpack(rq, rsf)) < 2e-2
    assert _rel(ref.nvfp4_unpack(q, sf) / 37.0, x) < 0.13                               # fp4: ~10 % per element


@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (130, 384, 512), (300, 200, 2048), (128, 4096, 7168), (1000, 1536, 4096)])
def test_gemm_nvfp4_dense(k, M, N, K):
    gen = torch.Generator(device="cuda").manual_seed(1)
    aq, asf = _random_operand(M, K, gen)
    bq, bsf = _random_operand(N, K, gen, lead=(1,))
    alpha = torch.tensor([0.37], device="cuda")
    want = ref.nvfp4_gemm(aq, asf, bq, bsf, alpha, out_fp32=True)
    got = k.nvfp4_gemm(aq, asf, bq, bsf, alpha, out_fp32=True)
    assert _rel(got, want) < 1e-4
    row_err = (got - want).norm(dim=1) / want.norm(dim=1).clamp_min(1e-12)
    assert row_err.max().item() < 1e-3, row_err.argmax().item()
    col_err = (got - want).norm(dim=0) / want.norm(dim=0).clamp_min(1e-12)
    assert col_err.max().item() < 1e-3, col_err.argmax().item()
    assert _rel(k.nvfp4_gemm(aq, asf, bq, bsf, alpha), want) < 5e-3                     # bf16 output


def test_gemm_nvfp4_grouped_contiguous(k):
    gen = torch.Generator(device="cuda").manual_seed(2)
    G, N, K = 5, 512, 1024
    counts = torch.tensor([130, 0, 1, 256, 77], dtype=torch.int32, device="cuda")
    starts = torch.tensor([0, 256, 256, 384, 640], dtype=torch.int32, device="cuda")
    R = 768
    aq, asf = _random_operand(R, K, gen)
    bq, bsf = _random_operand(N, K, gen, lead=(G,))
    alpha = torch.rand(G, device="cuda") + 0.5
    want = ref.nvfp4_gemm(aq, asf, bq, bsf, alpha, counts, starts, out_fp32=True)
    got = k.nvfp4_gemm(aq, asf, bq, bsf, alpha, counts, starts, out_fp32=True)
    for g in range(G):
        lo, n = int(starts[g]), int(counts[g])
        if n:
            assert _rel(got[lo:lo + n], want[lo:lo + n]) < 1e-4, g


@pytest.mark.parametrize("T,E,topk", [(1, 8, 2), (64, 32, 8), (700, 16, 4)])
def test_moe_experts_nvfp4(k, T, E, topk):
    torch.manual_seed(3)
    H, I = 512, 256
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w13q, w13sf, s13 = ref.nvfp4_quant_weight(torch.randn(E, 2 * I, H, device="cuda") * 0.05)
    w2q, w2sf, s2 = ref.nvfp4_quant_weight(torch.randn(E, H, I, device="cuda") * 0.05)
    in1 = torch.tensor(4.0 / (6 * 448), device="cuda")                   # activations up to ~4
    in2 = (torch.rand(E, device="cuda") + 0.5) * 2.0 / (6 * 448)
    idx, w = ref.moe_route(torch.randn(T, E, device="cuda"), None, topk, 1, 1, True, 1.0, "softmax")
    args = (x, idx, w, w13q, w13sf, in1 * s13, (1 / in1).reshape(1), w2q, w2sf, in2 * s2, 1 / in2, 0)
    got = k.moe_experts_nvfp4(*args)
    want = ref.moe_experts_nvfp4(*args)
    assert _rel(got, want) < 3e-2            # the intermediate is re-quantised to 4 bits: a rounding tie moves a whole step


def test_engine_with_nvfp4_experts_graph_equals_eager():
    """A small DeepSeek-style model whose routed experts are NVFP4 (W4A4 on the tensor cores), the rest bf16: eager and CUDA-graph
    execution give the same tokens, and the expert module on the GPU agrees with its PyTorch statement on the same weights."""
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models.config import tiny_deepseek_v3
    from nanoengine_b200.ops import sm100
    mc = tiny_deepseek_v3(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024, q_lora_rank=256, kv_lora_rank=512,
                          qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_attention_heads=16, quant="nvfp4")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (300, 150, 9)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(Config(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kvcache_block_size=64,
                         num_kvcache_blocks=64, max_num_seqs=8, enforce_eager=eager, seed=0))
        ex = llm.engine.executor.runner.model.model.layers["1"].mlp.experts
        assert ex.quant == "nvfp4" and ex.gate_up_proj.dtype == torch.uint8
        outs[eager] = [o["token_ids"] for o in llm.generate(prompts, sp)]
        if eager:
            x = torch.randn(50, 512, device="cuda", dtype=torch.bfloat16)
            idx, w = ref.moe_route(torch.randn(50, mc.n_routed_experts, device="cuda"), None, 2, 1, 1, True, 1.0, "softmax")
            args = (x, idx, w, ex.gate_up_proj, ex.gate_up_scale, ex.alpha1, ex.a1_gscale, ex.down_proj, ex.down_scale, ex.alpha2, ex.a2_gscale, 0)
            assert _rel(sm100.moe_experts_nvfp4(*args), ref.moe_experts_nvfp4(*args)) < 3e-2
        del llm
        torch.cuda.empty_cache()
    assert all(len(t) == 8 for t in outs[True])
    same = sum(a == b for a, b in zip(outs[True], outs[False]))
    assert same >= 2 and all(a[:3] == b[:3] for a, b in zip(outs[True], outs[False])), outs
    assert sm100.kernel_status()[0] == 0
