"""Kernels of the GLM5-next / Kimi-K3 families and the two models on the GPU against the plain PyTorch statement of the same
operators (fp32 on the same inputs)."""
import pytest
import torch

from nanoengine_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k():
    from nanoengine_b200.ops import sm100
    sm100.lib()
    sm100.clear_kernel_status()
    yield sm100
    assert sm100.kernel_status()[0] == 0


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("lower_bound", [-5.0, None])
@pytest.mark.parametrize("lens", [[1] * 6, [3, 1, 40, 2], [130]])
def test_kda_recurrent_kernel(k, lens, lower_bound):
    torch.manual_seed(1)
    H, Dk, Dv = 3, 128, 128
    B, T = len(lens), sum(lens)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    y = torch.randn(T, 2 * H * Dk + H * Dv + H * Dv, **bf)                  # [q | k | v | gate] rows, as the layer passes them
    q, kk = y[:, : H * Dk].view(T, H, Dk), y[:, H * Dk: 2 * H * Dk].view(T, H, Dk)
    v, gate = y[:, 2 * H * Dk: 2 * H * Dk + H * Dv].view(T, H, Dv), y[:, 2 * H * Dk + H * Dv:].view(T, H, Dv)
    raw_g = torch.randn(T, H * Dk, **bf)
    ab = torch.randn(T, Dk + H, **bf)
    b = ab[:, Dk:]
    A_log, dtb = torch.rand(H, device="cuda") - 0.5, torch.randn(H * Dk, device="cuda") * 0.5
    nw = (torch.rand(Dv, device="cuda") + 0.5).to(torch.bfloat16)
    state = torch.randn(B + 1, H, Dv, Dk, device="cuda") * 0.2
    slots = torch.randperm(B + 1, device="cuda")[:B].int()
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    fresh = (torch.arange(B, device="cuda") % 2 == 1).int()
    st_ref = state.clone()
    want = ref.kda_recurrent(q, kk, v, raw_g, b, A_log, dtb, lower_bound, st_ref, slots, cu, fresh, gate, nw, 1e-6)
    got = k.kda_recurrent(q, kk, v, raw_g, b, A_log, dtb, lower_bound, state, slots, cu, fresh, gate, nw, 1e-6)
    assert _rel(got, want) < 1e-2
    assert _rel(state, st_ref) < 1e-3


@pytest.mark.parametrize("D,rows,valid,write", [(7168, 9, 8, False), (7168, 4, 1, True), (256, 3, 2, True), (4096, 16, 16, False)])
def test_attention_residual_kernel(k, D, rows, valid, write):
    torch.manual_seed(2)
    T = 37
    big = torch.randn(T, rows + 1, D, device="cuda", dtype=torch.bfloat16)
    bank = big[:, : rows + (1 if write and valid == rows else 0)]
    prefix = torch.randn(T, D + 8, device="cuda", dtype=torch.bfloat16)[:, :D]      # a row-strided view
    ws = torch.randn(D, device="cuda") * 0.05
    wo = (torch.rand(D, device="cuda") + 0.5).to(torch.bfloat16)
    b_ref = bank.clone()
    wr = valid if write else -1
    want = ref.attn_res_mix(prefix, b_ref, valid, ws, wo, 1e-6, wr)
    got = k.attn_res_mix(prefix, bank, valid, ws, wo, 1e-6, wr)
    assert _rel(got, want) < 1e-2
    assert torch.equal(bank, b_ref)


@pytest.mark.parametrize("T,h,D,iters", [(5, 4, 6144, 3), (130, 4, 512, 1), (9, 2, 256, 4), (3, 1, 128, 2)])
def test_hyper_connection_kernels(k, T, h, D, iters):
    torch.manual_seed(3)
    x = torch.randn(T, h, D, device="cuda", dtype=torch.bfloat16)
    fn = torch.randn((2 + h) * h, h * D, device="cuda") * 0.05
    base = torch.randn((2 + h) * h, device="cuda") * 0.3
    scale = torch.tensor([1.0, 0.8, 1.3], device="cuda")
    y0, p0, c0 = ref.mhc_pre(x, fn, base, scale, iters, 1e-6)
    y1, p1, c1 = k.mhc_pre(x, fn, base, scale, iters, 1e-6)
    assert _rel(y1, y0) < 1e-2 and _rel(p1, p0) < 1e-2 and _rel(c1, c0) < 1e-2
    sub = torch.randn(T, D + 16, device="cuda", dtype=torch.bfloat16)[:, :D]
    assert _rel(k.mhc_post(sub, x, p0, c0), ref.mhc_post(sub, x, p0, c0)) < 5e-3


@pytest.mark.parametrize("act", [None, ("clamp", 2.0), ("situ", 4.0, 25.0), ("situ", 4.0, None)])
def test_gated_activation_kernel(k, act):
    torch.manual_seed(4)
    x = (torch.randn(70, 512, device="cuda") * 6).to(torch.bfloat16)
    want = ref.silu_and_mul(x, act=act)
    assert _rel(k.silu_and_mul(x, act=act), want) < 5e-3
    qa = k.silu_and_mul(x, True, act=act)                                           # e4m3 [T, I] with scales [I / 128, T]
    deq = qa.q.float().view(70, 2, 128) * qa.scales.t().reshape(70, 2, 1)
    assert _rel(deq.view(70, 256), want) < 4e-2
    o, g = torch.randn(33, 256, device="cuda", dtype=torch.bfloat16), torch.randn(33, 512, device="cuda", dtype=torch.bfloat16)[:, :256]
    assert _rel(k.sigmoid_mul(o, g), ref.sigmoid_mul(o, g)) < 5e-3


def _gpu_config(make, **over):
    base = dict(hidden_size=256, q_lora_rank=128, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                num_attention_heads=8, intermediate_size=512, moe_intermediate_size=128, linear_key_head_dim=128, linear_value_head_dim=128)
    base.update(over)
    return make(**base)


def _step_logits(runner, C, seqs, new_tokens, state_slots, is_prefill):
    b = C.RunnerIn()
    b.is_prefill = is_prefill
    b.seq_ids = list(range(len(seqs)))
    b.input_ids = [t for s, n in zip(seqs, new_tokens) for t in s[len(s) - n:]]
    b.positions = [p for s, n in zip(seqs, new_tokens) for p in range(len(s) - n, len(s))]
    b.q_lens, b.seq_lens = list(new_tokens), [len(s) for s in seqs]
    tables, offs, nxt = [], [0], 0
    for s in seqs:
        tables += list(range(nxt, nxt + 4)); nxt += 4; offs.append(len(tables))
    b.block_tables, b.block_offsets = tables, offs
    b.temperatures, b.sample_mask = [0.0] * len(seqs), [1] * len(seqs)
    b.state_slots = list(state_slots)
    b.handoff_slots = b.hisparse_slots = [-1] * len(seqs)
    ctx = runner.prepare(b)
    hidden = runner.forward(ctx)
    return runner.model.compute_logits(hidden[ctx.last_token_indices.long()]).float().cpu()


@pytest.mark.parametrize("family", ["glm5_next", "kimi_k3"])
def test_family_logits_match_fp32_cpu_model(family):
    """bf16 CUDA model against the fp32 CPU model on identical (bf16-rounded) weights: a ragged prefill, then decode steps.  Every
    expert is selected (top-8 of 8) so that no near-tie in a bf16 router sends a token elsewhere."""
    from nanoengine_b200 import Config
    from nanoengine_b200._native import _core as C
    from nanoengine_b200.models import config as mcfg
    from nanoengine_b200.models.weights import random_hf_weights
    from nanoengine_b200.runtime.model_runner import ModelRunner
    make = mcfg.tiny_glm5_next if family == "glm5_next" else mcfg.tiny_kimi_k3
    over = dict(num_experts_per_tok=8, n_group=1, topk_group=1)
    if family == "glm5_next":
        over.update(index_n_heads=0)                       # dense MLA here; the indexer path has its own test
    else:
        over.update(routed_expert_hidden_size=128)
    mc = _gpu_config(make, **over)
    W = [(n, t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=5, std=0.05)]
    g = torch.Generator().manual_seed(6)
    seqs = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (100, 9, 70)]
    runners = {}
    for dev, dt in (("cpu", "float32"), ("cuda", "bfloat16")):
        r = ModelRunner(Config(model="tiny", model_config=mc, dummy_weight=True, dtype=dt, device=dev, kvcache_block_size=64,
                               num_kvcache_blocks=16, max_num_seqs=4, enforce_eager=True))
        r.init_model()
        r.load_weights(iter(W))
        r.allocate_kvcache(16)
        runners[dev] = r
    slots = [2, 0, 1]
    cur = [list(s) for s in seqs]
    for step in range(3):
        new = [len(s) for s in cur] if step == 0 else [1] * len(cur)
        lc = _step_logits(runners["cpu"], C, cur, new, slots, step == 0)
        lg = _step_logits(runners["cuda"], C, cur, new, slots, step == 0)
        assert _rel(lg, lc) < 8e-2, f"step {step}: {_rel(lg, lc)}"
        cur = [s + [t] for s, t in zip(cur, lc.argmax(-1).tolist())]


@pytest.mark.parametrize("family", ["glm5_next", "kimi_k3"])
def test_family_on_gpu_graph_and_eager_agree(family):
    """fp8 experts and MLA projections, the fp8 latent cache (GLM5-next also with the lightning indexer and sparse attention):
    CUDA-graph replay and eager launches give the same tokens, and recycled state slots start clean."""
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models import config as mcfg
    from nanoengine_b200.ops import sm100
    make = mcfg.tiny_glm5_next if family == "glm5_next" else mcfg.tiny_kimi_k3
    over = dict(quant="fp8")
    if family == "glm5_next":
        over.update(index_n_heads=4, index_head_dim=128, index_topk=64, hc_mult=4)
    else:
        over.update(routed_expert_hidden_size=128)
    mc = _gpu_config(make, **over)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (150, 9, 80)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(Config(model="tiny", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kv_cache_dtype="fp8",
                         kvcache_block_size=64, num_kvcache_blocks=32, max_num_seqs=4, enforce_eager=eager, seed=0))
        outs[eager] = [o["token_ids"] for o in llm.generate(prompts, sp)]
        again = [o["token_ids"] for o in llm.generate(prompts, sp)]
        assert again == outs[eager]        # also for the sparse layers: the top-k list comes out in the same order every run
        del llm
        torch.cuda.empty_cache()
    assert all(len(t) == 8 for t in outs[True])
    # the graph pads the batch to its bucket, so the small-M GEMMs take another split and round differently; with random weights
    # (near-uniform logits) one flipped token changes everything after it.  Every prompt must agree on its first tokens, and the
    # runs must not drift apart everywhere.
    same = sum(a == b for a, b in zip(outs[True], outs[False]))
    assert same >= 1 and all(a[:3] == b[:3] for a, b in zip(outs[True], outs[False])), outs
    assert sm100.kernel_status()[0] == 0


# ---- Gemma4 -----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("D,window", [(256, 40), (512, 0), (128, 100), (256, 1)])
def test_windowed_gqa_attention_kernel(k, D, window):
    from nanoengine_b200.ops import sm100_attn
    torch.manual_seed(9)
    Hq, Hkv, bs = 8, 2, 64
    q_lens, ctx_lens = [1, 70, 5], [200, 70, 133]
    nb = sum((c + bs - 1) // bs for c in ctx_lens)
    kc = torch.randn(nb + 1, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(nb + 1, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    bt = torch.zeros(3, 4, dtype=torch.int32, device="cuda")
    nxt = 0
    for i, c in enumerate(ctx_lens):
        n = (c + bs - 1) // bs
        bt[i, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32, device="cuda"); nxt += n
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    cl = torch.tensor(ctx_lens, dtype=torch.int32, device="cuda")
    want = ref.gqa_attention_paged(q.float(), kc.float(), vc.float(), bt, cu, cl, D ** -0.5, window)
    got = sm100_attn.gqa_attention_paged(q, kc, vc, bt, cu, cl, D ** -0.5, window)
    assert _rel(got, want) < 1e-2


def _gemma_gpu_config():
    from nanoengine_b200.models.config import tiny_gemma4
    return tiny_gemma4(hidden_size=256, head_dim=256, global_head_dim=512, num_attention_heads=4, num_key_value_heads=1, intermediate_size=512,
                       hidden_size_per_layer_input=128, sliding_window=48)


def test_gemma4_logits_match_fp32_cpu_model():
    from nanoengine_b200 import Config
    from nanoengine_b200._native import _core as C
    from nanoengine_b200.models.weights import random_hf_weights
    from nanoengine_b200.runtime.model_runner import ModelRunner
    mc = _gemma_gpu_config()
    # the family's softmax scale is one and q / k are RMS-normalised: with random norm weights near one the scores would have a
    # standard deviation of sqrt(head_dim) and the softmax would amplify every rounding error, so the q / k norms are scaled down
    W = [(n, (t * (0.2 if n.endswith(("q_norm.weight", "k_norm.weight")) else 1.0)).to(torch.bfloat16).float())
         for n, t in random_hf_weights(mc, seed=5, std=0.05)]
    g = torch.Generator().manual_seed(6)
    seqs = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (100, 9, 70)]
    runners = {}
    for dev, dt in (("cpu", "float32"), ("cuda", "bfloat16")):
        r = ModelRunner(Config(model="tiny", model_config=mc, dummy_weight=True, dtype=dt, device=dev, kvcache_block_size=64,
                               num_kvcache_blocks=16, max_num_seqs=4, enforce_eager=True))
        r.init_model()
        r.load_weights(iter(W))
        r.allocate_kvcache(16)
        runners[dev] = r
    cur = [list(s) for s in seqs]
    for step in range(3):
        new = [len(s) for s in cur] if step == 0 else [1] * len(cur)
        lc = _step_logits(runners["cpu"], C, cur, new, [-1, -1, -1], step == 0)
        lg = _step_logits(runners["cuda"], C, cur, new, [-1, -1, -1], step == 0)
        assert _rel(lg, lc) < 5e-2, f"step {step}: {_rel(lg, lc)}"
        cur = [s + [t] for s, t in zip(cur, lc.argmax(-1).tolist())]


def test_gemma4_on_gpu_graph_and_eager_agree():
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.ops import sm100
    mc = _gemma_gpu_config()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (150, 9, 80)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(Config(model="tiny", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kvcache_block_size=64,
                         num_kvcache_blocks=32, max_num_seqs=4, enforce_eager=eager, seed=0))
        outs[eager] = [o["token_ids"] for o in llm.generate(prompts, sp)]
        assert [o["token_ids"] for o in llm.generate(prompts, sp)] == outs[eager]
        del llm
        torch.cuda.empty_cache()
    same = sum(a == b for a, b in zip(outs[True], outs[False]))
    assert same >= 2 and all(a[:3] == b[:3] for a, b in zip(outs[True], outs[False])), outs
    assert sm100.kernel_status()[0] == 0
