"""Gated delta-net kernels and the hybrid model on the GPU against the plain PyTorch statement of the same operators."""
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


@pytest.mark.parametrize("lens,uniform", [([1] * 9, True), ([7, 1, 2, 30, 3], False)])
def test_conv_with_carried_window(k, lens, uniform):
    torch.manual_seed(0)
    C, K, B = 384, 4, len(lens)
    T = sum(lens)
    x = torch.randn(T, C + 64, device="cuda", dtype=torch.bfloat16)[:, :C]          # a strided view, as the model passes
    w = (torch.randn(C, K, device="cuda") * 0.3).to(torch.bfloat16)
    state = torch.randn(B + 2, K - 1, C, device="cuda", dtype=torch.bfloat16)
    slots = torch.randperm(B + 2, device="cuda")[:B].int()
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    fresh = (torch.arange(B, device="cuda") % 3 == 0).int()
    st_ref = state.clone()
    want = ref.gdn_conv(x, w, st_ref, slots, cu, fresh)
    got = k.gdn_conv(x, w, state, slots, cu, fresh, uniform)
    assert _rel(got, want) < 5e-3
    assert torch.equal(state, st_ref)


@pytest.mark.parametrize("Dk,Dv,Hk,Hv", [(128, 128, 2, 4), (64, 64, 2, 2), (32, 32, 1, 4), (128, 64, 1, 2)])
@pytest.mark.parametrize("lens", [[1] * 5, [3, 1, 17, 2]])
def test_recurrent_step_kernel(k, Dk, Dv, Hk, Hv, lens):
    torch.manual_seed(1)
    B, T = len(lens), sum(lens)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    q, kk = torch.randn(T, Hk, Dk, **bf), torch.randn(T, Hk, Dk, **bf)
    v, z = torch.randn(T, Hv, Dv, **bf), torch.randn(T, Hv, Dv, **bf)
    ab = torch.randn(T, 2 * Hv, **bf)
    a, b = ab[:, :Hv], ab[:, Hv:]
    A_log, dtb = torch.rand(Hv, device="cuda"), torch.randn(Hv, device="cuda")
    nw = (torch.rand(Dv, device="cuda") + 0.5).to(torch.bfloat16)
    state = torch.randn(B + 1, Hv, Dv, Dk, device="cuda") * 0.2
    slots = torch.randperm(B + 1, device="cuda")[:B].int()
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    fresh = (torch.arange(B, device="cuda") % 2 == 1).int()
    st_ref = state.clone()
    want = ref.gdn_recurrent(q, kk, v, a, b, A_log, dtb, st_ref, slots, cu, fresh, z, nw, 1e-6)
    got = k.gdn_recurrent(q, kk, v, a, b, A_log, dtb, state, slots, cu, fresh, z, nw, 1e-6, max(lens), None)
    assert _rel(got, want) < 1e-2
    assert _rel(state, st_ref) < 1e-4


def test_long_sequences_take_the_chunked_form(k):
    torch.manual_seed(2)
    lens = [200, 5, 64]
    Hk, Hv, Dk, Dv = 2, 4, 128, 128
    B, T = len(lens), sum(lens)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    q, kk = torch.randn(T, Hk, Dk, **bf), torch.randn(T, Hk, Dk, **bf)
    v, z = torch.randn(T, Hv, Dv, **bf), torch.randn(T, Hv, Dv, **bf)
    a, b = torch.randn(T, Hv, **bf), torch.randn(T, Hv, **bf)
    A_log, dtb = torch.rand(Hv, device="cuda"), torch.randn(Hv, device="cuda")
    nw = (torch.rand(Dv, device="cuda") + 0.5).to(torch.bfloat16)
    state = torch.randn(B, Hv, Dv, Dk, device="cuda") * 0.2
    slots = torch.arange(B, device="cuda").int()
    cu_host = [0, 200, 205, 269]
    cu = torch.tensor(cu_host, dtype=torch.int32, device="cuda")
    fresh = torch.tensor([1, 0, 0], dtype=torch.int32, device="cuda")
    # oracle: the token-by-token scan in fp64-free fp32 on the CPU
    st_ref = state.cpu().clone()
    saved = ref.GDN_CHUNK_MIN_TOKENS
    try:
        ref.GDN_CHUNK_MIN_TOKENS = 1 << 30
        want = ref.gdn_recurrent(q.cpu(), kk.cpu(), v.cpu(), a.cpu(), b.cpu(), A_log.cpu(), dtb.cpu(), st_ref, slots.cpu(), cu.cpu(),
                                 fresh.cpu(), z.cpu(), nw.cpu(), 1e-6)
    finally:
        ref.GDN_CHUNK_MIN_TOKENS = saved
    got = k.gdn_recurrent(q, kk, v, a, b, A_log, dtb, state, slots, cu, fresh, z, nw, 1e-6, 200, cu_host)
    assert _rel(got.cpu(), want) < 1e-2
    assert _rel(state.cpu(), st_ref) < 1e-3


def test_rmsnorm_unit_offset_and_sigmoid_gate(k):
    torch.manual_seed(3)
    x = torch.randn(37, 256, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(256, device="cuda") * 0.1).to(torch.bfloat16)
    assert _rel(k.rmsnorm(x, w, 1e-6, False, True), ref.rmsnorm(x, w, 1e-6, False, True)) < 5e-3
    r = torch.randn_like(x)
    y, res = k.add_rmsnorm(x, r, w, 1e-6, True)
    y2, res2 = ref.add_rmsnorm(x, r, w, 1e-6, True)
    assert _rel(y, y2) < 5e-3 and torch.equal(res, res2)
    qg = torch.randn(19, 4, 64, device="cuda", dtype=torch.bfloat16)
    o = torch.randn(19, 4, 32, device="cuda", dtype=torch.bfloat16)
    assert _rel(k.sigmoid_gate(o, qg[..., 32:]), ref.sigmoid_gate(o, qg[..., 32:])) < 5e-3


@pytest.mark.parametrize("moe", [False, True])
def test_hybrid_model_on_gpu_graph_and_eager_agree(moe):
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models.config import tiny_qwen3_5
    mc = tiny_qwen3_5(moe=moe, hidden_size=256, head_dim=128, num_attention_heads=4, num_key_value_heads=2, linear_key_head_dim=64,
                      linear_value_head_dim=64, intermediate_size=512, moe_intermediate_size=128,
                      shared_expert_intermediate_size=128 if moe else 0)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (100, 9, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(Config(model="tiny-qwen3.5", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kvcache_block_size=64,
                         num_kvcache_blocks=32, max_num_seqs=4, enforce_eager=eager))
        outs[eager] = [o["token_ids"] for o in llm.generate(prompts, sp)]
        # the same prompts again: recycled state slots must start clean
        again = [o["token_ids"] for o in llm.generate(prompts, sp)]
        assert again == outs[eager]
    assert outs[True] == outs[False]


def _step_logits(runner, C, seqs, new_tokens, state_slots, is_prefill):
    """One engine step through the worker's own input preparation: `seqs` are the token lists after the step, `new_tokens` how many
    of each are fed now; returns the logits of every sequence's last token."""
    bs = runner.plan.block_size
    b = C.RunnerIn()
    b.is_prefill = is_prefill
    b.seq_ids = list(range(len(seqs)))
    b.input_ids = [t for s, n in zip(seqs, new_tokens) for t in s[len(s) - n:]]
    b.positions = [p for s, n in zip(seqs, new_tokens) for p in range(len(s) - n, len(s))]
    b.q_lens, b.seq_lens = list(new_tokens), [len(s) for s in seqs]
    tables, offs, nxt = [], [0], 0
    for s in seqs:
        nb = 4                                             # four pages reserved per sequence
        tables += list(range(nxt, nxt + nb)); nxt += nb; offs.append(len(tables))
    b.block_tables, b.block_offsets = tables, offs
    b.temperatures, b.sample_mask = [0.0] * len(seqs), [1] * len(seqs)
    b.state_slots = list(state_slots)
    b.handoff_slots = b.hisparse_slots = [-1] * len(seqs)
    ctx = runner.prepare(b)
    hidden = runner.forward(ctx)
    return runner.model.compute_logits(hidden[ctx.last_token_indices.long()]).float().cpu()


@pytest.mark.parametrize("moe", [False, True])
def test_hybrid_model_logits_match_fp32_cpu_model(moe):
    """The bf16 CUDA model against the fp32 CPU model on identical (bf16-rounded) weights: a ragged prefill, then decode steps.
    The routed variant selects every expert (top-8 of 8), so no near-tie in a bf16 router can send a token to another expert
    and the comparison stays a smooth function of the rounding error."""
    from nanoengine_b200 import Config
    from nanoengine_b200._native import _core as C
    from nanoengine_b200.models.config import tiny_qwen3_5
    from nanoengine_b200.models.weights import random_hf_weights
    from nanoengine_b200.runtime.model_runner import ModelRunner
    mc = tiny_qwen3_5(moe=moe, hidden_size=256, head_dim=128, num_attention_heads=4, num_key_value_heads=2, linear_key_head_dim=64,
                      linear_value_head_dim=64, intermediate_size=512, moe_intermediate_size=128,
                      shared_expert_intermediate_size=128 if moe else 0, num_experts_per_tok=8 if moe else 2)
    W = [(n, t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=5, std=0.05)]
    g = torch.Generator().manual_seed(6)
    seqs = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (100, 9, 70)]
    runners = {}
    for dev, dt in (("cpu", "float32"), ("cuda", "bfloat16")):
        r = ModelRunner(Config(model="tiny-qwen3.5", model_config=mc, dummy_weight=True, dtype=dt, device=dev, kvcache_block_size=64,
                               num_kvcache_blocks=16, max_num_seqs=4, enforce_eager=True))
        r.init_model()
        r.load_weights(iter(W))
        r.allocate_kvcache(16)
        runners[dev] = r
    slots = [2, 0, 1]
    cur = [list(s) for s in seqs]
    for step in range(4):
        new = [len(s) for s in cur] if step == 0 else [1] * len(cur)
        lc = _step_logits(runners["cpu"], C, cur, new, slots, step == 0)
        lg = _step_logits(runners["cuda"], C, cur, new, slots, step == 0)
        assert _rel(lg, lc) < (8e-2 if moe else 5e-2), f"step {step}: {_rel(lg, lc)}"      # eight bf16 experts per token add their rounding
        nxt = lc.argmax(-1).tolist()                       # both models continue with the fp32 model's tokens
        cur = [s + [t] for s, t in zip(cur, nxt)]


def test_hybrid_model_with_fp8_weights_runs_graph_and_eager():
    """fp8 block-scaled projections and experts under the delta-net and gated-attention layers (pre-quantised activations from the
    fused norms included): graph replay and eager launches must produce the same tokens."""
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models.config import tiny_qwen3_5
    mc = tiny_qwen3_5(moe=True, hidden_size=256, head_dim=128, num_attention_heads=4, num_key_value_heads=2, linear_key_head_dim=64,
                      linear_value_head_dim=64, intermediate_size=512, moe_intermediate_size=128, shared_expert_intermediate_size=128,
                      quant="fp8")
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 12)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = []
    for eager in (True, False):
        llm = LLM(Config(model="tiny-qwen3.5", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kvcache_block_size=64,
                         num_kvcache_blocks=32, max_num_seqs=4, enforce_eager=eager))
        outs.append([o["token_ids"] for o in llm.generate(prompts, sp)])
    assert outs[0] == outs[1] and all(len(o) == 6 for o in outs[0])
