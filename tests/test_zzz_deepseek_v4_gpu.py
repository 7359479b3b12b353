"""DeepSeek-V4 on the GPU: the bf16 CUDA model (this package's GEMM / norm / hyper-connection / router / expert kernels around the
PyTorch-op compressor and window / pooled-row attention) against the fp32 CPU model on the same weights.  Runs after every other
GPU test file."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


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


@pytest.mark.xfail(strict=False, reason="this family had not run on a GPU when the test was written; a pass is reported as XPASS")
@pytest.mark.parametrize("kv", ["auto", "fp8"])
def test_deepseek_v4_logits_match_fp32_cpu_model(kv):
    """A ragged prefill, then decode steps that cross compression-block boundaries of both ratios.  Every expert is selected (top-8
    of 8) so that no near-tie in a bf16 router sends a token elsewhere."""
    from nanoengine_b200 import Config
    from nanoengine_b200._native import _core as C
    from nanoengine_b200.models.config import tiny_deepseek_v4
    from nanoengine_b200.models.weights import random_hf_weights
    from nanoengine_b200.ops import sm100
    from nanoengine_b200.runtime.model_runner import ModelRunner
    sm100.lib()
    sm100.clear_kernel_status()
    mc = tiny_deepseek_v4(hidden_size=256, q_lora_rank=128, head_dim=192, qk_rope_head_dim=64, num_attention_heads=8, o_groups=2, o_lora_rank=128,
                          window_size=32, compress_ratios=[0, 4, 16], moe_intermediate_size=128, num_experts_per_tok=8, num_hash_layers=1)
    W = [(n, t if t.dtype == torch.int32 else t.to(torch.bfloat16).float()) for n, t in random_hf_weights(mc, seed=5, std=0.05)]
    g = torch.Generator().manual_seed(6)
    seqs = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (100, 9, 70)]
    runners = {}
    for dev, dt in (("cpu", "float32"), ("cuda", "bfloat16")):
        r = ModelRunner(Config(model="tiny", model_config=mc, dummy_weight=True, dtype=dt, device=dev, kvcache_block_size=64,
                               num_kvcache_blocks=16, max_num_seqs=4, kv_cache_dtype=kv if dev == "cuda" else "auto"))
        r.init_model()
        r.load_weights(iter(W))
        r.allocate_kvcache(16)
        runners[dev] = r
    slots = [2, 0, 1]
    cur = [list(s) for s in seqs]
    for step in range(5):
        new = [len(s) for s in cur] if step == 0 else [1] * len(cur)
        lc = _step_logits(runners["cpu"], C, cur, new, slots, step == 0)
        lg = _step_logits(runners["cuda"], C, cur, new, slots, step == 0)
        assert _rel(lg, lc) < 1e-1, f"step {step}: {_rel(lg, lc)}"
        cur = [s + [t] for s, t in zip(cur, lc.argmax(-1).tolist())]
    assert sm100.kernel_status()[0] == 0


def test_sqrt_softplus_routing_kernel():
    """The routing kernel's third scoring mode against the PyTorch statement (scores sqrt(softplus(x)), bias only in the choice,
    weights renormalised and scaled), including large logits where softplus(x) = x."""
    from nanoengine_b200.ops import reference as ref
    from nanoengine_b200.ops import sm100
    sm100.lib()
    torch.manual_seed(3)
    logits = torch.randn(37, 256, device="cuda") * 4
    logits[0, :8] = torch.tensor([25.0, 30.0, 41.0, 22.0, 60.0, 21.0, 35.0, 27.0], device="cuda")
    bias = torch.randn(256, device="cuda") * 0.05
    idx, w = sm100.moe_route(logits, bias, 6, 1, 1, True, 1.5, "sqrtsoftplus")
    ridx, rw = ref.moe_route(logits.cpu(), bias.cpu(), 6, 1, 1, True, 1.5, "sqrtsoftplus")
    order, rorder = idx.long().cpu().sort(-1), ridx.long().sort(-1)
    assert torch.equal(order.values, rorder.values)
    assert (w.cpu().gather(1, order.indices) - rw.gather(1, rorder.indices)).abs().max() < 1e-4
