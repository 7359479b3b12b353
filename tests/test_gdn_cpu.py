"""Gated delta-net pieces on CPU: the convolution with a carried window, the scan and chunked forms of the delta rule, and the
hybrid model end to end (chunked prefill and decode must continue the same recurrence as a one-shot prefill)."""
import pytest
import torch
import torch.nn.functional as F

from nanoengine_b200 import Config, LLM, SamplingParams
from nanoengine_b200.models.config import ModelConfig, tiny_qwen3_5
from nanoengine_b200.ops import reference as ref


def test_conv_matches_conv1d_and_carries_window():
    torch.manual_seed(0)
    C, K = 12, 4
    w = torch.randn(C, K)
    lens = [9, 1, 5]
    x = torch.randn(sum(lens), C)
    cu = torch.tensor([0, 9, 10, 15], dtype=torch.int32)
    slots = torch.tensor([2, 0, 1])
    state = torch.randn(4, K - 1, C)           # stale content that fresh sequences must ignore
    y = ref.gdn_conv(x, w, state, slots, cu, torch.ones(3, dtype=torch.int32))
    off = 0
    for n, slot in zip(lens, slots.tolist()):
        seq = x[off: off + n]
        want = F.silu(F.conv1d(seq.t()[None], w[:, None, :], padding=K - 1, groups=C)[0, :, :n].t())
        assert torch.allclose(y[off: off + n], want, atol=1e-5)
        full = torch.cat([torch.zeros(K - 1, C), seq], 0)
        assert torch.allclose(state[slot], full[-(K - 1):])
        off += n
    # the same sequence fed in two chunks gives the same outputs
    state2 = torch.zeros(4, K - 1, C)
    one = torch.tensor([0], dtype=torch.int32)
    a = ref.gdn_conv(x[:4], w, state2, torch.tensor([3]), torch.tensor([0, 4], dtype=torch.int32), one)
    b = ref.gdn_conv(x[4:9], w, state2, torch.tensor([3]), torch.tensor([0, 5], dtype=torch.int32), one * 0)
    assert torch.allclose(torch.cat([a, b]), y[:9], atol=1e-5)


@pytest.mark.parametrize("n", [64, 150, 257])
def test_chunked_form_equals_scan(n):
    torch.manual_seed(1)
    H, Dk, Dv = 3, 16, 8
    q = ref._l2norm(torch.randn(n, H, Dk)) * Dk ** -0.5
    k = ref._l2norm(torch.randn(n, H, Dk))
    v = torch.randn(n, H, Dv)
    g = -torch.rand(n, H)
    beta = torch.rand(n, H)
    S0 = torch.randn(H, Dv, Dk) * 0.1
    o1, S1 = ref.gdn_scan(q, k, v, g, beta, S0.clone())
    o2, S2 = ref.gdn_chunked(q, k, v, g, beta, S0.clone())
    assert (o1 - o2).abs().max() < 1e-5 and (S1 - S2).abs().max() < 1e-5


def test_recurrent_op_continues_across_calls():
    torch.manual_seed(2)
    T, Hk, Hv, Dk, Dv = 110, 2, 4, 16, 8
    q, k = torch.randn(T, Hk, Dk), torch.randn(T, Hk, Dk)
    v, z = torch.randn(T, Hv, Dv), torch.randn(T, Hv, Dv)
    a, b = torch.randn(T, Hv), torch.randn(T, Hv)
    A_log, dtb, nw = torch.rand(Hv), torch.randn(Hv), torch.rand(Dv) + 0.5
    slots = torch.tensor([1])

    def run(bounds, state):
        outs = []
        for i, (s, e) in enumerate(bounds):
            cu = torch.tensor([0, e - s], dtype=torch.int32)
            outs.append(ref.gdn_recurrent(q[s:e], k[s:e], v[s:e], a[s:e], b[s:e], A_log, dtb, state, slots, cu,
                                          torch.tensor([1 if i == 0 else 0], dtype=torch.int32), z[s:e], nw, 1e-6))
        return torch.cat(outs)

    st1, st2 = torch.randn(3, Hv, Dv, Dk), torch.randn(3, Hv, Dv, Dk)
    whole = run([(0, T)], st1)                                   # chunked form (>= 64 tokens)
    parts = run([(0, 80), (80, 109), (109, 110)], st2)           # chunked, then scan, then a decode step
    assert (whole - parts).abs().max() < 1e-4
    assert (st1[1] - st2[1]).abs().max() < 1e-4


def _llm(mc, **kw):
    base = dict(model="tiny-qwen3.5", model_config=mc, dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=16,
                num_kvcache_blocks=64, max_num_seqs=8)
    base.update(kw)
    if mc is None:
        base.pop("model_config"); base.pop("dummy_weight")
    return LLM(Config(**base))


@pytest.mark.parametrize("moe", [False, True])
def test_hybrid_model_prefill_chunks_and_decode_agree(moe):
    mc = tiny_qwen3_5(moe=moe)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    ref_out = [o["token_ids"] for o in _llm(mc).generate(prompts, sp)]
    # prompts split into 32-token chunks continue the same state
    chunked = [o["token_ids"] for o in _llm(mc, max_num_batched_tokens=32, enable_chunked_prefill=True).generate(prompts, sp)]
    assert chunked == ref_out
    # teacher forcing: the prompt plus the first five generated tokens, prefetched in one pass, predicts the sixth
    forced = _llm(mc).generate([p + o[:5] for p, o in zip(prompts, ref_out)], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    assert [o["token_ids"][0] for o in forced] == [o[5] for o in ref_out]


def test_state_slots_are_recycled_between_requests():
    """More requests than state slots: a slot's stale state must not leak into the next sequence that gets it."""
    mc = tiny_qwen3_5()
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 512, (12 + i,), generator=g).tolist() for i in range(6)]
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    wide = [o["token_ids"] for o in _llm(mc).generate(prompts, sp)]
    narrow = [o["token_ids"] for o in _llm(mc, max_num_seqs=2).generate(prompts, sp)]
    assert wide == narrow


def test_hf_config_of_the_hybrid_family_is_understood():
    d = {"architectures": ["Qwen3_5MoeForConditionalGeneration"],
         "text_config": {"hidden_size": 64, "num_hidden_layers": 8, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
                         "vocab_size": 100, "num_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 32,
                         "shared_expert_intermediate_size": 32, "full_attention_interval": 4, "linear_num_key_heads": 2,
                         "linear_num_value_heads": 4, "linear_key_head_dim": 16, "linear_value_head_dim": 16, "linear_conv_kernel_dim": 4,
                         "rope_parameters": {"rope_theta": 1e7, "partial_rotary_factor": 0.25}}}
    c = ModelConfig.from_dict(d)
    assert c.is_hybrid_gdn and not c.is_mla and c.n_routed_experts == 4 and c.rope_theta == 1e7 and c.partial_rotary_factor == 0.25
    assert [c.layer_type(i) for i in range(8)].count("full_attention") == 2 and c.layer_type(3) == "full_attention"
    assert c.norm_unit_offset and c.attn_output_gate and c.qk_norm


def test_hybrid_checkpoint_round_trip(tmp_path):
    """A checkpoint directory of the hybrid family (config.json + safetensors, with the non-`.weight` tensors A_log and dt_bias)
    loads into the same model as the tensors fed directly."""
    from nanoengine_b200.models.weights import random_hf_weights, save_hf_checkpoint
    mc = tiny_qwen3_5(moe=True)
    save_hf_checkpoint(str(tmp_path), mc, random_hf_weights(mc, seed=3))
    from_disk = _llm(None, model=str(tmp_path))
    direct = _llm(mc)
    direct.engine.executor.runner.load_weights(random_hf_weights(mc, seed=3))
    prompts = [list(range(5, 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    assert from_disk.generate(prompts, sp)[0]["token_ids"] == direct.generate(prompts, sp)[0]["token_ids"]
