"""The "ue8m0" scale format (power-of-two fp8 block scales; reference models/quant_config.py:39-44 and the ROUND_UE8M0 switches of
its quantisers): configuration plumbing and the PyTorch statements of the quantisers."""
import pytest
import torch

from nanoengine_b200.config import Config
from nanoengine_b200.models.config import ModelConfig, tiny_deepseek_v3
from nanoengine_b200.ops import reference as ref


@pytest.fixture()
def ue8m0():
    ref.set_scale_format("ue8m0")
    try:
        yield
    finally:
        ref.set_scale_format(None)


def _is_pow2(s):
    return bool(((s.float().contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())


def test_scale_fmt_round_trips_through_the_hf_config():
    mc = tiny_deepseek_v3(quant="fp8")
    d = mc.to_dict()
    assert "scale_fmt" not in d.get("quantization_config", {})
    d["quantization_config"]["scale_fmt"] = "ue8m0"
    mc2 = ModelConfig.from_dict(d)
    assert mc2.scale_fmt == "ue8m0" and mc2.to_dict()["quantization_config"]["scale_fmt"] == "ue8m0"
    assert Config(model_config=mc2, dummy_weight=True, device="cpu").resolved_scale_format() == "ue8m0"
    assert Config(model_config=mc, dummy_weight=True, device="cpu").resolved_scale_format() == "fp32"
    assert Config(model_config=mc, dummy_weight=True, device="cpu", fp8_scale_format="ue8m0").resolved_scale_format() == "ue8m0"
    with pytest.raises(ValueError):
        Config(model_config=mc, dummy_weight=True, device="cpu", fp8_scale_format="e8")


def test_quantisers_round_scales_up(ue8m0):
    torch.manual_seed(0)
    x = torch.randn(9, 512) * 5
    q, s = ref.quant_fp8_1x128(x)
    _, s0 = ref.quant_fp8_1x128(x, ue8m0=False)
    assert _is_pow2(s) and bool((s >= s0).all()) and bool((s < 2 * s0).all())
    assert (ref.dequant_fp8_1x128(q, s) - x).abs().max() < 0.07 * x.abs().max()
    w = torch.randn(200, 384) * 0.05
    wq, ws = ref.quant_fp8_block(w)
    assert _is_pow2(ws) and ws.shape == (2, 3)
    assert ((ref.dequant_fp8_block(wq, ws) - w).norm() / w.norm()).item() < 0.05
    # exact powers of two stay where they are
    assert torch.equal(ref._ceil_pow2(torch.tensor([0.5, 1.0, 1.0001, 3.0])), torch.tensor([0.5, 1.0, 2.0, 4.0]))


def test_checkpoint_scales_follow_the_format(ue8m0):
    torch.manual_seed(1)
    w = torch.randn(256, 256) * 0.05
    wq, ws = ref.quant_fp8_block(w, ue8m0=False)
    q2, s2 = ref.fp8_block_for_format(wq, ws)
    assert _is_pow2(s2) and not _is_pow2(ws)
    assert ((ref.dequant_fp8_block(q2, s2) - ref.dequant_fp8_block(wq, ws)).norm() / w.norm()).item() < 0.05
    ref.set_scale_format("fp32")
    q3, s3 = ref.fp8_block_for_format(wq, ws)
    assert q3 is wq and s3 is ws


def test_engine_follows_the_configured_format():
    from nanoengine_b200 import LLM, RequestIn, SamplingParams
    mc = tiny_deepseek_v3(quant="fp8")
    outs = {}
    try:
        for fmt in ("fp32", "ue8m0"):
            llm = LLM(Config(model_config=mc, dummy_weight=True, device="cpu", dtype="float32", fp8_scale_format=fmt, max_num_seqs=2,
                             max_num_batched_tokens=64, num_kvcache_blocks=16, kvcache_block_size=16, enable_prefix_caching=False))
            assert ref.scale_format() == fmt
            lin = next(m for m in llm.engine.executor.runner.model.modules() if getattr(m, "weight_scale_inv", None) is not None)
            assert _is_pow2(lin.weight_scale_inv) == (fmt == "ue8m0")
            llm.add_request_payload(RequestIn(1, [1, 2, 3, 4, 5], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)).to_bytes())
            outs[fmt] = [o["token_ids"] for o in llm.generate()][0]
            assert len(outs[fmt]) == 4
    finally:
        ref.set_scale_format(None)


def test_fp8_checkpoint_with_plain_scales_loads_under_ue8m0(tmp_path):
    """A checkpoint quantised with plain amax / 448 scales, served with fp8_scale_format="ue8m0": every block scale is re-quantised to
    a power of two at load (experts, merged projections and single linears alike) and the first-token logits stay close to the
    engine that keeps the checkpoint's own scales."""
    from nanoengine_b200 import LLM
    from nanoengine_b200.models.weights import random_hf_weights, save_hf_checkpoint
    mc = tiny_deepseek_v3(quant="fp8")
    save_hf_checkpoint(str(tmp_path), mc, random_hf_weights(mc, seed=5), quantize_fp8=True)
    logits = {}
    try:
        for fmt in ("fp32", "ue8m0"):
            llm = LLM(Config(model=str(tmp_path), device="cpu", dtype="float32", fp8_scale_format=fmt, max_num_seqs=2, max_num_batched_tokens=64,
                             num_kvcache_blocks=16, kvcache_block_size=16, enable_prefix_caching=False))
            model = llm.engine.executor.runner.model
            scales = [m.weight_scale_inv for m in model.modules() if getattr(m, "weight_scale_inv", None) is not None]
            scales += [s for m in model.modules() for s in (getattr(m, "gate_up_scale", None), getattr(m, "down_scale", None)) if s is not None]
            assert len(scales) > 6
            assert all(_is_pow2(s) for s in scales) == (fmt == "ue8m0")
            got = {}
            orig = model.compute_logits
            model.compute_logits = lambda h, _o=orig, _g=got: _g.setdefault("l", _o(h))
            from nanoengine_b200 import RequestIn, SamplingParams
            llm.add_request_payload(RequestIn(1, list(range(3, 40)), SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)).to_bytes())
            llm.generate()
            logits[fmt] = got["l"].float()
    finally:
        ref.set_scale_format(None)
    rel = ((logits["ue8m0"] - logits["fp32"]).norm() / logits["fp32"].norm()).item()
    assert rel < 0.1, rel
