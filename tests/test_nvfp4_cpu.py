"""NVFP4 (ModelOpt layout: packed e2m1, one e4m3 scale per 16 elements, one fp32 scale per matrix, one fp32 activation scale): the PyTorch
statements of the quantiser and the W4A4 expert path, the expert module, and a checkpoint round trip through the loader.
Parity: reference layers/backends/experts/nvfp4.py, kernel/cutedsl_nvfp4_moe.py, tests/test_nvfp4_deepep_recipe.py."""
import torch

from nanoengine_b200.models.config import ModelConfig, tiny_deepseek_v3
from nanoengine_b200.ops import reference as ref


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_quantiser_recipe():
    torch.manual_seed(0)
    x = torch.randn(7, 128) * 3
    g = torch.tensor([50.0])
    q, sf = ref.nvfp4_quant(x, g)
    assert q.dtype == torch.uint8 and q.shape == (7, 64) and sf.dtype == torch.float8_e4m3fn and sf.shape == (7, 8)
    xd = ref.nvfp4_unpack(q, sf) / 50.0
    assert _rel(xd, x) < 0.13
    # the scale is e4m3(g * amax / 6): the largest element of a block lands on +-6 (or 4 when the scale was rounded up)
    v = (x * 50.0).view(7, 8, 16) / sf.float().unsqueeze(-1)
    assert float(v.abs().amax(-1).max()) <= 6.6 and float(v.abs().amax(-1).min()) >= 5.0
    # per-group scales follow the row's group
    rg = torch.tensor([0, 0, 1, 1, 1, 2, 2])
    q2, sf2 = ref.nvfp4_quant(x, torch.tensor([50.0, 5.0, 50.0]), rg)
    assert torch.equal(q2[:2], q[:2]) and torch.equal(sf2[5:].view(torch.uint8), sf[5:].view(torch.uint8))
    assert not torch.equal(sf2[2:5].view(torch.uint8), sf[2:5].view(torch.uint8))
    # ties go to the even code, zero keeps no sign, the range saturates at 6
    assert ref._e2m1_codes(torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 9.0, -0.2, -6.5])).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 0, 15]


def test_weight_format_and_gemm():
    torch.manual_seed(1)
    w = torch.randn(3, 64, 256) * 0.05
    q, sf, s2 = ref.nvfp4_quant_weight(w)
    assert q.shape == (3, 64, 128) and sf.shape == (3, 64, 16) and s2.shape == (3,)
    wd = ref.nvfp4_unpack(q, sf) * s2.view(3, 1, 1)
    assert _rel(wd, w) < 0.13
    x = torch.randn(40, 256)
    aq, asf = ref.nvfp4_quant(x, torch.tensor([20.0]))
    counts, starts = torch.tensor([10, 0, 25]), torch.tensor([0, 10, 15])
    out = ref.nvfp4_gemm(aq, asf, q, sf, s2 / 20.0, counts, starts, out_fp32=True)
    xd = ref.nvfp4_unpack(aq, asf) / 20.0
    assert torch.allclose(out[:10], xd[:10] @ wd[0].t(), rtol=1e-4, atol=1e-5)
    assert torch.allclose(out[15:40], xd[15:40] @ wd[2].t(), rtol=1e-4, atol=1e-5)
    assert float(out[10:15].abs().max()) == 0.0


def test_expert_module_matches_its_dequantised_weights():
    from nanoengine_b200.models.layers import RoutedExperts
    torch.manual_seed(2)
    ex = RoutedExperts(4, 256, 256, torch.float32, "cpu", "nvfp4")
    ex.init_random(torch.Generator().manual_seed(1), std=0.05)
    x = torch.randn(24, 256)
    idx, w = ref.moe_route(torch.randn(24, 4), None, 2, 1, 1, True, 1.0, "softmax")
    y = ex(x, idx, w)
    W13 = ref.nvfp4_unpack(ex.gate_up_proj, ex.gate_up_scale) * ex.gate_up_scale_2[:, 0].view(-1, 1, 1)
    W2 = ref.nvfp4_unpack(ex.down_proj, ex.down_scale) * ex.down_scale_2.view(-1, 1, 1)
    assert _rel(y, ref.moe_experts(x, idx, w, W13, W2)) < 0.3          # activations go through 4 bits twice
    # gate and up halves were quantised apart: after preparation they share one per-matrix scale
    assert torch.equal(ex.gate_up_scale_2[:, 0], ex.gate_up_scale_2[:, 1])


def test_modelopt_checkpoint_round_trip(tmp_path):
    from nanoengine_b200 import Config, LLM, RequestIn, SamplingParams
    from nanoengine_b200.models.weights import random_hf_weights, save_hf_checkpoint
    mc = tiny_deepseek_v3(moe_intermediate_size=256, intermediate_size=512)
    W = dict(random_hf_weights(mc, seed=3))
    save_hf_checkpoint(str(tmp_path), mc, W.items(), quantize_nvfp4=True)
    assert ModelConfig.from_pretrained(str(tmp_path)).quant == "nvfp4"
    llm = LLM(Config(model=str(tmp_path), device="cpu", dtype="float32", max_num_seqs=2, max_num_batched_tokens=64, num_kvcache_blocks=16,
                     kvcache_block_size=16, enable_prefix_caching=False))
    model = llm.engine.executor.runner.model
    ex = model.model.layers["1"].mlp.experts
    assert ex.quant == "nvfp4" and ex.gate_up_proj.dtype == torch.uint8
    # the routed experts hold the checkpoint's bytes; the dense MLP and the shared expert were expanded to the activation dtype
    q, sf, s2 = ref.nvfp4_quant_weight(W["model.layers.1.mlp.experts.3.down_proj.weight"].float())
    assert torch.equal(ex.down_proj[3], q) and torch.equal(ex.down_scale[3].view(torch.uint8), sf.view(torch.uint8))
    assert float(ex.down_scale_2[3]) == float(s2)
    dense = model.model.layers["0"].mlp.down_proj.weight
    want = W["model.layers.0.mlp.down_proj.weight"]
    assert dense.dtype == torch.float32 and _rel(dense[: want.shape[0]], want) < 0.13
    llm.add_request_payload(RequestIn(1, [5, 6, 7, 8], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)).to_bytes())
    assert len([o["token_ids"] for o in llm.generate()][0]) == 3


def test_config_refuses_shapes_the_nvfp4_kernels_do_not_take():
    import pytest
    from nanoengine_b200 import Config
    ok = tiny_deepseek_v3(moe_intermediate_size=256, intermediate_size=512, quant="nvfp4")
    Config(model_config=ok, dummy_weight=True, device="cpu", dtype="float32")
    with pytest.raises(ValueError, match="multiples of 256"):
        Config(model_config=tiny_deepseek_v3(quant="nvfp4"), dummy_weight=True, device="cpu", dtype="float32")        # moe_intermediate_size 128
    with pytest.raises(ValueError, match="routed experts"):
        Config(model_config=tiny_deepseek_v3(quant="nvfp4", n_routed_experts=0, moe_intermediate_size=256), dummy_weight=True, device="cpu", dtype="float32")
