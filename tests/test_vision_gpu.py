"""Vision encoder on the GPU: the bf16 CUDA network (tcgen05 GEMMs, LayerNorm / GELU / rotary kernels, non-causal ragged
attention on the generic kernel) against the fp32 CPU model on the same weights, and a slot read through the pool."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_ragged_noncausal_attention_kernel():
    from nanoengine_b200.ops import reference as ref, sm100
    sm100.clear_kernel_status()
    torch.manual_seed(0)
    for H, D in ((16, 72), (4, 32), (3, 128)):
        lens = [70, 1, 33, 129]
        T = sum(lens)
        q, k, v = (torch.randn(T, H, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
        for causal in (False, True):
            want = ref.attention_varlen(q.float(), k.float(), v.float(), cu, D ** -0.5, causal)
            got = sm100.attention_varlen(q, k, v, cu, D ** -0.5, causal)
            assert _rel(got, want) < 1e-2, (H, D, causal)
    x = torch.randn(1000, 37, device="cuda", dtype=torch.bfloat16)
    assert _rel(sm100.gelu(x, True), ref.gelu(x, True)) < 5e-3 and _rel(sm100.gelu(x, False), ref.gelu(x, False)) < 5e-3
    assert sm100.kernel_status()[0] == 0


def test_vision_model_bf16_matches_fp32_cpu_and_pool_read():
    from nanoengine_b200.vl import EncoderConfig, EncoderEngine, VisionConfig, VisionModel
    from nanoengine_b200.vl.embedding_pool import EmbeddingReader
    from nanoengine_b200.vl.vision import random_vision_weights
    vc = VisionConfig(hidden_size=288, num_heads=4, depth=3, intermediate_size=512, out_hidden_size=256, in_channels=3, patch_size=4,
                      temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=256)          # head dim 72, as the full-size model
    W = [(n, t.to(torch.bfloat16).float()) for n, t in random_vision_weights(vc, seed=2)]
    cpu = VisionModel(vc, torch.float32, "cpu"); cpu.load_weights(W)
    gpu = VisionModel(vc, torch.bfloat16, "cuda"); gpu.load_weights(W)
    grids = [(1, 8, 12), (2, 4, 4), (1, 16, 16)]
    patches = torch.randn(sum(t * h * w for t, h, w in grids), vc.patch_dim).to(torch.bfloat16)
    want = cpu(patches.float(), grids)
    got = gpu(patches, grids)
    assert got.shape == want.shape and _rel(got.cpu(), want) < 3e-2
    eng = EncoderEngine(EncoderConfig(vision_config=vc, device="cuda", num_slots=2, max_tokens_per_slot=512))
    slot = eng.encode(patches, grids)
    rows = EmbeddingReader(eng.engine_info(direct=True)["pool"], "cuda").fetch(slot.slot, slot.num_tokens, torch.bfloat16)
    assert rows.shape == (slot.num_tokens, 256) and torch.equal(rows, eng.pool.read(slot.slot))
