"""Vision side on CPU: the vision transformer against a plain PyTorch restatement of the same network (Conv3d patch embedding,
per-image scaled-dot-product attention), the embedding pool, the encoder engine over its ZMQ service, and a language model
that consumes image embeddings in place of its image tokens (also with the prompt prefetched in chunks)."""
import torch
import torch.nn.functional as F

from nanoengine_b200 import Config, LLM, SamplingParams
from nanoengine_b200.vl import EmbeddingPool, EncoderConfig, EncoderEngine, VisionConfig, VisionModel
from nanoengine_b200.vl.encoder_engine import EncoderClient
from nanoengine_b200.vl.vision import random_vision_weights

VC = VisionConfig(hidden_size=64, num_heads=4, depth=2, intermediate_size=96, out_hidden_size=48, in_channels=3, patch_size=4,
                  temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=64)


def _dense_vit(W, c, patches, grids):
    """The same network written the long way (reference vl/vision/encoder.py), fp32."""
    H, nh = c.hidden_size, c.num_heads
    hd = H // nh
    x = F.conv3d(patches.view(-1, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size), W["visual.patch_embed.proj.weight"],
                 W["visual.patch_embed.proj.bias"], stride=(c.temporal_patch_size, c.patch_size, c.patch_size)).view(-1, H)
    S, m = int(c.num_position_embeddings ** 0.5), c.spatial_merge_size
    pos, coords = [], []
    for t, h, w in grids:
        table = W["visual.pos_embed.weight"].view(S, S, H).permute(2, 0, 1)[None]
        e = F.interpolate(table, size=(h, w), mode="bilinear", align_corners=True)[0].permute(1, 2, 0)        # [h, w, H]
        e = e.view(h // m, m, w // m, m, H).permute(0, 2, 1, 3, 4).reshape(h * w, H)
        pos.append(e.repeat(t, 1))
        rr = torch.arange(h).view(h // m, m)[:, None, :, None].expand(h // m, w // m, m, m).reshape(-1)
        cc = torch.arange(w).view(w // m, m)[None, :, None, :].expand(h // m, w // m, m, m).reshape(-1)
        coords.append(torch.stack([rr, cc], -1).repeat(t, 1))
    x = x + torch.cat(pos)
    coords = torch.cat(coords).float()
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2).float() / (hd // 2)))
    ang = torch.cat([coords[:, :1] * inv, coords[:, 1:] * inv], -1)
    emb = torch.cat([ang, ang], -1)
    cos, sin = emb.cos()[:, None], emb.sin()[:, None]
    rot = lambda v: torch.cat([-v[..., hd // 2:], v[..., : hd // 2]], -1)
    lens = [h * w for t, h, w in grids for _ in range(t)]
    for i in range(c.depth):
        p = f"visual.blocks.{i}."
        y = F.layer_norm(x, (H,), W[p + "norm1.weight"], W[p + "norm1.bias"], 1e-6)
        qkv = F.linear(y, W[p + "attn.qkv.weight"], W[p + "attn.qkv.bias"]).view(-1, 3, nh, hd)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
        outs, lo = [], 0
        for n in lens:
            o = F.scaled_dot_product_attention(q[lo:lo + n].transpose(0, 1)[None], k[lo:lo + n].transpose(0, 1)[None], v[lo:lo + n].transpose(0, 1)[None])
            outs.append(o[0].transpose(0, 1)); lo += n
        x = x + F.linear(torch.cat(outs).reshape(-1, H), W[p + "attn.proj.weight"], W[p + "attn.proj.bias"])
        y = F.layer_norm(x, (H,), W[p + "norm2.weight"], W[p + "norm2.bias"], 1e-6)
        x = x + F.linear(F.gelu(F.linear(y, W[p + "mlp.linear_fc1.weight"], W[p + "mlp.linear_fc1.bias"]), approximate="tanh"),
                         W[p + "mlp.linear_fc2.weight"], W[p + "mlp.linear_fc2.bias"])
    y = F.layer_norm(x, (H,), W["visual.merger.norm.weight"], W["visual.merger.norm.bias"], 1e-6).view(-1, H * m * m)
    return F.linear(F.gelu(F.linear(y, W["visual.merger.linear_fc1.weight"], W["visual.merger.linear_fc1.bias"])),
                    W["visual.merger.linear_fc2.weight"], W["visual.merger.linear_fc2.bias"])


def test_vision_model_matches_the_dense_network():
    W = dict(random_vision_weights(VC, seed=1))
    model = VisionModel(VC, torch.float32, "cpu")
    assert model.load_weights(W.items()) == len(W)
    grids = [(1, 4, 6), (2, 2, 4), (1, 8, 8)]                        # an image, a two-frame clip, a larger image
    T = sum(t * h * w for t, h, w in grids)
    patches = torch.randn(T, VC.patch_dim)
    got = model(patches, grids)
    want = _dense_vit(W, VC, patches, grids)
    assert got.shape == (T // 4, VC.out_hidden_size)
    assert (got - want).abs().max() < 2e-4


def test_embedding_pool_slots():
    pool = EmbeddingPool(3, 16, 8, "cpu", torch.float32)
    a, b = pool.allocate(5), pool.allocate(16)
    pool.write(a, torch.ones(5, 8)); pool.write(b, torch.full((16, 8), 2.0))
    assert pool.read(a).shape == (5, 8) and pool.read(b).sum() == 256 and pool.available_slots == 1
    assert pool.slot_byte_offset(b) == b * 16 * 8 * 4
    assert pool.free([a, a, 7]) == 1 and pool.available_slots == 2
    try:
        pool.allocate(17)
        assert False
    except RuntimeError:
        pass
    desc = pool.export(direct=True)
    from nanoengine_b200.vl.embedding_pool import EmbeddingReader
    assert torch.equal(EmbeddingReader(desc, "cpu").fetch(b, 16, torch.float32), pool.read(b))


def test_encoder_engine_direct_and_over_zmq(tmp_path):
    ep = f"ipc://{tmp_path}/enc.sock"
    eng = EncoderEngine(EncoderConfig(vision_config=VC, device="cpu", dtype="float32", num_slots=4, max_tokens_per_slot=64, endpoint=ep,
                                      max_patches_per_batch=40))
    try:
        grids = [(1, 4, 6), (1, 4, 4), (1, 2, 2)]
        patches = torch.randn(sum(t * h * w for t, h, w in grids), VC.patch_dim)
        direct = eng.encode(patches, grids)                                      # three images in groups of <= 40 patches
        assert direct.num_tokens == 11 and direct.hidden_size == 48 and direct.grid_thw == [list(g) for g in grids]
        whole = eng.model(patches, grids)
        assert (eng.pool.read(direct.slot) - whole).abs().max() < 1e-5           # grouping does not change the rows
        cli = EncoderClient(ep)
        remote = cli.encode(patches, grids)
        assert remote.slot != direct.slot and remote.num_tokens == 11
        assert torch.equal(eng.pool.read(remote.slot), eng.pool.read(direct.slot))
        assert cli.info()["available_slots"] == 2 and cli.free([remote.slot, direct.slot]) == 2 and eng.pool.available_slots == 4
        try:
            cli.encode(patches[:5], grids)                                        # a bad request is an error reply, not a dead service
            assert False
        except RuntimeError as e:
            assert "patches" in str(e)
        assert cli.info()["kind"] == "vision_encoder"
        cli.close()
    finally:
        eng.shutdown()


def test_language_model_consumes_image_embeddings():
    """Image rows replace the embeddings of the image tokens: the result equals a model whose embedding table holds those rows at
    fresh token ids, for a whole-prompt prefill and for 16-token chunks."""
    from nanoengine_b200.models.config import tiny_deepseek_v3
    mc = tiny_deepseek_v3()
    IMG = 7
    emb = torch.randn(6, mc.hidden_size) * 0.02
    prompt = [3, 11, IMG, IMG, IMG, 25, 99, IMG, IMG, IMG, 14] + list(range(30, 60))
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)

    def run(**kw):
        llm = LLM(Config(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=16,
                         num_kvcache_blocks=32, max_num_seqs=4, enable_prefix_caching=False, **kw))
        return llm

    a = run()
    # oracle: spare vocabulary rows 1000.. take the image rows, the prompt names them instead of the image token
    table = a.engine.executor.runner.model.model.embed_tokens.weight
    table[1000:1006] = emb
    it = iter(range(1000, 1006))
    want = a.generate([[next(it) if t == IMG else t for t in prompt]], sp)[0]["token_ids"]
    for kw in ({}, dict(max_num_batched_tokens=16, enable_chunked_prefill=True)):
        b = run(**kw)
        b.engine.add_vision_request(prompt, IMG, embeddings=emb, sampling_params=sp)
        assert b.generate()[0]["token_ids"] == want
        assert not b.engine.executor.runner.__dict__["_vision"]                  # released once the prompt is in
    # through an encoder's pool
    pool = EmbeddingPool(2, 8, mc.hidden_size, "cpu", torch.float32)
    s = pool.allocate(6); pool.write(s, emb)
    from nanoengine_b200.vl.encoder_engine import VisionSlot
    c = run()
    c.engine.add_vision_request(prompt, IMG, vision_slot=VisionSlot("e", s, 6, mc.hidden_size, []), pool_desc=pool.export(direct=True), sampling_params=sp)
    assert c.generate()[0]["token_ids"] == want
    try:
        c.engine.add_vision_request(prompt[:5], IMG, embeddings=emb, sampling_params=sp)          # 3 image tokens, 6 rows
        assert False
    except Exception as e:
        assert "image tokens" in str(e)


def test_encoder_http_front():
    import base64
    from fastapi.testclient import TestClient
    from nanoengine_b200.server.vl_server import build_app
    eng = EncoderEngine(EncoderConfig(vision_config=VC, device="cpu", dtype="float32", num_slots=2, max_tokens_per_slot=32))
    cli = TestClient(build_app(eng))
    assert cli.get("/health").json()["available_slots"] == 2
    patches = torch.randn(16, VC.patch_dim)
    r = cli.post("/encode", json={"patches": base64.b64encode(patches.numpy().tobytes()).decode(), "grid_thw": [[1, 4, 4]], "dtype": "float32"})
    assert r.status_code == 200 and r.json()["num_tokens"] == 4
    assert cli.post("/encode", json={"patches": "", "grid_thw": [[1, 4, 4]]}).status_code == 400
    assert cli.post("/free", json={"slots": [r.json()["slot"]]}).json()["freed"] == 1
    assert cli.get("/info").json()["kind"] == "vision_encoder"
