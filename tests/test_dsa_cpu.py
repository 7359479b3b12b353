"""DSA (lightning indexer + sparse MLA) on the CPU engine: with top-k >= context the model is exactly dense; with a small
top-k the sparse attention output equals dense attention restricted to the selected keys; indexer cache layout round-trips."""
import torch

from nanoengine_b200 import Config, LLM, SamplingParams
from nanoengine_b200.ops import reference as ref


def _llm(index_topk, **kw):
    over = dict(index_n_heads=4, index_head_dim=32, index_topk=index_topk, architecture="DeepseekV32ForCausalLM")
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64,
                hf_overrides=over)
    base.update(kw)
    return LLM(Config(**base))


def _prompts():
    g = torch.Generator().manual_seed(11)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 25)]


def test_large_topk_equals_dense_model():
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    dense = LLM(Config(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64))
    want = [o["token_ids"] for o in dense.generate(_prompts(), sp)]
    got = [o["token_ids"] for o in _llm(4096).generate(_prompts(), sp)]
    assert got == want       # the indexer's own weights draw from separate generators, so the shared weights are identical


def test_small_topk_runs_sparse_and_differs_only_through_selection():
    llm = _llm(8)
    runner = llm.engine.executor.runner
    seen = {}
    orig = ref.mla_attention_paged

    def spy(q, cache, bt, cu, cl, scale, R, sparse_indices=None):
        out = orig(q, cache, bt, cu, cl, scale, R, sparse_indices)
        if sparse_indices is not None:
            seen["sparse"] = sparse_indices.clone()
            # dense attention over exactly the selected slots must give the same result
            T = q.shape[0]
            flat = cache.view(-1, cache.shape[-1])
            for t in range(min(T, 4)):
                idx = sparse_indices[t][sparse_indices[t] >= 0].long()
                kv = flat[idx].float()
                p = torch.softmax(torch.einsum("hd,nd->hn", q[t].float(), kv) * scale, -1)
                assert torch.allclose(out[t].float(), p @ kv[:, :R], atol=1e-5)
        return out

    ref.mla_attention_paged = spy
    try:
        outs = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    finally:
        ref.mla_attention_paged = orig
    assert len(outs) == 2 and "sparse" in seen
    sp = seen["sparse"]
    assert sp.shape[1] == 8 and (sp >= -1).all()
    for row in sp:
        vals = row[row >= 0]
        assert vals.numel() == vals.unique().numel()      # no key is selected twice


def test_indexer_scoring_formula_and_topk_translation():
    torch.manual_seed(0)
    q = torch.randn(3, 4, 32); k = torch.randn(50, 32); w = torch.rand(3, 4)
    q8, qs = ref.quant_fp8_per_token_pow2(q.reshape(12, 32)); q8, qs = q8.view(3, 4, 32), qs.view(3, 4)
    k8, ks = ref.quant_fp8_per_token_pow2(k)
    got = ref.indexer_logits(q8, qs, w, k8, ks)
    qd, kd = q8.float() * qs.unsqueeze(-1), k8.float() * ks.unsqueeze(-1)
    want = (torch.relu(torch.einsum("thd,nd->thn", qd, kd)) * w.unsqueeze(-1)).sum(1)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)
    assert torch.all(torch.log2(ks) == torch.log2(ks).round())          # power-of-two scales
    idx = ref.indexer_topk(got, torch.tensor([10, 50, 3]), 8)
    assert (idx[0] < 10).all() and (idx[2][idx[2] >= 0] < 3).all() and (idx[2] == -1).sum() == 5
    bt = torch.tensor([[7, 2, 9, 4]]).expand(3, -1)
    phys = ref.logical_to_physical(idx, bt, 16)
    i = idx[1, 0].item()
    assert phys[1, 0].item() == bt[1, i // 16].item() * 16 + i % 16 and (phys[idx < 0] == -1).all()
    h = ref.hadamard(torch.eye(8))
    assert torch.allclose(h @ h.t(), torch.eye(8), atol=1e-6)           # orthonormal


def test_host_swap_moves_indexer_pages_with_the_kv_pages():
    """A preempted DSA sequence comes back from the host tier with its indexer keys, not only its latent KV rows."""
    import torch
    from nanoengine_b200.models.config import tiny_deepseek_v3
    from nanoengine_b200.runtime.cache import KVCache, make_cache_plan
    mc = tiny_deepseek_v3(index_topk=8, index_n_heads=4, index_head_dim=128)
    plan = make_cache_plan(mc, "bfloat16", 16)
    assert plan.indexer
    c = KVCache(plan, 10, "cpu")
    c.allocate_host(4)
    assert sorted(c.host_families) == ["indexer", "mla_kv"]
    g = torch.Generator().manual_seed(0)
    c.kv.copy_(torch.randn(c.kv.shape, generator=g).to(c.kv.dtype))
    c.indexer.copy_(torch.randint(0, 255, c.indexer.shape, generator=g, dtype=torch.uint8))
    want = [v.clone() for b in (2, 5) for v in c.block_views(b)]
    c.swap([2, 5], [1, 3], to_host=True)
    for b in (2, 5):
        for v in c.block_views(b):
            v.zero_()
    c.swap([1, 3], [7, 8], to_host=False)
    got = [v for b in (7, 8) for v in c.block_views(b)]
    assert len(got) == 4 and all(torch.equal(a, b) for a, b in zip(got, want))
