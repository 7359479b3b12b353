"""The file-backed third KV tier: block files, index recovery, eviction, and the engine path that brings a prompt's
blocks back from files after the device prefix cache lost them."""
import os

import pytest
import torch

from nanoengine_b200 import Config, LLM, SamplingParams
from nanoengine_b200.runtime.cache import KVCache, make_cache_plan
from nanoengine_b200.runtime.l3_store import L3Store, prompt_block_hashes
from nanoengine_b200.models.config import tiny_deepseek_v3


def _cache(num_blocks=8, kv="bfloat16"):
    plan = make_cache_plan(tiny_deepseek_v3(), kv, 16)
    c = KVCache(plan, num_blocks, "cpu")
    g = torch.Generator().manual_seed(0)
    flat = c.kv.view(torch.uint8) if c.kv.dtype == torch.float8_e4m3fn else c.kv
    flat.copy_(torch.randn(flat.shape, generator=g).to(flat.dtype) if flat.dtype != torch.uint8
               else torch.randint(0, 255, flat.shape, generator=g, dtype=torch.uint8))
    return c


@pytest.mark.parametrize("kv", ["bfloat16", "fp8"])
def test_store_load_roundtrip_and_recovery(tmp_path, kv):
    c = _cache(kv=kv)
    st = L3Store(c, str(tmp_path))
    want3 = [v.clone() for v in c.block_views(3)]
    assert st.store([(0xABCDEF, 3), (0x12345, 5)]) == [0xABCDEF, 0x12345]
    assert st.exists([1, 0xABCDEF, 0x12345]) == [0xABCDEF, 0x12345] and st.match([0xABCDEF, 7, 0x12345]) == 1
    assert os.path.exists(os.path.join(str(tmp_path), "rank0", f"{0xABCDEF:016x}.kv"))
    for v in c.block_views(6):
        v.zero_()
    assert st.load([(0xABCDEF, 6)]) == 1
    for a, b in zip(c.block_views(6), want3):
        assert torch.equal(a, b)
    # a new store object over the same directory finds the files again
    st2 = L3Store(c, str(tmp_path))
    assert len(st2) == 2 and st2.exists([0x12345]) == [0x12345]
    # a missing file is an error, and the index forgets it
    os.unlink(os.path.join(str(tmp_path), "rank0", f"{0x12345:016x}.kv"))
    with pytest.raises(FileNotFoundError):
        st2.load([(0x12345, 1)])
    assert st2.exists([0x12345]) == []
    s = st.stats()
    assert s["n_store"] == 2 and s["n_load"] == 1 and s["GiB_stored"] > 0


def test_capacity_evicts_least_recent_and_deletes_its_file(tmp_path):
    c = _cache()
    st = L3Store(c, str(tmp_path), capacity_blocks=2)
    st.store([(11, 0), (12, 1)])
    st.load([(11, 2)])                 # 11 is now the most recent
    st.store([(13, 3)])                # evicts 12
    assert st.exists([11, 12, 13]) == [11, 13] and st.n_evicted == 1
    assert not os.path.exists(os.path.join(str(tmp_path), "rank0", f"{12:016x}.kv"))


def test_foreign_layout_is_rejected(tmp_path):
    a = L3Store(_cache(kv="bfloat16"), str(tmp_path))
    a.store([(99, 1)])
    b = L3Store(_cache(kv="fp8"), str(tmp_path))       # other layout: the file is not adopted
    assert len(b) == 0


def _llm(tmp_path, **kw):
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=4,
                num_kvcache_blocks=24, seed=0, l3_dir=str(tmp_path), enable_prefix_caching=True)
    base.update(kw)
    return LLM(Config(**base))


def test_engine_reloads_prefix_blocks_from_files(tmp_path):
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 1024, (70,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a = _llm(tmp_path)
    want = a.generate([prompt], sp)[0]["token_ids"]
    hashes = prompt_block_hashes(prompt, 16)
    assert len(hashes) == 4
    store = a.engine.executor.runner.l3
    assert store.exists(hashes) == hashes                         # the prompt's full blocks were persisted as they were published
    # a second engine over the same directory starts with an empty device cache and still skips the prefix
    b = _llm(tmp_path)
    assert b.engine.scheduler.num_cached_blocks(0) == 0
    got = b.generate([prompt], sp)[0]["token_ids"]
    assert got == want
    assert b.engine.executor.runner.l3.n_load == 4
    m = b.engine.scheduler.metrics_summary()
    assert m["prefix_hit_tokens"] >= 64 if "prefix_hit_tokens" in m else True
    # wipe the device prefix cache of the first engine: the same prompt comes back from files, not from recompute
    a.engine.scheduler.reset_prefix_cache()
    n0 = store.n_load
    assert a.generate([prompt], sp)[0]["token_ids"] == want
    assert store.n_load == n0 + 4


def test_engine_survives_a_vanished_block_file(tmp_path):
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 1024, (50,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    a = _llm(tmp_path)
    want = a.generate([prompt], sp)[0]["token_ids"]
    hashes = prompt_block_hashes(prompt, 16)
    os.unlink(os.path.join(str(tmp_path), "rank0", f"{hashes[1]:016x}.kv"))
    a.engine.scheduler.reset_prefix_cache()
    free_before = a.engine.scheduler.num_free_blocks(0)
    assert a.generate([prompt], sp)[0]["token_ids"] == want        # falls back to recomputing
    assert a.engine.scheduler.num_free_blocks(0) == free_before    # and the reserved blocks were returned


def test_blocks_of_other_weights_are_not_adopted(tmp_path):
    """Same cache layout, other model tag (another checkpoint of the same shape) or an older weight generation: the files stay
    on disk unread; after a generation bump the old files are gone and the directory remembers the generation."""
    c = _cache()
    a = L3Store(c, str(tmp_path), tag="model-A")
    a.store([(7, 1), (8, 2)])
    assert len(L3Store(c, str(tmp_path), tag="model-A")) == 2
    assert len(L3Store(c, str(tmp_path), tag="model-B")) == 0
    assert a.bump_generation() == 1 and len(a) == 0
    assert not [n for n in os.listdir(os.path.join(str(tmp_path), "rank0")) if n.endswith(".kv")]
    a.store([(9, 3)])
    again = L3Store(c, str(tmp_path), tag="model-A")               # a restart cannot have the updated weights: it starts clean
    assert again.generation == 0 and len(again) == 0


def test_live_weight_update_drops_the_file_tier(tmp_path):
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, 1024, (70,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    a = _llm(tmp_path)
    a.generate([prompt], sp)
    store = a.engine.executor.runner.l3
    assert len(store) == 4
    # new weights: scale one norm weight so the KV of the same prompt changes
    name, w = next((n, p) for n, p in a.engine.executor.runner.model.named_parameters() if n.endswith("layers.0.input_layernorm.weight"))
    a.update_weights([("model." + name.split("model.", 1)[1] if not name.startswith("model.") else name, w.detach() * 1.5)])
    assert len(store) == 0 and store.generation == 1
    want = a.generate([prompt], sp)[0]["token_ids"]
    assert store.n_load == 0                                         # nothing stale was imported
    b = _llm(tmp_path)
    assert len(b.engine.executor.runner.l3) == 0                     # a fresh engine has the checkpoint's weights, not the updated ones
    assert want is not None
