"""Hot / cold tier of the sparse-attention cache on CPU: the staging operator against its invariants, and a DSA decode engine
with the tier (prompts migrated from a prefill engine) against the same model on a plain hybrid engine."""
import pytest
import torch

from nanoengine_b200 import Config, LLM, RequestMigrate, SamplingParams
from nanoengine_b200.models.config import tiny_deepseek_v3
from nanoengine_b200.ops import reference as ref
from nanoengine_b200.parallel.kv_transfer import KVMigrator, LocalTransport
from nanoengine_b200.runtime.hisparse import HiSparseTier


def _tier(hot_rows=64, max_ctx=256, pages=8, page_rows=16, row=8):
    cold = [torch.arange(pages * page_rows * row, dtype=torch.float32).remainder(251).to(torch.uint8).view(pages, page_rows, row)]
    return HiSparseTier(1, 2, hot_rows, max_ctx, row, cold, "cpu"), cold[0]


def test_stage_loads_misses_keeps_hits_and_evicts_idle_rows():
    tier, cold = _tier()
    L = tier.layer(0)
    bt = torch.tensor([[3, 1, 4, 0, 5, 2, 6, 7]], dtype=torch.int32)                 # logical page -> cold page
    rows = cold.view(-1, 8)

    def cold_row(p):
        return rows[int(bt[0, p // 16]) * 16 + p % 16]

    slots, topk = torch.tensor([1]), 40
    sel = torch.full((1, topk), -1, dtype=torch.int32)
    sel[0, :30] = torch.arange(0, 60, 2, dtype=torch.int32)                          # 30 even positions
    ids, new = ref.hisparse_stage(L, sel, slots, torch.tensor([100]), bt)             # the new token sits at position 99
    assert (ids[0, 30:] == -1).all() and (ids[0, :30] >= 64).all() and (ids[0, :30] < 128).all() and len(set(ids[0, :30].tolist())) == 30
    for i in range(30):
        assert torch.equal(tier.hot[0, int(ids[0, i])], cold_row(int(sel[0, i])))
    assert int(tier.pos_to_hot[0, 1, 99]) == int(new[0]) - 64
    first = ids.clone()
    # the same list again: all hits, nothing moves
    ids2, _ = ref.hisparse_stage(L, sel, slots, torch.tensor([101]), bt)
    assert torch.equal(ids2[0, :30], first[0, :30])
    # 40 other positions with only 64 hot rows: rows of this step's list are never evicted, older ones are
    sel3 = torch.arange(1, 81, 2, dtype=torch.int32).view(1, 40)
    ids3, _ = ref.hisparse_stage(L, sel3, slots, torch.tensor([102]), bt)
    assert len(set(ids3[0].tolist())) == 40 and (ids3 >= 64).all()
    for i in range(40):
        assert torch.equal(tier.hot[0, int(ids3[0, i])], cold_row(int(sel3[0, i])))
    resident = {int(p) for p in tier.hot_to_pos[0, 1].tolist() if p >= 0}
    assert set(sel3[0].tolist()) <= resident and len(resident) <= 64
    for p in resident:                                                                # the two tables stay inverse to each other
        assert int(tier.hot_to_pos[0, 1, int(tier.pos_to_hot[0, 1, p])]) == p
    assert (tier.pos_to_hot[0, 0] == -1).all()                                        # the other slot is untouched


def test_writeback_and_slot_reset():
    tier, cold = _tier()
    L = tier.layer(0)
    tier.hot[0, 70] = torch.arange(8, dtype=torch.uint8) + 100
    ref.hisparse_writeback(L["hot"], L["cold"], torch.tensor([70]), torch.tensor([37]))
    assert torch.equal(cold.view(-1, 8)[37], torch.arange(8, dtype=torch.uint8) + 100)
    tier.pos_to_hot[0, 1, 5] = 3
    tier.assign(1, seq_id=9)
    assert int(tier.pos_to_hot[0, 1, 5]) == -1 and tier.loads == 1
    tier.pos_to_hot[0, 1, 5] = 3
    tier.assign(1, seq_id=9)                                                          # same owner: nothing is reset
    assert int(tier.pos_to_hot[0, 1, 5]) == 3 and tier.loads == 1


def _mc():
    return tiny_deepseek_v3(index_n_heads=2, index_head_dim=32, index_topk=32)


def _cfg(mode, **kw):
    base = dict(model="tiny-deepseek-v3", model_config=_mc(), dummy_weight=True, dtype="float32", device="cpu", kvcache_block_size=64,
                max_num_seqs=4, num_kvcache_blocks=32, mode=mode, max_model_len=512)
    base.update(kw)
    return Config(**base)


def test_config_guards():
    with pytest.raises(ValueError):
        _cfg("hybrid", enable_hisparse=True, hisparse_device_buffer_size=128)          # decode engines only
    with pytest.raises(ValueError):
        _cfg("decode", enable_hisparse=True, hisparse_device_buffer_size=64)           # smaller than index_topk + 64
    with pytest.raises(ValueError):
        Config(model="tiny-deepseek-v3", dtype="float32", device="cpu", mode="decode", enable_hisparse=True)   # no indexer


def test_hot_cold_decode_engine_equals_hybrid_engine():
    """Prompts of 150 / 40 / 97 tokens, top-32 selection, 128 hot rows per sequence: the long sequences evict and reload rows
    on most steps, and every token must equal the resident-cache engine's."""
    g = torch.Generator().manual_seed(31)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (150, 40, 97)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in LLM(_cfg("hybrid")).generate(prompts, sp)}
    prefill = LLM(_cfg("prefill", engine_id="p0"))
    decode = LLM(_cfg("decode", engine_id="d0", enable_hisparse=True, hisparse_device_buffer_size=128))
    runner = decode.engine.executor.runner
    assert runner.cache.hisparse is not None and runner.cache.kv.device.type == "cpu"
    tr = LocalTransport([prefill.engine.executor.runner], [runner])
    decode.engine.migrator = KVMigrator(tr, decode.engine.engine_info(), prefill.engine.engine_info())
    firsts = {}
    for b in prefill.generate(prompts, sp, return_serialized=True):
        sid, first = RequestMigrate.from_bytes(b).metadata
        firsts[sid] = first
        decode.add_request_payload(b)
    got = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
    assert got == want
    assert runner.cache.hisparse.loads == 3


def test_dummy_prefill_decode_engine_runs_the_serving_flow():
    decode = LLM(_cfg("decode", engine_id="d1", enable_hisparse=True, hisparse_device_buffer_size=128, dummy_prefill=True))
    outs = decode.generate([list(range(1, 90)), list(range(5, 30))], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    assert sorted(len(o["token_ids"]) for o in outs) == [4, 4]        # the made-up first token counts as the first of the five
