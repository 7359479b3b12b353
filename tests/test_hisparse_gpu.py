"""Hot / cold tier on the GPU: the staging kernel against the plain PyTorch statement on the same tables, and a DSA decode engine
whose latent cache lives in pinned host memory against a resident-cache engine (eager and under CUDA graphs)."""
import pytest
import torch

from nanoengine_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _tiers(hot_rows, max_ctx, pages, row):
    from nanoengine_b200.runtime.hisparse import HiSparseTier
    g = torch.Generator().manual_seed(3)
    cold = torch.randint(0, 255, (pages, 64, row), dtype=torch.uint8, generator=g)
    gpu = HiSparseTier(1, 3, hot_rows, max_ctx, row, [cold.clone().pin_memory()], "cuda")
    cpu = HiSparseTier(1, 3, hot_rows, max_ctx, row, [cold.clone()], "cpu")
    return gpu, cpu


def test_stage_kernel_matches_the_reference_step_by_step():
    from nanoengine_b200.ops import sm100
    sm100.clear_kernel_status()
    hot_rows, max_ctx, topk, row = 256, 1024, 128, 576
    gpu, cpu = _tiers(hot_rows, max_ctx, 48, row)
    B = 3
    bt = torch.randperm(48).view(B, 16).int()                                    # disjoint cold pages per sequence
    slots = torch.tensor([2, 0, 1], dtype=torch.int32)
    g = torch.Generator().manual_seed(4)
    ctx = [700, 90, 400]
    for step in range(6):
        sel = torch.full((B, topk), -1, dtype=torch.int32)
        for b in range(B):
            n = min(topk, ctx[b])
            # a list that overlaps the previous step's (the same generator stream, drifting window) and contains the new position
            cand = torch.cat([torch.tensor([ctx[b] - 1]), torch.randperm(ctx[b] - 1, generator=g)[: n - 1]])     # distinct positions
            sel[b, :n] = cand.int()
        cl = torch.tensor(ctx, dtype=torch.int32)
        want_ids, want_new = ref.hisparse_stage(cpu.layer(0), sel, slots, cl, bt)
        got_ids, got_new = sm100.hisparse_stage(gpu.layer(0), sel.cuda(), slots.cuda(), cl.cuda(), bt.cuda())
        torch.cuda.synchronize()
        assert torch.equal(got_new.cpu(), want_new), step
        assert torch.equal(got_ids.cpu(), want_ids), step                       # same victims in the same order, hence the same ids
        assert torch.equal(gpu.pos_to_hot.cpu(), cpu.pos_to_hot) and torch.equal(gpu.hot_to_pos.cpu(), cpu.hot_to_pos)
        # every listed position other than the new token's holds its cold row
        cold = gpu.cold[0].view(-1, row)
        for b in range(B):
            for i, p in enumerate(sel[b].tolist()):
                if p >= 0 and p != ctx[b] - 1:
                    assert torch.equal(gpu.hot[0, int(got_ids[b, i])].cpu(), cold[int(bt[b, p // 64]) * 64 + p % 64])
        # the key path writes the new row, the write-back copies it to the cold page
        new_rows = torch.randint(0, 255, (B, row), dtype=torch.uint8)
        gpu.hot[0][got_new] = new_rows.cuda()
        cpu.hot[0][want_new] = new_rows
        sm_map = torch.tensor([int(bt[b, (ctx[b] - 1) // 64]) * 64 + (ctx[b] - 1) % 64 for b in range(B)])
        sm100.hisparse_writeback(gpu.layer(0)["hot"], gpu.layer(0)["cold"], got_new, sm_map.cuda())
        ref.hisparse_writeback(cpu.layer(0)["hot"], cpu.layer(0)["cold"], want_new, sm_map)
        torch.cuda.synchronize()
        assert torch.equal(gpu.cold[0], cpu.cold[0])
        ctx = [c + 1 for c in ctx]
    assert sm100.kernel_status()[0] == 0


@pytest.mark.parametrize("eager", [True, False])
def test_hot_cold_decode_engine_equals_resident_engine(eager):
    from nanoengine_b200 import Config, LLM, RequestMigrate, SamplingParams
    from nanoengine_b200.models.config import tiny_deepseek_v3
    from nanoengine_b200.ops import sm100
    from nanoengine_b200.parallel.kv_transfer import KVMigrator, LocalTransport
    mc = tiny_deepseek_v3(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024, q_lora_rank=256, kv_lora_rank=512,
                          qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_attention_heads=16, quant="fp8",
                          index_topk=64, index_n_heads=8, index_head_dim=128)

    def cfg(mode, **kw):
        return Config(model="tiny-deepseek-v3", model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kv_cache_dtype="fp8",
                      kvcache_block_size=64, num_kvcache_blocks=64, max_num_seqs=4, max_model_len=1024, seed=0, mode=mode, **kw)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (300, 150, 90)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in LLM(cfg("hybrid", enforce_eager=True)).generate(prompts, sp)}
    prefill = LLM(cfg("prefill", engine_id="p0", enforce_eager=True))
    decode = LLM(cfg("decode", engine_id="d0", enable_hisparse=True, hisparse_device_buffer_size=128, enforce_eager=eager))
    runner = decode.engine.executor.runner
    assert runner.cache.kv.device.type == "cpu" and runner.cache.kv.is_pinned()
    decode.engine.migrator = KVMigrator(LocalTransport([prefill.engine.executor.runner], [runner]), decode.engine.engine_info(),
                                        prefill.engine.engine_info())
    firsts = {}
    for b in prefill.generate(prompts, sp, return_serialized=True):
        sid, first = RequestMigrate.from_bytes(b).metadata
        firsts[sid] = first
        decode.add_request_payload(b)
    got = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
    if not eager:
        assert runner.graphs is not None and runner.graphs.graphs
    # random weights leave near-ties that the different summation order of hot rows may flip late in a sequence
    same = sum(got[k] == want[k] for k in want)
    assert same >= 2 and all(got[k][:4] == want[k][:4] for k in want), (got, want)
    assert sm100.kernel_status()[0] == 0
