"""Scheduler / block-manager scenarios on the native control plane.

Modelled on the reference's Rust scenarios (rust/src/scheduler/tests.rs:254-852): migration
retention, slot exhaustion, per-DP limits, host swap, prefix reuse/eviction, chunked prefill
versus prefix hits, speculative reservation and bundle truncation.
"""
import pytest

from nanoengine_b200._native import _core as C


def make(num_blocks=64, block_size=4, **kw):
    cfg = C.SchedulerConfig()
    cfg.num_blocks = num_blocks
    cfg.block_size = block_size
    cfg.max_num_seqs = kw.pop("max_num_seqs", 8)
    cfg.max_num_batched_tokens = kw.pop("max_num_batched_tokens", 64)
    cfg.max_model_len = kw.pop("max_model_len", 4096)
    cfg.eos_token_ids = kw.pop("eos", [2])
    for k, v in kw.items():
        setattr(cfg, k, v)
    return C.Scheduler(cfg)


def add(s, sid, toks, max_tokens=8, **kw):
    sp = C.SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw)
    s.add_request_bytes(C.RequestIn(sid, toks, sp).to_bytes())


def step(s, tok_fn=lambda sid, i: 7, n_per_seq=1):
    r = s.schedule()
    if not r.has_work:
        return r, []
    outs = []
    for b in r.batches:
        ids, toks = [], []
        for i, sid in enumerate(b.seq_ids):
            if b.sample_mask[i]:
                ids.append(sid)
                toks.append([tok_fn(sid, j) for j in range(n_per_seq)])
        outs.append(C.RunnerOut(ids, toks))
    return r, s.postprocess_runner_outs(outs)


def run_all(s, **kw):
    done = {}
    for _ in range(10000):
        if s.is_finished():
            break
        _, outs = step(s, **kw)
        for o in outs:
            done.setdefault(o.seq_id, []).extend(o.token_ids)
    return done


def test_prefill_then_decode_until_max_tokens():
    s = make()
    add(s, 1, list(range(10, 20)), max_tokens=3)
    r, outs = step(s)
    assert r.is_prefill and r.num_tokens == 10
    assert outs[0].token_ids == [7] and outs[0].status == C.RUNNING
    r, outs = step(s)
    assert not r.is_prefill and r.batches[0].input_ids == [7] and r.batches[0].positions == [10]
    r, outs = step(s)
    assert outs[0].status == C.FINISHED
    assert s.is_finished() and s.num_free_blocks() == 64


def test_prefill_has_priority_and_existing_running_are_preserved():
    s = make()
    add(s, 1, [5] * 6)
    step(s)
    add(s, 2, [6] * 6)
    r, _ = step(s)
    assert r.is_prefill and r.batches[0].seq_ids == [2]
    r, _ = step(s)
    assert not r.is_prefill and sorted(r.batches[0].seq_ids) == [1, 2]


def test_eos_stops_unless_ignored():
    s = make()
    add(s, 1, [5] * 4, max_tokens=10)
    add(s, 2, [6] * 4, max_tokens=4, ignore_eos=True)
    done = run_all(s, tok_fn=lambda sid, i: 2)
    assert done[1] == [2] and done[2] == [2, 2, 2, 2]


def test_chunked_prefill_splits_by_token_budget():
    s = make(max_num_batched_tokens=8)
    add(s, 1, list(range(100, 120)), max_tokens=1)
    r, outs = step(s)
    assert r.num_tokens == 8 and outs[0].status == C.PREFILLING and outs[0].token_ids == []
    r, outs = step(s)
    assert r.batches[0].positions[0] == 8 and outs[0].status == C.PREFILLING
    r, outs = step(s)
    assert r.num_tokens == 4 and outs[0].status == C.FINISHED and outs[0].token_ids == [7]


def test_prefix_cache_reuse_after_release_and_cap_at_tokens_minus_one():
    s = make()
    prompt = list(range(50, 58))  # two full blocks
    add(s, 1, prompt, max_tokens=1)
    run_all(s)
    assert s.num_cached_blocks() >= 1
    add(s, 2, prompt, max_tokens=1)
    r, _ = step(s)
    # 8 tokens, 2 cached blocks would cover all 8 -> capped at (8-1)//4 = 1 block
    assert r.prefix_hit_tokens == 4 and r.num_tokens == 4
    assert r.batches[0].positions == [4, 5, 6, 7]


def test_prefix_cache_can_be_disabled_and_gdn_never_uses_it():
    for kw in ({"enable_prefix_caching": False}, {"cache_plan": C.PLAN_GDN | C.PLAN_GQA, "num_state_slots": 4}):
        s = make(**kw)
        assert not s.config.prefix_cache_effective()
        add(s, 1, list(range(8)) + [9], max_tokens=1)
        run_all(s)
        add(s, 2, list(range(8)) + [9], max_tokens=1)
        r, _ = step(s)
        assert r.prefix_hit_tokens == 0 and r.num_tokens == 9


def test_chunked_prefill_keeps_prefix_hit_separate_from_chunk_offset():
    s = make(max_num_batched_tokens=6)
    base = list(range(200, 212))
    add(s, 1, base, max_tokens=1)
    run_all(s)
    add(s, 2, base + [1, 2, 3, 4, 5, 6, 7, 8], max_tokens=1)
    r, _ = step(s)
    assert r.prefix_hit_tokens == 12
    first = r.batches[0].positions[0]
    assert first == r.prefix_hit_tokens and r.num_tokens == 6
    r, _ = step(s)
    assert r.batches[0].positions[0] == first + 6


def test_lru_eviction_of_cached_blocks_when_pool_is_short():
    s = make(num_blocks=6)
    add(s, 1, list(range(16)), max_tokens=1)
    run_all(s)
    assert s.num_cached_blocks() > 0
    add(s, 2, list(range(100, 120)), max_tokens=1)  # needs 5-6 blocks -> must evict
    done = run_all(s)
    assert done[2] == [7]


def test_decode_growth_preempts_least_recently_scheduled_and_recomputes():
    s = make(num_blocks=4, block_size=4, enable_prefix_caching=False)
    add(s, 1, [1] * 7, max_tokens=8)
    add(s, 2, [3] * 7, max_tokens=8)
    done = run_all(s)
    assert len(done[1]) == 8 and len(done[2]) == 8
    assert s.num_free_blocks() == 4


def test_host_swap_restores_without_prefill():
    s = make(num_blocks=4, block_size=4, enable_prefix_caching=False, num_host_blocks=8, swap_cooldown_steps=1)
    add(s, 1, [1] * 7, max_tokens=6)
    add(s, 2, [3] * 7, max_tokens=6)
    saw_out = saw_in = False
    prefill_steps = 0
    done = {}
    for _ in range(200):
        if s.is_finished():
            break
        r, outs = step(s)
        prefill_steps += int(r.has_work and r.is_prefill)
        for b in r.batches:
            saw_out |= bool(b.swap_out_src)
            saw_in |= bool(b.swap_in_src)
        for o in outs:
            done.setdefault(o.seq_id, []).extend(o.token_ids)
    assert saw_out and saw_in
    assert prefill_steps == 1  # both prompts prefilled once; the swapped sequence was never recomputed
    assert len(done[1]) == 6 and len(done[2]) == 6
    assert s.num_free_host_blocks() == 8


def test_max_num_seqs_and_slots_are_per_dp_rank():
    s = make(attention_dp=2, max_num_seqs=1, num_handoff_slots=1, num_speculative_tokens=1)
    for i in range(3):
        add(s, i + 1, [4] * 5)
    r, _ = step(s)
    assert [len(b.seq_ids) for b in r.batches] == [1, 1]
    assert s.num_waiting() == 1
    assert s.num_free_handoff_slots(0) == 0 and s.num_free_handoff_slots(1) == 0


def test_idle_dp_rank_gets_dummy_batch():
    s = make(attention_dp=2)
    add(s, 1, [4] * 5)
    r, _ = step(s)
    assert len(r.batches) == 2 and sum(b.is_dummy for b in r.batches) == 1


def test_exhausted_state_slot_keeps_request_waiting():
    s = make(cache_plan=C.PLAN_GDN | C.PLAN_GQA, num_state_slots=1)
    add(s, 1, [4] * 5, max_tokens=2)
    add(s, 2, [4] * 5, max_tokens=2)
    r, _ = step(s)
    assert r.batches[0].seq_ids == [1] and s.num_waiting() == 1
    done = run_all(s)
    assert set(done) == {1, 2}


def test_speculative_reservation_and_bundle_truncation():
    s = make(block_size=4, num_speculative_tokens=2, num_handoff_slots=4)
    add(s, 1, [9] * 4, max_tokens=10)
    step(s)
    assert len(s.get(1).block_table) == 2       # prompt 4 + N=2 look-ahead -> 6 tokens -> 2 blocks
    r, _ = s.schedule(), None
    assert len(s.get(1).block_table) == 3       # decode: 5 tokens + 2N = 9 -> 3 blocks
    outs = s.postprocess_runner_outs([C.RunnerOut([1], [[5, 2, 6]])])  # EOS in the middle of the bundle
    assert outs[0].token_ids == [5, 2] and outs[0].status == C.FINISHED
    summary = s.metrics_summary()
    assert summary["generated_tokens"] == 3  # first token + the two applied ones


def test_bundle_stops_at_request_token_limit():
    s = make(num_speculative_tokens=2, num_handoff_slots=2)
    add(s, 1, [9] * 4, max_tokens=3)
    step(s)
    s.schedule()
    outs = s.postprocess_runner_outs([C.RunnerOut([1], [[5, 6, 7]])])
    assert outs[0].token_ids == [5, 6] and outs[0].status == C.FINISHED


def test_prefill_mode_hands_over_and_frees():
    s = make(mode=C.MODE_PREFILL, engine_id="p0")
    add(s, 1, [9] * 6, max_tokens=5)
    _, outs = step(s)
    assert outs[0].status == C.TO_BE_MIGRATED and s.is_finished()
    blobs = s.export_to_be_migrated()
    assert len(blobs) == 1 and blobs[0].metadata == (1, 7)
    assert s.export_to_be_migrated() == []
    assert s.num_free_blocks() < 64
    assert s.free_to_be_migrated([1]) == 1 and s.num_free_blocks() == 64

    d = make(mode=C.MODE_DECODE)
    d.add_request_bytes(blobs[0].to_bytes())
    r = d.schedule()
    # pending migration is retained but not runnable
    assert not r.has_work and len(r.migrations) == 1 and not d.is_finished()
    m = r.migrations[0]
    assert m.seq_ids == [1] and len(m.local_blocks) == len(m.remote_blocks) == 2
    d.complete_migration([1], True)
    r, outs = step(d)
    assert not r.is_prefill and r.batches[0].input_ids == [7] and r.batches[0].positions == [6]


def test_failed_migration_releases_everything():
    p = make(mode=C.MODE_PREFILL)
    add(p, 1, [9] * 6)
    step(p)
    blob = p.export_to_be_migrated()[0]
    d = make(mode=C.MODE_DECODE)
    d.add_request_bytes(blob.to_bytes())
    d.schedule()
    d.complete_migration([1], False)
    assert d.is_finished() and d.num_free_blocks() == 64


def test_abort_mid_prefill_releases_blocks():
    s = make(max_num_batched_tokens=4)
    add(s, 1, [9] * 12)
    step(s)
    assert s.num_free_blocks() < 64
    assert s.abort(1) and not s.abort(1)
    assert s.is_finished() and s.num_free_blocks() == 64


def test_affinity_routing_waits_three_steps_for_preferred_rank():
    s = make(attention_dp=2, routing=C.AFFINITY, max_num_seqs=1)
    sp = C.SamplingParams(temperature=0.0, max_tokens=50)
    s.add_request(C.RequestIn(1, [1] * 5, sp, affinity_key=77))
    step(s)
    pref = s.get(1).dp_idx
    s.add_request(C.RequestIn(2, [1] * 5, sp, affinity_key=77))
    for _ in range(3):
        step(s)
        assert s.num_waiting() == 1  # preferred rank is full; holds out
    step(s)
    assert s.num_waiting() == 0 and s.get(2).dp_idx != pref


def test_wire_roundtrip_and_corruption():
    sp = C.SamplingParams(temperature=0.5, max_tokens=3, ignore_eos=True, return_completion_logprobs=True)
    r = C.RequestIn(42, [1, 2, 3], sp, affinity_key=9, vision_slots=[4])
    b = r.to_bytes()
    q = C.RequestIn.from_bytes(b)
    assert (q.seq_id, q.prompt_token_ids, q.affinity_key, q.vision_slots) == (42, [1, 2, 3], 9, [4])
    assert q.sampling_params.ignore_eos and abs(q.sampling_params.temperature - 0.5) < 1e-7
    with pytest.raises(ValueError):
        C.RequestIn.from_bytes(b[:-3])
    with pytest.raises(ValueError):
        C.RequestIn.from_bytes(b"\x00" + b[1:])
    with pytest.raises(ValueError):
        C.StepOut.from_bytes(b)
    bad = bytearray(b); bad[10:14] = b"\xff\xff\xff\x7f"
    with pytest.raises(ValueError):
        C.RequestIn.from_bytes(bytes(bad))
    p = C.WirePacket(C.ACT_ADD, b)
    assert C.WirePacket.from_bytes(p.to_bytes()).payload == b


def test_runner_input_preparation():
    s = make(block_size=4)
    add(s, 1, list(range(10)))
    add(s, 2, list(range(6)))
    r = s.schedule()
    b = C.RunnerIn.from_bytes(s.serialize_run_batches()[0])
    d = b.prepare(4)
    assert d["cu_seqlens_q"].tolist() == [0, 10, 16] and d["cu_seqlens_k"].tolist() == [0, 10, 16]
    bt = d["block_tables"].reshape(2, -1)
    for i, pos in enumerate(range(10)):
        assert d["slot_mapping"][i] == bt[0][pos // 4] * 4 + pos % 4
    assert d["last_token_indices"].tolist() == [9, 15]


def test_metrics_prometheus_names():
    s = make()
    add(s, 1, [3] * 5, max_tokens=3)
    run_all(s)
    text = s.metrics_prometheus()
    for name in ("dlengine_up", "dlengine_requests", "dlengine_tokens", "dlengine_step_count",
                 "dlengine_ttft_seconds_bucket", "dlengine_tpot_seconds_count", "dlengine_kv_blocks",
                 "dlengine_running_requests_per_dp", "dlengine_prefix_cache_hit_rate"):
        assert name in text


def test_metrics_report_the_host_tier_hot_slots_and_waiting_migrations():
    s = make()
    text = s.metrics_prometheus()
    assert 'dlengine_requests{state="waiting_migration"} 0' in text
    assert "dlengine_host_kv_blocks" not in text and "dlengine_hisparse_slots" not in text        # tiers that do not exist are not listed
    s = make(num_host_blocks=8, num_hisparse_slots=4, cache_plan=C.PLAN_HISPARSE)
    add(s, 1, [3] * 9, max_tokens=4)
    s.schedule()
    text = s.metrics_prometheus()
    assert 'dlengine_host_kv_blocks{dp="0",state="used"} 0' in text and 'dlengine_host_kv_blocks{dp="0",state="total"} 8' in text
    assert 'dlengine_hisparse_slots{state="used"} 1' in text and 'dlengine_hisparse_slots{state="total"} 4' in text


def test_block_pool_states_and_l3_index():
    p = C.BlockPool(4, 4, True)
    ids = p.allocate(2)
    assert [p.state(i) for i in ids] == [1, 1]
    h = C.chain_hash(0, [1, 2, 3, 4])
    p.commit(ids[0], h)
    p.release(ids)
    assert p.num_cached() == 1 and p.num_free() == 4
    m, last = p.match_prefix([1, 2, 3, 4, 5])
    assert m == [ids[0]] and last == h and p.refcount(ids[0]) == 1
    assert p.allocate(4) is None
    l3 = C.L3Index(2)
    assert l3.insert(1, 10) == 0 and l3.insert(2, 20) == 0
    assert l3.lookup(1) == 10
    assert l3.insert(3, 30) == 2  # LRU entry evicted
    assert l3.match([1, 3, 9]) == 2 and len(l3) == 2


def test_exhausted_mtp_handoff_slot_keeps_request_waiting():
    """Mirror of the reference scenario exhausted_mtp_handoff_slot_keeps_request_waiting (rust/src/scheduler/tests.rs:288)."""
    s = make(num_speculative_tokens=1, num_handoff_slots=1)
    add(s, 1, [4] * 5, max_tokens=3)
    add(s, 2, [4] * 5, max_tokens=3)
    r, _ = step(s)
    assert r.batches[0].seq_ids == [1] and s.num_waiting() == 1 and s.num_free_handoff_slots() == 0
    done = run_all(s)
    assert set(done) == {1, 2} and s.num_free_handoff_slots() == 1


def test_prefix_cache_survives_decode_growth_and_release():
    """Blocks published during prefill stay valid while the sequence grows by decode and after it is released
    (rust/src/scheduler/tests.rs:540)."""
    s = make()
    prompt = list(range(100, 109))                  # two full blocks + 1
    add(s, 1, prompt, max_tokens=6)
    step(s)
    assert s.num_cached_blocks() == 2
    run_all(s)                                       # grows to 15 tokens: the third block fills during decode
    assert s.num_cached_blocks() >= 2
    add(s, 2, prompt + [7, 7, 7], max_tokens=1)
    r, _ = step(s)
    assert r.prefix_hit_tokens >= 8


def test_step_reports_prefix_hits_per_dp_rank():
    """Per-rank hit accounting (rust/src/scheduler/tests.rs:604): the rank that served the prompt before reports the hit."""
    s = make(attention_dp=2)
    prompt = list(range(30, 39))
    add(s, 1, prompt, max_tokens=1)                  # rank 0
    run_all(s)
    add(s, 2, [1] * 9, max_tokens=1)                 # rank 1
    add(s, 3, prompt, max_tokens=1)                  # rank 0 again: hits
    r, _ = step(s)
    assert r.prefix_hit_tokens == 8
    text = s.metrics_prometheus()
    assert "dlengine_prefix_cache_hit_rate_per_dp" in text


def test_reset_prefix_cache_stops_live_sequences_from_publishing():
    """After the cached prefixes are dropped (weights changed), a sequence that was already running holds KV that is stale in
    part: nothing it fills later may be published - in particular not under a hash chained from before the reset, which
    would skip the tokens in between."""
    s = make()
    add(s, 1, list(range(200, 206)), max_tokens=12)          # 6 tokens: one full block published, second block half full
    step(s)
    assert s.num_cached_blocks() == 1
    s.reset_prefix_cache()
    assert s.num_cached_blocks() == 0
    run_all(s)                                               # fills blocks 2..4 while decoding
    assert s.num_cached_blocks() == 0
    add(s, 2, list(range(200, 206)), max_tokens=1)           # a fresh request publishes again
    run_all(s)
    assert s.num_cached_blocks() == 1


def test_import_holds_the_cached_head_of_its_chain():
    """begin_import over [cached, missing, missing] with a pool that has to evict to make room: the cached head must not be
    the block that gets evicted for its own tail."""
    p = C.BlockPool(3, 4, True)
    h = [C.chain_hash(0, [1, 2, 3, 4])]
    h.append(C.chain_hash(h[0], [5, 6, 7, 8]))
    h.append(C.chain_hash(h[1], [9, 9, 9, 9]))
    ids = p.allocate(3)
    p.commit(ids[0], h[0])
    p.release(ids)                                           # block ids[0] is cached and unreferenced (LRU), two are free
    spare = p.allocate(1)                                    # leaves one free block: the import of two needs an eviction
    got = p.begin_import(h)
    assert got[0] == -1 and len(got) == 2 and got[1] >= 0    # the pool ran dry instead of evicting the head
    assert p.refcount(ids[0]) == 1
    p.finish_import(h[: len(got)], got, True)
    assert p.refcount(ids[0]) == 0 and p.num_cached() == 2
    m, last = p.match_prefix([1, 2, 3, 4, 5, 6, 7, 8, 0])
    assert len(m) == 2 and last == h[1]
    p.release(spare)


def test_dummy_batch_of_an_idle_rank_survives_the_wire():
    """An idle SPMD rank runs a dummy batch through the same bytes path as a real one: it must parse."""
    from nanoengine_b200.engine.llm_engine import _dummy_batch
    for prefill in (False, True):
        b = C.RunnerIn.from_bytes(_dummy_batch(prefill).to_bytes())
        assert b.is_dummy and b.is_prefill == prefill and b.num_seqs == 0


def test_status_line_names_requests_cache_and_throughput():
    s = make(num_host_blocks=8)
    add(s, 1, [3] * 9, max_tokens=3)
    run_all(s)
    add(s, 2, [4] * 5, max_tokens=2)
    line = s.status_line("hybrid")
    assert line.startswith("[engine ") and " hybrid] run=0 wait=1 mig=0 | kv=" in line and "/64 blk host=0/8 blk" in line
    assert "tput pf=" in line and "dec=" in line and line.rstrip().endswith("done=1")
