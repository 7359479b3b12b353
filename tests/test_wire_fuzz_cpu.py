"""Property tests of the C++ wire protocol and scheduler: arbitrary and mutated bytes never crash a parser (they raise ValueError),
round trips are exact, and random request streams leave the block pool balanced."""
import random

from hypothesis import given, settings, strategies as st

from nanoengine_b200._native import _core as C

PARSERS = [C.RequestIn, C.RequestMigrate, C.MigrationIn, C.RunnerIn, C.RunnerOut, C.WirePacket]


@settings(derandomize=True, max_examples=200, deadline=None)
@given(st.binary(max_size=256))
def test_arbitrary_bytes_are_rejected_not_crashed_on(data):
    for cls in PARSERS:
        try:
            cls.from_bytes(data)
        except ValueError:
            pass


@settings(derandomize=True, max_examples=150, deadline=None)
@given(st.lists(st.integers(0, 2 ** 31 - 1), min_size=1, max_size=64), st.integers(1, 2 ** 40), st.floats(0, 4, allow_nan=False),
       st.integers(1, 4096), st.booleans(), st.integers(0, 2 ** 60), st.data())
def test_request_round_trip_and_single_byte_mutations(tokens, seq_id, temp, max_tokens, ignore_eos, affinity, data):
    sp = C.SamplingParams(temperature=temp, max_tokens=max_tokens, ignore_eos=ignore_eos)
    b = C.RequestIn(seq_id, tokens, sp, affinity).to_bytes()
    r = C.RequestIn.from_bytes(b)
    assert r.seq_id == seq_id and list(r.prompt_token_ids) == tokens and r.affinity_key == affinity
    assert abs(r.sampling_params.temperature - temp) < 1e-6 and r.sampling_params.max_tokens == max_tokens
    pos = data.draw(st.integers(0, len(b) - 1))
    bad = bytearray(b)
    bad[pos] ^= data.draw(st.integers(1, 255))
    try:
        C.RequestIn.from_bytes(bytes(bad))          # a flipped byte parses to something else or is refused; never a crash
    except ValueError:
        pass
    try:
        C.RequestIn.from_bytes(b[: data.draw(st.integers(0, len(b) - 1))])      # truncation
    except ValueError:
        pass


@settings(derandomize=True, max_examples=40, deadline=None)
@given(st.integers(0, 2 ** 32 - 1))
def test_random_request_streams_leave_the_block_pool_balanced(seed):
    rng = random.Random(seed)
    cfg = C.SchedulerConfig()
    cfg.num_blocks, cfg.block_size, cfg.max_num_seqs = 32, 4, 4
    cfg.max_num_batched_tokens, cfg.max_model_len, cfg.eos_token_ids = 32, 256, [2]
    cfg.enable_prefix_caching = rng.random() < 0.5
    s = C.Scheduler(cfg)
    next_id, live = 1, set()
    for _ in range(rng.randint(5, 40)):
        if rng.random() < 0.5 and len(live) < 12:
            toks = [rng.randint(3, 50) for _ in range(rng.randint(1, 40))]
            s.add_request_bytes(C.RequestIn(next_id, toks, C.SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 6))).to_bytes())
            live.add(next_id); next_id += 1
        if live and rng.random() < 0.15:
            victim = rng.choice(sorted(live))
            s.abort(victim); live.discard(victim)
        res = s.schedule()
        if not res.has_work:
            continue
        outs = []
        for b in s.serialize_run_batches():
            rin = C.RunnerIn.from_bytes(b)          # what a worker receives
            ids = [sid for sid, m in zip(rin.seq_ids, rin.sample_mask) if m]
            outs.append(C.RunnerOut(ids, [[rng.choice([2, 7, 9])] for _ in ids]).to_bytes())
        for o in s.postprocess_runner_out_bytes(outs, 1.0):
            if o.status == C.FINISHED:
                live.discard(o.seq_id)
    for sid in sorted(live):
        s.abort(sid)
    assert s.is_finished()
    assert s.num_free_blocks() == 32
