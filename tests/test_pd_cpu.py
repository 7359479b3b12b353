"""Prefill/decode disaggregation on CPU engines in one process: a prompt prefilled on one engine and decoded on another
yields exactly the tokens of a hybrid engine; incompatible engines are refused; a vanished peer fails only that request."""
import pytest
import torch

from nanoengine_b200 import Config, LLM, RequestMigrate, SamplingParams
from nanoengine_b200.parallel.kv_transfer import KVMigrator, LocalTransport, check_compatible


def _cfg(mode, **kw):
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=64, mode=mode)
    base.update(kw)
    return Config(**base)


def _prompts():
    g = torch.Generator().manual_seed(21)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (30, 17, 45)]


def _pair(**kw):
    prefill, decode = LLM(_cfg("prefill", engine_id="p0", **kw)), LLM(_cfg("decode", engine_id="d0", **kw))
    tr = LocalTransport([prefill.engine.executor.runner], [decode.engine.executor.runner])
    decode.engine.migrator = KVMigrator(tr, decode.engine.engine_info(), prefill.engine.engine_info())
    return prefill, decode


def test_pd_pipeline_equals_hybrid():
    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in LLM(_cfg("hybrid")).generate(_prompts(), sp)}
    prefill, decode = _pair()
    blobs = prefill.generate(_prompts(), sp, return_serialized=True)
    assert len(blobs) == 3
    firsts = {}
    for b in blobs:
        m = RequestMigrate.from_bytes(b)
        sid, first = m.metadata
        firsts[sid] = first
        decode.add_request_payload(b)
    outs = {o["seq_id"]: o["token_ids"] for o in decode.generate()}
    got = {sid: [firsts[sid]] + toks for sid, toks in outs.items()}
    assert got == want
    assert prefill.free_to_be_migrated_ids(list(firsts)) == 3
    assert prefill.engine.scheduler.num_free_blocks() == 64


def test_pd_with_mtp_hands_the_drafts_over():
    kw = dict(hf_overrides={"num_nextn_predict_layers": 1}, num_speculative_tokens=2)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in LLM(_cfg("hybrid", **kw)).generate(_prompts()[:2], sp)}
    prefill, decode = _pair(**kw)
    blobs = prefill.generate(_prompts()[:2], sp, return_serialized=True)
    firsts = {}
    for b in blobs:
        sid, first = RequestMigrate.from_bytes(b).metadata
        firsts[sid] = first
        decode.add_request_payload(b)
    outs = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
    assert outs == want


def test_incompatible_engines_and_vanished_peer():
    a = {"architecture": "X", "block_size": 64, "kv_cache_dtype": "fp8", "num_hidden_layers": 4, "mtp_num_kv_layers": 0, "num_blocks": 8}
    with pytest.raises(ValueError):
        check_compatible(a, dict(a, block_size=16))
    prefill, decode = _pair()
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    blobs = prefill.generate(_prompts()[:2], sp, return_serialized=True)
    decode.engine.migrator.fail_next = True          # the first transfer fails on the host; no GPU fault involved
    for b in blobs:
        decode.add_request_payload(b)
    outs = decode.generate()
    assert len(outs) == 1                              # the failed request was dropped, the other one decoded
    assert decode.engine.scheduler.num_free_blocks() == 64


def _push_pair(**kw):
    from nanoengine_b200.parallel.kv_transfer import connect_inproc
    prefill, decode = LLM(_cfg("prefill", engine_id="p0", **kw)), LLM(_cfg("decode", engine_id="d0", **kw))
    connect_inproc(prefill.engine, decode.engine)
    return prefill, decode


def test_push_protocol_equals_hybrid():
    """The push transport end to end on CPU engines: the decode workers publish their pools, the prefill worker maps them and
    copies pages by the same (plane, page) arithmetic the GPU kernel uses, completion flags gate the admission."""
    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in LLM(_cfg("hybrid")).generate(_prompts(), sp)}
    prefill, decode = _push_pair()
    firsts = {}
    for b in prefill.generate(_prompts(), sp, return_serialized=True):
        sid, first = RequestMigrate.from_bytes(b).metadata
        firsts[sid] = first
        decode.add_request_payload(b)
    outs = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
    assert outs == want
    flags = decode.engine.executor.runner.pd_flags
    assert sorted(int(v) for v in flags if int(v) > 0) == [1, 2, 3]        # one ticket per request, each raised once
    summary = decode.engine.scheduler.metrics_summary()
    assert summary.get("transfer_bytes", 1) > 0


def test_push_with_mtp_and_indexer_pages():
    """A DSA model with MTP: indexer key pages travel with the latent pages and the draft hand-off row lands in the decode
    engine's table."""
    from nanoengine_b200.models.config import tiny_deepseek_v3
    mc = tiny_deepseek_v3(index_topk=8, index_n_heads=4, index_head_dim=128, num_nextn_predict_layers=1)
    kw = dict(model_config=mc, num_speculative_tokens=2, dummy_weight=True)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in LLM(_cfg("hybrid", **kw)).generate(_prompts()[:2], sp)}
    prefill, decode = _push_pair(**kw)
    assert [f["name"] for f in decode.engine.executor.runner.cache.page_families()] == ["mla_kv", "indexer"]
    firsts = {}
    for b in prefill.generate(_prompts()[:2], sp, return_serialized=True):
        sid, first = RequestMigrate.from_bytes(b).metadata
        firsts[sid] = first
        decode.add_request_payload(b)
    outs = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
    assert outs == want


def test_push_whose_producer_never_runs_fails_only_that_request():
    prefill, decode = _push_pair()
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    blobs = prefill.generate(_prompts()[:2], sp, return_serialized=True)
    tr = decode.engine.migrator.transport
    real = tr.pusher
    tr.pusher = lambda reqs: [0] + real(reqs[1:])            # the first request's push is never queued: its flag never comes
    for b in blobs:
        decode.add_request_payload(b)
    outs = decode.generate()
    assert len(outs) == 1
    assert decode.engine.scheduler.num_free_blocks() == 64


def test_layout_mismatch_is_refused_at_connect_time():
    from nanoengine_b200.parallel.kv_transfer import check_families
    a = [{"name": "mla_kv", "planes": 2, "page_bytes": 1024}]
    with pytest.raises(ValueError):
        check_families(a, [{"name": "mla_kv", "planes": 2, "page_bytes": 2048}])
    with pytest.raises(ValueError):
        check_families(a, a + [{"name": "indexer", "planes": 2, "page_bytes": 64}])


def test_pd_packets_between_engine_processes_round_trip():
    """The ACT_PD_OPEN / ACT_PD_PUSH envelopes: memory handles travel as hex inside JSON and reach every prefill worker as bytes;
    a ZMQ DEALER/ROUTER pair carries them, errors come back as errors."""
    import json
    import threading
    import zmq
    from nanoengine_b200._native import _core as C
    from nanoengine_b200.parallel.kv_transfer import PdPeerClient, _hexify, serve_pd_packet

    class FakeExecutor:
        def __init__(self):
            self.calls = []

        def collective_rpc(self, method, *args):
            self.calls.append((method, args))
            if method == "pd_open_pool":
                return [1, 1]
            if method == "pd_push":
                return [[10, 0], [0, 20]]                      # two prefill workers, each served its own request
            raise KeyError(method)

    class FakeEngine:
        executor = FakeExecutor()

        def engine_info(self):
            return {"id": "p0", "num_blocks": 9}

    eng = FakeEngine()
    ep = "inproc://pd-test"
    ctx = zmq.Context.instance()
    srv = ctx.socket(zmq.ROUTER)
    srv.bind(ep)

    def serve(n):
        for _ in range(n):
            ident, payload = srv.recv_multipart()
            pkt = C.WirePacket.from_bytes(payload)
            try:
                reply = serve_pd_packet(eng, pkt.action, pkt.payload)
            except Exception as e:
                reply = json.dumps({"error": str(e)}).encode()
            srv.send_multipart([ident, C.WirePacket(pkt.action, reply).to_bytes()])

    th = threading.Thread(target=serve, args=(3,), daemon=True)
    th.start()
    cli = PdPeerClient(ep, timeout_s=5.0)
    pools = [{"dp": 0, "tp": 0, "num_blocks": 4, "families": [{"name": "mla_kv", "planes": 2, "plane_stride": 64, "page_bytes": 16, "tensor": b"\\x01\\x02"}],
              "flags": b"\\x03", "handoff": None}]
    out = cli.call(C.ACT_PD_OPEN, {"key": "d0", "pools": _hexify(pools)})
    assert out["mapped"] == 2 and out["info"]["id"] == "p0"
    method, (key, got) = eng.executor.calls[0]
    assert method == "pd_open_pool" and key == "d0" and got[0]["families"][0]["tensor"] == b"\\x01\\x02" and got[0]["flags"] == b"\\x03"
    assert cli.call(C.ACT_PD_PUSH, {"key": "d0", "reqs": [{"src_dp": 0}, {"src_dp": 1}]})["sizes"] == [10, 20]
    eng.executor.collective_rpc = lambda *a: (_ for _ in ()).throw(ValueError("kv push: page ids outside the pools"))
    with pytest.raises(RuntimeError, match="outside the pools"):
        cli.call(C.ACT_PD_PUSH, {"key": "d0", "reqs": [{"src_dp": 0}]})
    th.join(timeout=5)
    srv.close(0)


def _state_family_configs():
    from nanoengine_b200.models.config import tiny_deepseek_v4, tiny_glm5_next, tiny_qwen3_5
    return {"qwen3.5": (tiny_qwen3_5(moe=True), 512), "glm5-next": (tiny_glm5_next(), 512), "deepseek-v4": (tiny_deepseek_v4(head_dim=80), 512)}


@pytest.mark.parametrize("family", ["qwen3.5", "glm5-next", "deepseek-v4"])
@pytest.mark.parametrize("transport", ["local", "push"])
def test_families_with_per_sequence_state_migrate_their_state(family, transport):
    """A sequence of a family with per-sequence state (delta-rule state and convolution window; compressor carries and pooled-row
    pages) decodes on the other engine exactly as on a hybrid engine: the state slot of the prefill side travels with the pages
    into the slot the decode scheduler assigned, which differs from the source slot here."""
    mc, vocab = _state_family_configs()[family]
    kw = dict(model="tiny", model_config=mc, dummy_weight=True)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (30, 17, 45)]
    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in LLM(_cfg("hybrid", **kw)).generate(prompts, sp)}
    prefill, decode = LLM(_cfg("prefill", engine_id="p0", **kw)), LLM(_cfg("decode", engine_id="d0", **kw))
    if transport == "local":
        tr = LocalTransport([prefill.engine.executor.runner], [decode.engine.executor.runner])
        decode.engine.migrator = KVMigrator(tr, decode.engine.engine_info(), prefill.engine.engine_info())
    else:
        from nanoengine_b200.parallel.kv_transfer import connect_inproc
        connect_inproc(prefill.engine, decode.engine)
    firsts = {}
    blobs = prefill.generate(prompts, sp, return_serialized=True)
    for b in reversed(blobs):                      # admitted in the other order: source and destination slots differ
        sid, first = RequestMigrate.from_bytes(b).metadata
        firsts[sid] = first
        decode.add_request_payload(b)
    outs = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
    assert outs == want
