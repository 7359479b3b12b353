"""CLI flag parsing, monitor stack generation, trace merging/compaction, request dump, checkpoint round trip, live weight update."""
import json
import os

import torch

from nanoengine_b200 import Config, LLM, SamplingParams
from nanoengine_b200.models.config import tiny_deepseek_v3
from nanoengine_b200.models.weights import random_hf_weights, save_hf_checkpoint
from nanoengine_b200.server.cli import main as cli_main, parse_config_args
from nanoengine_b200.utils.monitor import write_monitor_stack
from nanoengine_b200.utils.request_dump import RequestDumper
from nanoengine_b200.utils.trace_merger import compact_trace, merge_traces, summarize_kernels


def test_cli_flags_and_role_overrides():
    common, roles = parse_config_args(["--attention_dp", "8", "--ffn-ep", "8", "--enforce_eager", "--prefill.max_num_seqs", "4",
                                       "--decode.num_speculative_tokens", "2", "--hf_overrides", '{"n_group": 1}'])
    assert common == {"attention_dp": 8, "ffn_ep": 8, "enforce_eager": True, "hf_overrides": {"n_group": 1}}
    assert roles == {"prefill": {"max_num_seqs": 4}, "decode": {"num_speculative_tokens": 2}}


def test_monitor_stack(tmp_path):
    files = write_monitor_stack(str(tmp_path), ["127.0.0.1:8000", "127.0.0.1:8001"])
    text = open(os.path.join(tmp_path, "prometheus.yml")).read()
    assert '"127.0.0.1:8001"' in text and any(f.endswith("nanoengine-overview.json") for f in files)
    dash = json.load(open(os.path.join(tmp_path, "grafana", "dashboards", "nanoengine-overview.json")))
    assert any("dlengine_ttft_seconds_bucket" in p["targets"][0]["expr"] for p in dash["panels"])
    assert cli_main(["monitor", "--targets", "a:1", "--out", str(tmp_path / "m2")]) == 0


def test_trace_merge_compact_summarize(tmp_path):
    def tr(ts0, name):
        return {"traceEvents": [{"ph": "M", "name": "process_name", "pid": 1, "args": {"name": "python"}},
                                {"ph": "X", "cat": "kernel", "name": name, "pid": 1, "tid": 7, "ts": ts0, "dur": 50.0},
                                {"ph": "X", "cat": "kernel", "name": "tiny", "pid": 1, "tid": 7, "ts": ts0 + 60, "dur": 0.5},
                                {"ph": "X", "cat": "python_function", "name": "f", "pid": 1, "tid": 1, "ts": ts0, "dur": 500}]}
    p0, p1 = tmp_path / "t.rank0.json", tmp_path / "t.rank1.json"
    p0.write_text(json.dumps(tr(1000, "gemm"))); p1.write_text(json.dumps(tr(9000, "gemm")))
    merged = tmp_path / "merged.json"
    assert merge_traces([str(p0), str(p1)], str(merged)) == 8
    evs = json.load(open(merged))["traceEvents"]
    assert len({e["pid"] for e in evs}) == 2 and min(e["ts"] for e in evs if e["ph"] == "X") == 0
    small = tmp_path / "small.json"
    assert compact_trace(str(merged), str(small)) == 4       # metadata + the two long kernels
    assert summarize_kernels(str(merged))[0][:2] == ("gemm", 2)


def test_request_dump(tmp_path):
    d = RequestDumper(path=str(tmp_path / "req.jsonl"))
    d.dump({"seq_id": 1, "prompt_len": 5})
    assert json.loads(open(tmp_path / "req.jsonl").read())["seq_id"] == 1
    assert not RequestDumper().enabled


def _gen(llm, prompt):
    return llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))[0]["token_ids"]


def test_checkpoint_roundtrip_bf16_and_fp8_and_weight_update(tmp_path):
    cfg = tiny_deepseek_v3()
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 1024, (20,), generator=g).tolist()
    base = dict(dtype="float32", device="cpu", kvcache_block_size=16, num_kvcache_blocks=32)
    # bf16 checkpoint: weights rounded to bf16 on disk -> compare against an engine built from the same rounded tensors
    ck = tmp_path / "ck"
    save_hf_checkpoint(str(ck), cfg, random_hf_weights(cfg, seed=3))
    assert os.path.exists(ck / "config.json")
    from_disk = LLM(Config(model=str(ck), **base))
    ref_llm = LLM(Config(model="tiny-deepseek-v3", seed=3, **base))
    ref_llm.engine.executor.runner.load_weights((n, t.to(torch.bfloat16).float()) for n, t in random_hf_weights(cfg, seed=3))
    assert _gen(from_disk, prompt) == _gen(ref_llm, prompt)
    # fp8 block-quantised checkpoint loads through the weight_scale_inv path
    ck8 = tmp_path / "ck8"
    save_hf_checkpoint(str(ck8), cfg, random_hf_weights(cfg, seed=3), quantize_fp8=True)
    q = LLM(Config(model=str(ck8), **base))
    assert q.config.model_config.quant == "fp8" and len(_gen(q, prompt)) == 5
    # live weight update: swap in another checkpoint without rebuilding the engine
    ck2 = tmp_path / "ck2"
    save_hf_checkpoint(str(ck2), cfg, random_hf_weights(cfg, seed=9))
    other = LLM(Config(model=str(ck2), **base))
    assert from_disk.update_weights(str(ck2)) > 0
    assert _gen(from_disk, prompt) == _gen(other, prompt)


def test_graph_branch_lanes_are_folded(tmp_path):
    from nanoengine_b200.utils.trace_merger import compact_stream_lanes
    evs = [{"ph": "M", "name": "thread_name", "pid": 1, "tid": t, "args": {"name": f"stream {t}"}} for t in range(7, 13)]
    for t in range(7, 12):                               # five copies of the same branch: gate_up GEMM, SwiGLU, down GEMM
        for i, n in enumerate(["gemm", "silu", "gemm"]):
            evs.append({"ph": "X", "cat": "kernel", "name": n, "pid": 1, "tid": t, "ts": 100 * t + 10 * i, "dur": 5})
    evs.append({"ph": "X", "cat": "kernel", "name": "mla", "pid": 1, "tid": 12, "ts": 5, "dur": 50})      # the main stream
    src, dst = tmp_path / "t.json", tmp_path / "c.json"
    src.write_text(json.dumps({"traceEvents": evs}))
    assert compact_stream_lanes(str(src), str(dst)) == 4
    out = json.load(open(dst))["traceEvents"]
    kernels = [e for e in out if e.get("ph") == "X"]
    assert len(kernels) == 16 and {e["tid"] for e in kernels} == {7, 12}
    assert sum(1 for e in out if e.get("ph") == "M") == 2


def test_trace_compactor_folds_short_repeats_and_drops_python_frames(tmp_path):
    import json
    from nanoengine_b200.utils.trace_compactor import compact_events, compact_file
    ev = [{"ph": "X", "cat": "python_function", "name": "f", "pid": 1, "tid": 1, "ts": 0, "dur": 100}]
    ev += [{"ph": "X", "cat": "kernel", "name": "tiny", "pid": 1, "tid": 7, "ts": 10 + 3 * i, "dur": 2} for i in range(50)]
    ev += [{"ph": "X", "cat": "kernel", "name": "gemm", "pid": 1, "tid": 7, "ts": 200, "dur": 80},
           {"ph": "X", "cat": "kernel", "name": "tiny", "pid": 1, "tid": 7, "ts": 300, "dur": 2},
           {"ph": "s", "cat": "ac2g", "name": "flow", "pid": 1, "tid": 1, "ts": 5},
           {"ph": "M", "name": "process_name", "pid": 1, "args": {"name": "rank0"}}]
    out = list(compact_events(ev))
    names = [(e["name"], e.get("args", {}).get("count", 1)) for e in out if e.get("ph") == "X"]
    assert ("tiny", 50) in names and ("gemm", 1) in names and ("tiny", 1) in names and not any(n == "f" for n, _ in names)
    folded = next(e for e in out if e.get("args", {}).get("count") == 50)
    assert folded["ts"] == 10 and folded["ts"] + folded["dur"] == 10 + 3 * 49 + 2
    assert any(e.get("ph") == "M" for e in out)
    src, dst = tmp_path / "t.json", tmp_path / "c.json"
    src.write_text(json.dumps({"traceEvents": ev, "displayTimeUnit": "ms"}))
    st = compact_file(str(src), str(dst))
    assert st["events_in"] == len(ev) and st["events_out"] == len(out)
    assert json.loads(dst.read_text())["displayTimeUnit"] == "ms"


def test_nvtx_ranges_are_free_when_off_and_harmless_without_a_gpu():
    from nanoengine_b200.utils import nvtx
    assert not nvtx.enabled()
    with nvtx.range("x"):
        pass
    nvtx.enable(True)
    with nvtx.range("y"):
        pass
    nvtx.enable(False)


def test_routing_strategy_accepts_both_spellings():
    from nanoengine_b200 import Config
    for given, want in (("LeastBatch", "least_batch"), ("RoundRobin", "round_robin"), ("least_cache", "least_cache"), ("Affinity", "affinity")):
        assert Config(model="tiny-deepseek-v3", device="cpu", routing_strategy=given).routing_strategy == want
    import pytest
    with pytest.raises(ValueError):
        Config(model="tiny-deepseek-v3", device="cpu", routing_strategy="Random")
