"""The scripts under examples/ run end to end on CPU with tiny random-weight models (each in its own interpreter, as a user runs
them), and the disaggregated example prints what the single-engine example prints."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, *args, timeout=240):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *args], capture_output=True, text=True, timeout=timeout,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert p.returncode == 0, p.stderr[-2000:]
    return p.stdout.strip().splitlines()


def test_offline_and_disaggregated_examples_agree():
    a = _run("non_disagg.py", "--device", "cpu", "--max_tokens", "6", "--prompt", "hello there", "--prompt", "two plus two")
    b = _run("disagg.py", "--device", "cpu", "--max_tokens", "6", "--prompt", "hello there", "--prompt", "two plus two")
    assert len(a) == 2 and a == b


def test_dummy_prefill_and_encoder_examples():
    out = _run("dummy_prefill.py", "--device", "cpu", "--context", "40", "--max_tokens", "4", "--num_requests", "3")
    assert out[-1].startswith("3 sequences x 40 tokens of context")
    out = _run("encoder_engine.py", "--device", "cpu", "--max_tokens", "3")
    assert out[0].startswith("encoded 2 images into slot") and "generated 3 tokens" in out[1]


def test_http_load_generator_example():
    out = _run("bench_serving.py", "--self_host", "--requests", "5", "--rate", "0", "--prompt_len", "8:1,20:1", "--max_tokens", "4")
    rec = json.loads(out[-1])
    assert rec["requests"] == 5 and rec["ttft_ms_p50"] > 0
