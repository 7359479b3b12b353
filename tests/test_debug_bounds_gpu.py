"""The bounds-checked kernel build (NE_DEBUG_BOUNDS=1): a table entry past the registered bound is recorded in the status words
and its access skipped, and an engine run on that build gives the tokens of the ordinary build.  The out-of-range entries used
here still lie inside the tensors the test allocated, so nothing can fault whatever the check does."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

_SCRIPT = r"""
import torch
from nanoengine_b200.ops import sm100
FP8 = torch.float8_e4m3fn
assert sm100.lib()._name.endswith("libne_kernels_dbg.so")
sm100.clear_kernel_status()
cache = torch.zeros(8, 64, 576, dtype=torch.uint8, device="cuda").view(FP8)            # 512 rows allocated ...
assert sm100.debug_set_bounds(cache_rows=256, cache_pages=4, state_slots=0, experts=0)    # ... 256 declared
T = 3
ckv = torch.randn(T, 512, device="cuda", dtype=torch.bfloat16)
kpe = torch.randn(T, 64, device="cuda", dtype=torch.bfloat16)
slots = torch.tensor([10, 300, -1], device="cuda")
sm100.mla_kv_store(cache, slots, ckv, kpe)
torch.cuda.synchronize()
rows = cache.view(torch.uint8).view(-1, 576)
assert rows[10].any() and not rows[300].any(), "row 10 is written, row 300 (past the declared bound) is skipped"
st = sm100.kernel_status()
assert st[0] == 4 and st[4] == 300, st                                                  # ST_BAD_INDEX with the offending value
sm100.clear_kernel_status()
# a bad page id in a block table: the generic attention kernel drops the key instead of reading it
kc = torch.randn(8, 64, 2, 64, device="cuda", dtype=torch.bfloat16); vc = torch.randn_like(kc)
q = torch.randn(1, 8, 64, device="cuda", dtype=torch.bfloat16)
from nanoengine_b200.ops import sm100_attn
bt = torch.tensor([[1, 6]], dtype=torch.int32, device="cuda")                           # page 6 >= 4 declared pages
out = sm100_attn.gqa_attention_paged(q, kc, vc, bt, torch.tensor([0, 1], dtype=torch.int32, device="cuda"),
                                     torch.tensor([100], dtype=torch.int32, device="cuda"), 0.125)
torch.cuda.synchronize()
st = sm100.kernel_status()
assert st[0] == 4 and st[4] == 6, st
only_first = sm100_attn.gqa_attention_paged(q, kc, vc, bt[:, :1].contiguous(), torch.tensor([0, 1], dtype=torch.int32, device="cuda"),
                                            torch.tensor([64], dtype=torch.int32, device="cuda"), 0.125)
assert (out.float() - only_first.float()).abs().max() < 1e-2                            # the keys of the bad page did not take part
sm100.clear_kernel_status()
# an engine on the checked build
from nanoengine_b200 import Config, LLM, SamplingParams
llm = LLM(Config(model="tiny-deepseek-v3", dtype="bfloat16", device="cuda", kv_cache_dtype="fp8", kvcache_block_size=64, num_kvcache_blocks=32,
                 max_num_seqs=4, seed=0))
toks = [o["token_ids"] for o in llm.generate([list(range(3, 90)), list(range(7, 30))], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))]
assert sm100.kernel_status()[0] == 0
print("TOKENS", toks)
"""


def _run(env_extra):
    env = dict(os.environ, **env_extra)
    r = subprocess.run([sys.executable, "-c", _SCRIPT if env_extra.get("NE_DEBUG_BOUNDS") == "1" else _PLAIN], env=env, capture_output=True, text=True,
                       timeout=280, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return [l for l in r.stdout.splitlines() if l.startswith("TOKENS")][-1]


_PLAIN = r"""
from nanoengine_b200 import Config, LLM, SamplingParams
llm = LLM(Config(model="tiny-deepseek-v3", dtype="bfloat16", device="cuda", kv_cache_dtype="fp8", kvcache_block_size=64, num_kvcache_blocks=32,
                 max_num_seqs=4, seed=0))
print("TOKENS", [o["token_ids"] for o in llm.generate([list(range(3, 90)), list(range(7, 30))], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))])
"""


def test_checked_build_catches_bad_entries_and_runs_the_engine():
    lib = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "nanoengine_b200", "_native", "libne_kernels_dbg.so")
    if not os.path.exists(lib):
        from nanoengine_b200.build_native import build_kernels
        build_kernels(debug_bounds=True)
    checked = _run({"NE_DEBUG_BOUNDS": "1"})
    plain = _run({"NE_DEBUG_BOUNDS": "0"})
    assert checked == plain
