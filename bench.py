"""Headline benchmark: DeepSeek-V3-shape fp8 MoE serving step (decode tokens/s, plus prefill tokens/s) on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 20 --warmup 5

Workload (weak scaling: per-GPU work is fixed): every GPU serves 128 concurrent requests with 2048-token uniform-random
prompts (synthetic), fp8 e4m3 weights with 128x128 block scales, fp8 paged MLA KV cache (64-token pages), attention
data-parallel and experts expert-parallel over the N GPUs.  The model is the DeepSeek-V3 architecture - 61 layers (3 dense),
hidden 7168, 128 MLA heads, top-8 sigmoid routing with 8 groups / top-4 groups, one shared expert - with 32 routed experts
per GPU, i.e. 256 experts at N = 8 (the named configuration); at smaller N the expert count shrinks with the GPU count,
because the 256-expert model does not fit fewer than 8 GPUs.  Weights are random-init in the HF layout.

One timed "step" is one decode step of the whole job (N x 128 tokens).  `value` is whole-job decode output tokens/s
timed on the device (CUDA events around K graph replays + lm_head + sampling, max over ranks); `e2e` is the same metric
through the public API (LLM.step(): scheduler, H2D of the step inputs from pinned memory, forward, sampling, D2H of the
tokens).  Prefill tokens/s from the prompt phase is reported beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_VALUE = None   # the reference publishes no number for this metric/config


def _clock_sampler(stop, out):
    q = "clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    idx = os.environ.get("LOCAL_RANK", "0")
    while not stop.is_set():
        try:
            r = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", idx], capture_output=True, text=True, timeout=5)
            f = [x.strip() for x in r.stdout.strip().split(",")]
            if len(f) >= 7:
                out.append(f)
        except Exception:
            pass
        stop.wait(0.2)


def _summarise_clocks(samples):
    if not samples:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
    mhz = sorted(int(s[0]) for s in samples if s[0].isdigit())
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in samples)]
    return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": int(samples[0][1]) if samples[0][1].isdigit() else None,
            "reasons": reasons, "samples": len(samples)}


def reference_arm(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference cannot be installed offline: its scheduler and wire protocol are the Rust "
                      "extension dlengine._engine, whose build backend (maturin + a Rust toolchain) is absent, and its DeepSeek-V3 path imports "
                      "deep_gemm, deep_ep and flash_mla, which are not in the image (tvm_ffi, flashinfer, flash_attn, triton and the CUTLASS DSL are)"}))
    return 0


def _fill_random_cache(cache):
    """Random finite e4m3 bytes in the latent pages and the indexer keys, small positive key scales: what a prefill would have
    left, as far as the cost of a decode step goes."""
    import torch
    dev = "cuda" if torch.cuda.is_available() else "cpu"           # generated on the GPU, also for pages that live in host memory
    g = torch.Generator(device=dev).manual_seed(7)

    def rnd_bytes(shape):
        return (torch.randint(0, 0x70, shape, dtype=torch.uint8, generator=g, device=dev)
                | (torch.randint(0, 2, shape, dtype=torch.uint8, generator=g, device=dev) << 7))

    kv = cache.kv.view(torch.uint8)
    for l in range(kv.shape[0]):                                   # layer by layer: the host-side generator buffers stay small
        kv[l].copy_(rnd_bytes(tuple(kv[l].shape)))
    if cache.indexer is not None:
        L, nb, pb = cache.indexer.shape
        D = pb // 64 - 4
        for l in range(L):
            page = torch.empty(nb, pb, dtype=torch.uint8, device=dev)
            page[:, : 64 * D] = rnd_bytes((nb, 64 * D))
            page[:, 64 * D:] = (torch.rand(nb, 64, generator=g, device=dev) * 0.01 + 0.001).view(torch.uint8)
            cache.indexer[l].copy_(page)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="deepseek-v3", choices=["deepseek-v3", "deepseek-v32", "qwen3-235b"],
                    help="deepseek-v3: the headline (fp8, attention-DP + EP); deepseek-v32: the same body with the DSA indexer and sparse "
                         "attention (long-context decode, see --synthetic-context); qwen3-235b: bf16 GQA MoE with tensor-parallel attention + "
                         "EP (the batch is shared by the TP ranks: --seqs-per-gpu is then the size of the whole batch)")
    ap.add_argument("--synthetic-context", action="store_true",
                    help="decode-only: sequences are admitted with --prompt-len tokens of context whose cache rows are random bytes (no "
                         "prefill pass; a 64 x 65,536-token prefill would take minutes).  The decode step does all of its work.")
    ap.add_argument("--hisparse", type=int, default=0, help="with --synthetic-context: hot rows per sequence of the hot / cold cache tier "
                    "(the latent cache then lives in pinned host memory)")
    ap.add_argument("--scale-format", default="ue8m0", choices=["fp32", "ue8m0"],
                    help="fp8 block scales of the DeepSeek shapes: ue8m0 (powers of two, as the V3.1 / V3.2 checkpoints ship them; the tensor cores "
                         "apply them) or fp32 (the original V3 recipe; applied on the CUDA cores)")
    ap.add_argument("--seqs-per-gpu", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=61, help="debug only: anything but 61 marks the result invalid")
    ap.add_argument("--experts-per-gpu", type=int, default=32)
    ap.add_argument("--profile-range", action="store_true",
                    help="bracket the device-timed decode steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    ap.add_argument("--profile-prefill", action="store_true", help="bracket the second prompt step instead")
    ap.add_argument("--mtp", type=int, default=0, help="speculative decoding with this many draft tokens per step (1 MTP layer)")
    ap.add_argument("--force-accept", type=int, default=-1, help="with --mtp: pin the number of accepted drafts per step (random-init "
                    "predictors accept next to nothing on their own)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models.config import deepseek_v3

    N = args.gpus
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != N:
        raise SystemExit(f"--gpus {N} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {N}")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)

    qwen = args.model == "qwen3-235b"
    if qwen:
        from nanoengine_b200.models.config import qwen3_235b
        if args.experts_per_gpu == 32:
            args.experts_per_gpu = 16                    # 128 experts over 8 GPUs
        if args.layers == 61:
            args.layers = 94
        mc = qwen3_235b(n_routed_experts=args.experts_per_gpu * N, num_hidden_layers=args.layers)
    elif args.model == "deepseek-v32":
        from nanoengine_b200.models.config import deepseek_v32
        mc = deepseek_v32(n_routed_experts=args.experts_per_gpu * N, num_hidden_layers=args.layers)
    else:
        mc = deepseek_v3(n_routed_experts=args.experts_per_gpu * N, num_hidden_layers=args.layers, num_nextn_predict_layers=1 if args.mtp else 0)
    S, P = args.seqs_per_gpu, args.prompt_len
    per_step = (args.force_accept + 1) if (args.mtp and args.force_accept >= 0) else 1
    total_new = (args.warmup + args.steps + 8) * per_step + 2 * args.mtp
    pages = (P + total_new + 63) // 64 + 1
    cfg = Config(model=args.model, model_config=mc, dummy_weight=True, dtype="bfloat16", device="cuda", kv_cache_dtype="bfloat16" if qwen else "fp8",
                 max_num_seqs=S, max_num_batched_tokens=16384, max_model_len=P + total_new + 64, num_kvcache_blocks=S * pages + 16,
                 attention_dp=1 if qwen else N, attention_tp=N if qwen else 1, ffn_ep=N, executor_backend="spmd", enable_prefix_caching=False,
                 cuda_graph_max_bs=S, seed=0 if qwen else rank, num_speculative_tokens=args.mtp,
                 mode="decode" if args.synthetic_context else "hybrid", dummy_prefill=args.synthetic_context,
                 fp8_scale_format=args.scale_format, enable_hisparse=args.hisparse > 0, hisparse_device_buffer_size=args.hisparse or 4096,
                 hisparse_host_gb=(S * pages + 16) * 64 * 576 * args.layers / 2 ** 30 + 1)
    t_build = time.time()
    llm = LLM(cfg)
    runner = llm.engine.executor.runner
    if args.synthetic_context:
        _fill_random_cache(runner.cache)
    if args.mtp and args.force_accept >= 0:
        runner.mtp_runner.force_accept = args.force_accept
    build_s = time.time() - t_build

    g = torch.Generator().manual_seed(1234 + (0 if qwen else rank))        # tensor-parallel ranks serve the same requests
    sp = SamplingParams(temperature=0.0, max_tokens=total_new, ignore_eos=True)
    for i in range(S):
        llm.add_request(torch.randint(0, mc.vocab_size, (P,), generator=g).tolist(), sp)

    def sync():
        torch.cuda.synchronize()
        if N > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if N == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- prompt phase: S * P tokens per GPU in steps of 16384 tokens (first step is warm-up and not timed)
    prefill_ms, prefill_tok = 0.0, 0
    first = True
    while llm.engine.scheduler.num_waiting() > 0 or llm.engine.scheduler.num_prefilling(0) > 0:
        sync()
        prof = args.profile_prefill and not first and prefill_tok == 0
        if prof:
            torch.cuda.profiler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.step()
        e1.record()
        e1.synchronize()
        if prof:
            torch.cuda.profiler.stop()
        ntok = llm.engine.scheduler.metrics_summary()["prompt_tokens"]
        if not first:
            prefill_ms += e0.elapsed_time(e1)
            prefill_tok += ntok - prev_tok
        prev_tok = ntok
        first = False
    prefill_ms = max_over_ranks(prefill_ms)

    # ---- decode: warm-up (captures the graph), then K timed steps through the public API
    for _ in range(args.warmup):
        llm.step()
    runner.h2d_bytes = runner.d2h_bytes = 0
    stop, samples = threading.Event(), []
    th = threading.Thread(target=_clock_sampler, args=(stop, samples), daemon=True)
    th.start()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        outs = llm.step()
        assert len(outs) == S, len(outs)
    e1.record()
    e1.synchronize()
    sync()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    h2d, d2h = runner.h2d_bytes // args.steps, runner.d2h_bytes // args.steps

    # ---- device-timed: replay the same decode step (graph + lm_head + sampling) K times on resident inputs.
    # Each step streams the full weight set (~100 GB), far beyond the 126 MB L2, so no cache flush is needed between steps.
    if args.mtp:
        launches = runner.mtp_runner.count_step_launches()
        step_fn = runner.mtp_runner.make_resident_step()
        graph_ok = None
    else:
        graph_ok = runner.graph_step_equals_eager()      # outside the timed region: the replayed step samples what an eager step samples
        launches = runner.count_step_launches()
        step_fn = runner.make_resident_decode_step()
    for _ in range(3):
        step_fn()
    sync()
    if args.profile_range:
        torch.cuda.profiler.start()
    e0.record()
    for _ in range(args.steps):
        step_fn()
    e1.record()
    e1.synchronize()
    if args.profile_range:
        torch.cuda.profiler.stop()
    sync()
    dev_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    stop.set()
    th.join(timeout=2)

    if rank == 0:
        tokens_per_step = S * (1 if qwen else N) * per_step
        value = tokens_per_step / (dev_ms * 1e-3)
        out = {
            "metric": "decode out tok/s (whole job; per-GPU = value / n_gpus) at TPOT = ms_per_step; prefill tok/s beside it",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": N, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None if BASELINE_VALUE is None else value / BASELINE_VALUE,
            "dtype": "bf16" if qwen else "fp8 weights + fp8 KV, bf16 activations",
            "data": ("synthetic: random cache rows standing in for the prompts (no prefill pass), random-init weights (HF layout)"
                     if args.synthetic_context else "synthetic uniform-random token ids, random-init weights (HF layout)"),
            "config": {"model": (f"Qwen3-235B-A22B shape: {args.layers} layers, hidden 4096, 64/4 GQA heads, {args.experts_per_gpu * N} experts "
                                 f"({args.experts_per_gpu}/GPU) top-8, bf16") if qwen else
                                (f"DeepSeek-{'V3.2 (DSA top-2048' + (', hot / cold tier ' + str(args.hisparse) + ' rows' if args.hisparse else '') + ')' if args.model == 'deepseek-v32' else 'V3'} shape: {args.layers} layers, hidden 7168, 128 MLA heads, {args.experts_per_gpu * N} routed experts "
                                 f"({args.experts_per_gpu}/GPU) top-8, 1 shared"), "global_batch": tokens_per_step, "seq_len": P,
                       "parallelism": f"tp{N} attention + ep{N} experts" if qwen else f"dp{N} attention + ep{N} experts",
                       "fp8_scale_format": None if qwen else args.scale_format,
                       "l2": "inputs (the weights streamed every step) exceed L2; no flush",
                       "valid": (args.layers == 94 and args.experts_per_gpu == 16) if qwen else (args.layers == 61 and args.experts_per_gpu == 32 and (S == 128 or args.model == "deepseek-v32"))},
            "decode_tok_s_per_gpu": round(value / N, 1), "tpot_ms": round(dev_ms, 3), "tpot_slo_50ms_met": dev_ms <= 50.0,
            "prefill_tok_s": round(prefill_tok * (1 if qwen else N) / (prefill_ms * 1e-3), 1) if prefill_ms > 0 else None,
            "prefill_tok_s_per_gpu": round(prefill_tok / (N if qwen else 1) / (prefill_ms * 1e-3), 1) if prefill_ms > 0 else None,
            "e2e": {"value": round(tokens_per_step / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 3),
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches * args.steps), "launches_per_step": int(launches),
            "clocks": _summarise_clocks(samples), "build_s": round(build_s, 1), "impl": "ours", "graph_equals_eager": graph_ok,
            "mtp": None if not args.mtp else {"draft_tokens": args.mtp, "forced_accept": args.force_accept, "tokens_per_seq_per_step": per_step,
                                             "accepted_per_verify": round(runner.mtp_runner.accepted_total / max(1, runner.mtp_runner.verify_steps), 3)},
        }
        print(json.dumps(out))
    if N > 1:
        dist.barrier()
    llm.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
