"""Open-loop serving benchmark: Poisson arrivals into the engine, p50 / p99 TTFT and TPOT, output tokens per second.

    python benchmarks/serving_bench.py --model deepseek-v3 --layers 61 --rate 8 --requests 64 --prompt-len 2048 --out-len 64
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29544 \\
        benchmarks/serving_bench.py --gpus 8 ...            # one engine per GPU (attention DP + EP), one arrival stream per rank

Requests (synthetic token ids, random-init weights) arrive on a Poisson clock of `--rate` requests per second per GPU and
are handed to the engine's public API (`LLM.add_request` / `LLM.step`) when due; the loop never waits for a request to
finish before admitting the next, so queueing shows up in TTFT.  TTFT = arrival -> first generated token, TPOT = mean gap
between a request's later tokens; both on the host clock (this is an end-to-end figure; kernel timings live in bench.py).
Rank 0 prints one JSON line with the whole-job figures.

Parity: the reference measures serving with an external OpenAI client against `dlengine serve`
(bench/k3_partition/results/gb200_full_serving/result.json: TTFT, mean TPOT per prompt length).
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pct(xs, p):
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(p / 100.0 * len(xs)))]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--model", default="deepseek-v3")
    ap.add_argument("--layers", type=int, default=61)
    ap.add_argument("--experts-per-gpu", type=int, default=32)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--rate", type=float, default=8.0, help="arrivals per second per GPU")
    ap.add_argument("--requests", type=int, default=64, help="requests per GPU")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--out-len", type=int, default=64)
    ap.add_argument("--max-num-seqs", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--scale-format", default="ue8m0", choices=["fp32", "ue8m0"], help="fp8 block scales (see bench.py)")
    args = ap.parse_args()

    import torch
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.models.config import PRESETS
    from nanoengine_b200._native import _core as C

    N = args.gpus
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != N:
        raise SystemExit(f"--gpus {N} but WORLD_SIZE={world}")
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    over = {"num_hidden_layers": args.layers}
    if args.model.startswith("deepseek"):
        over.update(n_routed_experts=args.experts_per_gpu * N, num_nextn_predict_layers=0)
    mc = PRESETS[args.model](**over) if args.model != "tiny-deepseek-v3" else PRESETS[args.model]()
    P, O, S = args.prompt_len, args.out_len, args.max_num_seqs
    pages = (P + O + 63) // 64 + 1
    kw = dict(model=args.model, model_config=mc, dummy_weight=True, device=args.device, max_num_seqs=S,
              max_model_len=P + O + 64, enable_prefix_caching=False, seed=rank)
    if cuda:
        kw.update(dtype="bfloat16", kv_cache_dtype="fp8", fp8_scale_format=args.scale_format, max_num_batched_tokens=16384, num_kvcache_blocks=S * pages + 16,
                  attention_dp=N, ffn_ep=N, executor_backend="spmd" if N > 1 else "inproc", cuda_graph_max_bs=S)
    else:
        kw.update(dtype="float32", kvcache_block_size=16, num_kvcache_blocks=max(64, S * ((P + O) // 16 + 2)))
    llm = LLM(Config(**kw))

    rng = random.Random(args.seed + rank)
    g = torch.Generator().manual_seed(args.seed + rank)
    arrivals, t = [], 0.0
    for _ in range(args.requests):
        t += rng.expovariate(args.rate)
        arrivals.append(t)
    prompts = [torch.randint(0, mc.vocab_size, (P,), generator=g).tolist() for _ in range(args.requests)]
    sp = SamplingParams(temperature=0.0, max_tokens=O, ignore_eos=True)

    # one throw-away request warms the kernels and captures the decode graphs
    llm.add_request(prompts[0], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    while not llm.engine.is_finished():
        llm.step()
    if N > 1:
        torch.distributed.barrier()

    t0 = time.perf_counter()
    due, born, first, last, count, gaps = 0, {}, {}, {}, {}, {}
    done = 0
    flag = torch.zeros(1, dtype=torch.int32)
    while True:
        if N > 1:
            # every rank keeps stepping (idle ranks run the dummy batches the expert all-to-all needs) until all are done
            flag[0] = int(done < args.requests)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX)
            if int(flag[0]) == 0:
                break
        elif done >= args.requests:
            break
        now = time.perf_counter() - t0
        while due < args.requests and arrivals[due] <= now:
            sid = llm.add_request(prompts[due], sp)
            born[sid] = t0 + arrivals[due]
            due += 1
        outs = llm.step()
        tnow = time.perf_counter()
        for o in outs:
            sid = o.seq_id
            if sid not in born:
                continue
            n_new = len(o.token_ids)
            if sid not in first:
                first[sid] = tnow
                count[sid] = 0
                gaps[sid] = []
            else:
                gaps[sid].append((tnow - last[sid]) / max(n_new, 1))
            last[sid] = tnow
            count[sid] += n_new
            if o.status == C.FINISHED:
                done += 1
        if not outs and due < args.requests and N == 1:
            time.sleep(min(0.002, max(0.0, arrivals[due] - (time.perf_counter() - t0))))
    wall = time.perf_counter() - t0
    ttft = [(first[s] - born[s]) * 1e3 for s in first]
    tpot = [sum(v) / len(v) * 1e3 for v in gaps.values() if v]
    tokens = sum(count.values())
    if N > 1:
        import torch.distributed as dist
        obj = [None] * N
        dist.all_gather_object(obj, (ttft, tpot, tokens, wall))
        ttft = [x for o in obj for x in o[0]]
        tpot = [x for o in obj for x in o[1]]
        tokens = sum(o[2] for o in obj)
        wall = max(o[3] for o in obj)
    if rank == 0:
        print(json.dumps({"bench": "serving", "n_gpus": N, "model": args.model, "layers": args.layers, "rate_per_gpu": args.rate,
                          "requests": args.requests * N, "prompt_len": P, "out_len": O,
                          "ttft_ms_p50": round(pct(ttft, 50), 2), "ttft_ms_p99": round(pct(ttft, 99), 2),
                          "tpot_ms_p50": round(pct(tpot, 50), 3) if tpot else None, "tpot_ms_p99": round(pct(tpot, 99), 3) if tpot else None,
                          "out_tok_s": round(tokens / wall, 1), "wall_s": round(wall, 2), "data": "synthetic, random-init weights"}))
    llm.shutdown()


if __name__ == "__main__":
    main()
