"""Open-loop HTTP load generator for the OpenAI-compatible server (or the gateway in front of several engines): Poisson arrivals,
streamed chat completions, time to first token and time per output token as the client sees them.

    python -m nanoengine_b200.server.cli serve tiny-deepseek-v3 --device cpu --dtype float32 --port 8000 &
    python examples/bench_serving.py --url http://127.0.0.1:8000 --rate 4 --requests 32 --prompt_len 64 --max_tokens 32

`--self_host` starts a tiny CPU engine and the HTTP app on a free local port inside this process, which is what the example's test uses.
Parity: reference examples/bench_serving.py, mixed_dataset.py (prompt length mixes)."""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import random
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_prompts(n: int, prompt_len: str, seed: int):
    """`prompt_len`: one length, or a mix "len:weight,len:weight" (e.g. 128:3,2048:1); lengths count words of filler text."""
    rng = random.Random(seed)
    mix = []
    for part in str(prompt_len).split(","):
        ln, _, w = part.partition(":")
        mix.append((int(ln), float(w or 1)))
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta"]
    out = []
    for _ in range(n):
        ln = rng.choices([m[0] for m in mix], [m[1] for m in mix])[0]
        out.append(" ".join(rng.choice(words) for _ in range(ln)))
    return out


async def one_request(post_stream, model: str, prompt: str, max_tokens: int, rec: dict):
    body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens, "temperature": 0.0,
            "stream": True, "ignore_eos": True}
    t0 = time.perf_counter()
    stamps = []
    async for line in post_stream("/v1/chat/completions", body):
        if not line.startswith("data:") or line.strip() == "data: [DONE]":
            continue
        delta = json.loads(line[5:])["choices"][0].get("delta", {})
        if delta.get("content") is not None or delta.get("tool_calls"):
            stamps.append(time.perf_counter())
    rec["ttft"] = (stamps[0] - t0) if stamps else float("nan")
    rec["tpot"] = ((stamps[-1] - stamps[0]) / (len(stamps) - 1)) if len(stamps) > 1 else float("nan")
    rec["chunks"] = len(stamps)
    rec["e2e"] = time.perf_counter() - t0


def http_poster(url: str):
    import aiohttp
    session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None))

    async def post_stream(path, body):
        async with session.post(url.rstrip("/") + path, json=body) as resp:
            resp.raise_for_status()
            async for raw in resp.content:
                yield raw.decode("utf-8", "replace").strip()

    return post_stream, session.close


def self_hosted(model: str):
    """A tiny CPU engine (its own process) behind the HTTP app, served by uvicorn on a free local port in a thread of this process.
    Returns the URL and a function that shuts both down."""
    import socket
    import threading
    import uvicorn
    from nanoengine_b200 import Config
    from nanoengine_b200.server.engine_server import EngineClient, spawn_backend
    from nanoengine_b200.server.openai_server import create_app
    from nanoengine_b200.server.tokenizer import load_tokenizer
    cfg = Config(model=model, dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=256)
    proc, endpoint = spawn_backend(cfg)
    engine = EngineClient(endpoint, proc)
    app = create_app(engine, load_tokenizer(cfg.model, cfg.model_config.vocab_size), model)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    t0 = time.time()
    while not server.started and time.time() - t0 < 30:
        time.sleep(0.05)

    def stop():
        server.should_exit = True
        th.join(timeout=10)
        engine.destroy()
        if proc.is_alive():
            proc.terminate()
        proc.join(timeout=10)

    return f"http://127.0.0.1:{port}", stop


async def run(args) -> dict:
    stop = None
    if args.self_host:
        args.url, stop = self_hosted(args.model)
    post_stream, close = http_poster(args.url)
    prompts = make_prompts(args.requests, args.prompt_len, args.seed)
    rng = random.Random(args.seed + 1)
    recs, tasks = [], []
    t0 = time.perf_counter()
    try:
        for p in prompts:
            rec = {}
            recs.append(rec)
            tasks.append(asyncio.create_task(one_request(post_stream, args.model, p, args.max_tokens, rec)))
            if args.rate > 0:
                await asyncio.sleep(rng.expovariate(args.rate))
        await asyncio.gather(*tasks)
    finally:
        await close()
        if stop is not None:
            stop()
    wall = time.perf_counter() - t0

    def pct(xs, q):
        xs = sorted(x for x in xs if x == x)
        return xs[min(len(xs) - 1, int(q * len(xs)))] * 1e3 if xs else float("nan")

    ttft, tpot = [r["ttft"] for r in recs], [r["tpot"] for r in recs]
    return {"requests": len(recs), "rate": args.rate, "wall_s": round(wall, 2), "ttft_ms_p50": round(pct(ttft, 0.5), 1),
            "ttft_ms_p99": round(pct(ttft, 0.99), 1), "tpot_ms_p50": round(pct(tpot, 0.5), 2), "tpot_ms_p99": round(pct(tpot, 0.99), 2),
            "chunks_per_request": round(statistics.mean(r["chunks"] for r in recs), 1),
            "requests_per_s": round(len(recs) / wall, 2)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--self_host", action="store_true")
    ap.add_argument("--model", default="tiny-deepseek-v3")
    ap.add_argument("--rate", type=float, default=4.0, help="arrivals per second (0 = all at once)")
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--prompt_len", default="32", help='words per prompt, or a mix such as "32:3,512:1"')
    ap.add_argument("--max_tokens", type=int, default=16)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    print(json.dumps(asyncio.run(run(args))))
    return 0


if __name__ == "__main__":
    sys.exit(main())
