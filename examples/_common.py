"""Shared argument handling of the examples: a checkpoint directory, or a preset shape with random weights (`--dummy`)."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))      # run from a source tree without installing

import torch  # noqa: E402


def base_parser(description: str) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--model", default="tiny-deepseek-v3", help="checkpoint directory (HF layout) or a preset name (random weights)")
    ap.add_argument("--device", default="auto", choices=["auto", "cuda", "cpu"])
    ap.add_argument("--dtype", default=None, help="bfloat16 on a GPU, float32 on the CPU unless given")
    ap.add_argument("--kvcache_block_size", type=int, default=None)
    ap.add_argument("--num_kvcache_blocks", type=int, default=None)
    ap.add_argument("--max_num_seqs", type=int, default=8)
    ap.add_argument("--attention_dp", type=int, default=1)
    ap.add_argument("--attention_tp", type=int, default=1)
    ap.add_argument("--ffn_ep", type=int, default=1)
    ap.add_argument("--num_speculative_tokens", type=int, default=0)
    ap.add_argument("--max_tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--ignore_eos", action="store_true")
    ap.add_argument("--prompt", action="append", help="may be given several times")
    return ap


def config_kwargs(args, **extra) -> dict:
    cuda = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
    kw = dict(model=args.model, device="cuda" if cuda else "cpu", dtype=args.dtype or ("bfloat16" if cuda else "float32"),
              max_num_seqs=args.max_num_seqs, attention_dp=args.attention_dp, attention_tp=args.attention_tp, ffn_ep=args.ffn_ep,
              num_speculative_tokens=args.num_speculative_tokens)
    kw["kvcache_block_size"] = args.kvcache_block_size or (64 if cuda else 16)
    if args.num_kvcache_blocks or not cuda:
        kw["num_kvcache_blocks"] = args.num_kvcache_blocks or 256
    if args.num_speculative_tokens:
        kw["hf_overrides"] = {"num_nextn_predict_layers": 1}
    kw.update(extra)
    return kw


def encode_prompts(args, config):
    """Token ids of the prompts (through the chat template when the tokenizer has one) and the tokenizer."""
    from nanoengine_b200.server.tokenizer import load_tokenizer
    tok = load_tokenizer(config.model, config.model_config.vocab_size)
    prompts = args.prompt or ["What is 1+1?", "Name three prime numbers."]
    ids = [tok.apply_chat_template([{"role": "user", "content": p}]) for p in prompts]
    return prompts, ids, tok
