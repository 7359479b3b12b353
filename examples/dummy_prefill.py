"""A decode-only engine fed with requests whose context was never prefilled: the engine admits each prompt as if its cache pages
had arrived from a prefill engine (`dummy_prefill=True`) and starts decoding at once.  Used to load a decode deployment at a
chosen context length without paying for the prefill.

    python examples/dummy_prefill.py --context 512 --max_tokens 16

Parity: reference examples/dummy_prefill.py, dummy_engine.py."""
import sys
import time

import torch

from _common import base_parser, config_kwargs


def main(argv=None) -> int:
    ap = base_parser(__doc__)
    ap.add_argument("--context", type=int, default=256, help="tokens of (never computed) context per sequence")
    ap.add_argument("--num_requests", type=int, default=4)
    args = ap.parse_args(argv)
    from nanoengine_b200 import Config, LLM, SamplingParams
    config = Config(**config_kwargs(args, mode="decode", dummy_prefill=True, dummy_weight=True,
                                    max_model_len=args.context + args.max_tokens + 64))
    llm = LLM(config)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, ignore_eos=True)
    for _ in range(args.num_requests):
        llm.add_request(torch.randint(0, config.model_config.vocab_size, (args.context,), generator=g).tolist(), sp)
    t0 = time.time()
    outs = llm.generate()
    dt = time.time() - t0
    n = sum(len(o["token_ids"]) for o in outs)
    print(f"{len(outs)} sequences x {args.context} tokens of context: {n} tokens in {dt:.2f} s ({n / dt:.1f} tok/s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
