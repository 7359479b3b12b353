"""Offline generation on one engine (prefill and decode in the same process group).

    python examples/non_disagg.py                                   # tiny random-weight model, CPU or GPU
    python examples/non_disagg.py --model /models/DeepSeek-V3 --attention_dp 8 --ffn_ep 8 --max_tokens 64

Parity: reference examples/non_disagg.py (Config -> LLM -> RequestIn payloads -> offline.generate)."""
import sys

from _common import base_parser, config_kwargs, encode_prompts


def main(argv=None) -> int:
    args = base_parser(__doc__).parse_args(argv)
    from nanoengine_b200 import Config, LLM, RequestIn, SamplingParams
    from nanoengine_b200.offline import generate
    config = Config(**config_kwargs(args))
    prompts, ids, tok = encode_prompts(args, config)
    llm = LLM(config)
    sp = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    for i, p in enumerate(ids):
        llm.add_request_payload(RequestIn(i + 1, p, sp).to_bytes())          # the wire form a server would hand the engine
    done = {}
    for out in generate(llm):                                                # yields as sequences finish
        done[out["seq_id"]] = out["token_ids"]
    for i, text in enumerate(prompts):
        print(f"[{i + 1}] {text!r} -> {tok.decode(done[i + 1])!r}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
