"""Prefill / decode disaggregation with both engines in this process: the prompts are prefilled on one engine, their cache pages
move to the other (a peer-store push between GPUs, a copy between CPU engines), and decoding continues there.

    python examples/disagg.py
    python examples/disagg.py --model /models/DeepSeek-V3 --prefill_device cuda:0 --decode_device cuda:1

Parity: reference examples/disagg.py (prefill.generate(return_serialized=True) -> RequestMigrate blobs ->
decode.add_request_payload -> prefill.free_to_be_migrated_ids)."""
import sys

from _common import base_parser, config_kwargs, encode_prompts


def main(argv=None) -> int:
    ap = base_parser(__doc__)
    ap.add_argument("--prefill_device", default=None, help="e.g. cuda:0 (default: the --device choice)")
    ap.add_argument("--decode_device", default=None, help="e.g. cuda:1")
    args = ap.parse_args(argv)
    from nanoengine_b200 import Config, LLM, RequestMigrate, SamplingParams
    from nanoengine_b200.parallel.kv_transfer import connect_inproc
    pre_cfg = Config(**config_kwargs(args, mode="prefill", engine_id="prefill-0"))
    dec_cfg = Config(**config_kwargs(args, mode="decode", engine_id="decode-0"))
    prompts, ids, tok = encode_prompts(args, pre_cfg)
    prefill, decode = LLM(pre_cfg), LLM(dec_cfg)
    connect_inproc(prefill.engine, decode.engine)        # the decode side publishes its page pool, the prefill side opens it
    sp = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    blobs = prefill.generate(ids, sp, return_serialized=True)
    firsts = {}
    for blob in blobs:
        seq_id, first_token = RequestMigrate.from_bytes(blob).metadata
        firsts[seq_id] = first_token
        decode.add_request_payload(blob)
    outs = {o["seq_id"]: [firsts[o["seq_id"]]] + o["token_ids"] for o in decode.generate()}
    prefill.free_to_be_migrated_ids(list(firsts))         # the prefill engine may reuse the pages now
    for (seq_id, toks), text in zip(sorted(outs.items()), prompts):
        print(f"[{seq_id}] {text!r} -> {tok.decode(toks)!r}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
