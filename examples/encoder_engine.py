"""A vision encoder engine feeding a language-model engine: images are encoded once into a pool of embedding slots, the language
model reads the rows in place of its image tokens.

    python examples/encoder_engine.py                      # tiny random-weight encoder and language model, CPU or GPU

The encoder here runs in this process; `python -m nanoengine_b200.server.cli serve-encoder ...` runs it as a service that
engines reach over ZMQ (`nanoengine_b200.vl.encoder_engine.EncoderClient`).
Parity: reference examples/test_encoder_engine.py, test_vl.py."""
import sys

from _common import base_parser, config_kwargs

import torch


def main(argv=None) -> int:
    ap = base_parser(__doc__)
    ap.add_argument("--image_token_id", type=int, default=7)
    args = ap.parse_args(argv)
    from nanoengine_b200 import Config, LLM, SamplingParams
    from nanoengine_b200.vl import EncoderConfig, EncoderEngine, VisionConfig
    kw = config_kwargs(args, enable_prefix_caching=False)
    config = Config(**kw)
    H = config.model_config.hidden_size
    vc = VisionConfig(hidden_size=64, num_heads=4, depth=2, intermediate_size=96, out_hidden_size=H, in_channels=3, patch_size=4,
                      temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=64)
    enc = EncoderEngine(EncoderConfig(vision_config=vc, device=kw["device"], dtype=kw["dtype"], num_slots=4, max_tokens_per_slot=64))
    try:
        # two images of 4 x 6 and 4 x 4 patches: (4*6 + 4*4) / (2*2 merge) = 10 embedding rows
        grids = [(1, 4, 6), (1, 4, 4)]
        patches = torch.randn(sum(t * h * w for t, h, w in grids), vc.patch_dim)
        slot = enc.encode(patches, grids)
        print(f"encoded {len(grids)} images into slot {slot.slot}: {slot.num_tokens} rows of width {slot.hidden_size}")
        img = args.image_token_id
        prompt = [3, 11] + [img] * 6 + [25, 99] + [img] * 4 + [14, 15, 16]
        llm = LLM(config)
        sp = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, ignore_eos=True)
        llm.engine.add_vision_request(prompt, img, vision_slot=slot, pool_desc=enc.pool.export(direct=True), sampling_params=sp)
        out = llm.generate()[0]
        print(f"generated {len(out['token_ids'])} tokens: {out['token_ids']}")
        enc.pool.free(slot.slot)
    finally:
        enc.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
