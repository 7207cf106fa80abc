"""Minimal use of the public API with a random-init tiny model (no checkpoint needed):

    python example.py            # CPU
    python example.py --cuda     # B200, CUDA-graph decode, scaled-FP8 KV
"""

import sys

import numpy as np

from prism_infer_b200 import LLM, SamplingParams


def main() -> None:
    cuda = "--cuda" in sys.argv
    llm = LLM("random:tiny", max_model_len=512, kvcache_block_size=256 if cuda else 16, num_kvcache_blocks=32,
              compression_mode="scaled_fp8_kv" if cuda else "off", enforce_eager=not cuda,
              **({} if cuda else {"device": "cpu"}))
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    print(llm.generate(["12 34 56 78"], sp)[0])
    image = np.random.default_rng(0).integers(0, 256, (224, 224, 3), dtype=np.uint8)
    print(llm.generate_vl("1 2 3", image, sp))
    print(llm.generate_video("4 5 6", [image] * 4, sp))
    print(llm.multimodal_prefix_cache_metadata())
    llm.exit()


if __name__ == "__main__":
    main()
