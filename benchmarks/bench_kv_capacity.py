"""KV capacity accounting: bytes per page and token capacity for bf16 versus scaled-FP8
pages at a byte budget (the reference's ``bench_kv_capacity.py`` and ``docs/RESULTS.md:128-137``:
4 068.000 -> 2 097.562 MiB for 113 pages, 28 928 -> 56 320 tokens at about 4 GiB)."""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200.config import Config  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--budget-bytes", type=int, default=4_282_122_240)
    ap.add_argument("--tp", type=int, default=1)
    args = ap.parse_args()
    out = {}
    for mode in ("off", "fp8_kv", "scaled_fp8_kv"):
        cfg = Config("random:qwen3-vl-8b", compression_mode=mode, tensor_parallel_size=args.tp)
        per = cfg.kv_bytes_per_page() * args.tp
        pages = args.budget_bytes // per
        out[mode] = {"bytes_per_page": per, "pages": pages, "tokens": pages * 256, "mib_for_113_pages": 113 * per / 2**20}
    out["scaled_over_bf16_bytes"] = out["scaled_fp8_kv"]["bytes_per_page"] / out["off"]["bytes_per_page"]
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
