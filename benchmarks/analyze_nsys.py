"""Summarise an Nsight Systems SQLite export of an engine run (reference
``benchmarks/analyze_nsys.py``): per engine step and per named NVTX range the kernel count and
time, graph execution time, runtime API counts, copies, GPU busy time and the launch-to-kernel
gap; the kernels of the whole capture grouped by name.

Capture on a machine that has Nsight Systems, e.g.

    nsys profile --trace=cuda,nvtx --capture-range=cudaProfilerApi -o capture \
        python benchmarks/trace_prefix_hit.py --out trace.json
    nsys export --type sqlite capture.nsys-rep

then, anywhere:

    python benchmarks/analyze_nsys.py capture.sqlite --prefill-steps 1 \
        --target-range prism::runner.run_model --output summary.json
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200.analysis.nsys_trace import analyze_nsys_sqlite  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("sqlite")
    ap.add_argument("--engine-range", default="prism::engine.step")
    ap.add_argument("--prefill-steps", type=int, default=1)
    ap.add_argument("--target-range", action="append", default=[])
    ap.add_argument("--top", type=int, default=20)
    ap.add_argument("--output")
    ap.add_argument("--quiet", action="store_true", help="write --output without printing the summary")
    args = ap.parse_args()
    result = analyze_nsys_sqlite(args.sqlite, engine_range=args.engine_range, prefill_steps=args.prefill_steps,
                                 target_ranges=args.target_range, top=args.top)
    text = json.dumps(result, indent=2, sort_keys=True)
    if args.output:
        out = Path(args.output)
        if out.exists():
            raise FileExistsError(f"refusing to overwrite {out}")
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(text + "\n", encoding="utf-8")
    if not args.quiet:
        print(text)


if __name__ == "__main__":
    main()
