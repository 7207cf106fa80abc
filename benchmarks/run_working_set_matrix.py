"""Working-set study matrix: {fit, knee, pressure} working sets x {vision_only, dense_prefix,
compact_prefix} cache variants, one ``bench_online.py`` process per cell (mirrors the
reference's ``benchmarks/run_working_set_matrix.py:92-233``).

A cell's result file is written by the child through a temporary name and renamed, so a file
that exists is complete.  ``--resume`` validates finished cells against the benchmark schema
and skips them; an interrupted cell (temporary or invalid file) is archived under
``<out>/interrupted/`` and run again.

    python benchmarks/run_working_set_matrix.py --out results/ws [--resume] [--tp 1] [--requests 600]
    python benchmarks/summarize_working_set.py results/ws
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from prism_infer_b200.analysis import benchmark_schema  # noqa: E402

# working sets as (groups, min images, max images): dense pages needed against the 220-page budget
WORKING_SETS = {
    "fit": dict(groups=21, min_images=1, max_images=8),        # about 70% of the budget
    "knee": dict(groups=42, min_images=1, max_images=8),       # at the budget
    "pressure": dict(groups=42, min_images=7, max_images=8),   # about 150% of the budget
}
VARIANTS = ("vision_only", "dense_prefix", "compact_prefix")


def cell_name(ws: str, variant: str) -> str:
    return f"{ws}__{variant}"


def cell_is_complete(path: str) -> bool:
    try:
        with open(path) as fh:
            rec = json.load(fh)
        benchmark_schema.validate_benchmark_record(rec)
        return True
    except Exception:
        return False


def plan_cells(out_dir: str, resume: bool, only: list[str]) -> list[tuple[str, str, str]]:
    """(working set, variant, result path) of the cells that still have to run."""
    todo = []
    for ws in WORKING_SETS:
        for variant in VARIANTS:
            name = cell_name(ws, variant)
            if only and name not in only and ws not in only and variant not in only:
                continue
            path = os.path.join(out_dir, name + ".json")
            if os.path.exists(path) or os.path.exists(path + ".tmp"):
                if resume and cell_is_complete(path):
                    continue
                archive = os.path.join(out_dir, "interrupted")
                os.makedirs(archive, exist_ok=True)
                for p in (path, path + ".tmp"):
                    if os.path.exists(p):
                        shutil.move(p, os.path.join(archive, f"{int(time.time())}_{os.path.basename(p)}"))
            todo.append((ws, variant, path))
    return todo


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--only", nargs="*", default=[], help="cell, working-set or variant names")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--requests", type=int, default=600)
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--pages", type=int, default=220)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--image-size", type=int, default=448)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    todo = plan_cells(args.out, args.resume, args.only)
    print(json.dumps({"cells_to_run": [cell_name(w, v) for w, v, _ in todo]}), flush=True)
    if args.dry_run:
        return
    for ws, variant, path in todo:
        spec = WORKING_SETS[ws]
        cmd = [sys.executable, os.path.join(ROOT, "benchmarks", "bench_online.py"), "--variant", variant, "--model", args.model,
               "--groups", str(spec["groups"]), "--min-images", str(spec["min_images"]), "--max-images", str(spec["max_images"]),
               "--requests", str(args.requests), "--rate", str(args.rate), "--pages", str(args.pages), "--tp", str(args.tp),
               "--image-size", str(args.image_size), "--out", path + ".tmp"]
        if args.tp > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.tp}",
                   "--master-addr", "127.0.0.1"] + cmd[1:]
        t0 = time.time()
        rc = subprocess.call(cmd)
        if rc != 0 or not cell_is_complete(path + ".tmp"):
            print(json.dumps({"cell": cell_name(ws, variant), "status": "failed", "returncode": rc}), flush=True)
            continue
        os.replace(path + ".tmp", path)
        print(json.dumps({"cell": cell_name(ws, variant), "status": "done", "seconds": round(time.time() - t0, 1)}), flush=True)


if __name__ == "__main__":
    main()
