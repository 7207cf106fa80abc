"""Table of a working-set matrix directory written by ``run_working_set_matrix.py``: per cell
TTFT p50 / p99, end-to-end p50 / p99, recomputed prompt tokens, output tokens/s, resident media
and evictions (the columns of the reference's ``benchmarks/summarize_working_set.py:81-334``).

    python benchmarks/summarize_working_set.py results/ws [--markdown]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200.analysis import benchmark_schema  # noqa: E402

COLUMNS = ("ttft_p50_ms", "ttft_p99_ms", "e2e_p50_ms", "e2e_p99_ms", "recomputed_prompt_tokens", "output_tokens_per_s",
           "resident_media", "prefix_evictions")


def load_cells(directory: str) -> dict[str, dict]:
    cells = {}
    for name in sorted(os.listdir(directory)):
        if not name.endswith(".json"):
            continue
        with open(os.path.join(directory, name)) as fh:
            rec = json.load(fh)
        benchmark_schema.validate_benchmark_record(rec)
        cells[name[:-5]] = rec
    return cells


def summary_rows(cells: dict[str, dict]) -> list[dict]:
    rows = []
    for name, rec in cells.items():
        result = rec.get("results", rec)
        ws, _, variant = name.partition("__")
        row = {"working_set": ws, "variant": variant}
        for col in COLUMNS:
            row[col] = result.get(col)
        rows.append(row)
    return rows


def to_markdown(rows: list[dict]) -> str:
    head = ["working_set", "variant", *COLUMNS]
    lines = ["| " + " | ".join(head) + " |", "|" + "---|" * len(head)]
    for r in rows:
        cells = []
        for h in head:
            v = r.get(h)
            cells.append(f"{v:.1f}" if isinstance(v, float) else str(v))
        lines.append("| " + " | ".join(cells) + " |")
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("directory")
    ap.add_argument("--markdown", action="store_true")
    args = ap.parse_args()
    rows = summary_rows(load_cells(args.directory))
    print(to_markdown(rows) if args.markdown else json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
