"""Select the MVBench questions that share their video with at least one other question: the
repeated-visual-context subset of the video quality runs (reference: ``scripts/build_mvbench_repeated_subset.py``).

Reads the dataset's task JSON files and a media map, writes (into a new directory) the selected question
records in selection order, a manifest with one entry per media group, and the sample-id list.  Media stay
pending; ``materialize_mvbench_media`` extracts them.

    python -m prism_infer_b200.utils.build_mvbench_repeated_subset --json-dir raw/mvbench/json \
        --media-map mvbench_media_map.json --out data/quality/mvbench_repeated [--revision <dataset revision>]
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Any

from ..analysis import mvbench
from ..analysis import quality_materialization as qm
from ..analysis.identity import canonical_json_sha256

ALGORITHM = "all_exact_mvbench_source_contract_groups"


def build(*, json_dir: str | Path, media_map_path: str | Path, out_root: str | Path, revision: str | None = None) -> dict[str, Any]:
    out = Path(out_root)
    if out.exists():
        raise FileExistsError(f"output directory already exists: {out}")
    media_map = mvbench.MediaMap.load(media_map_path)
    if revision is not None and revision != media_map.revision:
        raise ValueError(f"media map describes revision {media_map.revision!r}, asked for {revision!r}")
    population = mvbench.Population.load(json_dir, media_map)
    records, groups = mvbench.repeated_media_groups([population.records[s] for s in population.sample_ids])
    ids = tuple(str(r["sample_id"]) for r in records)
    selection = qm.SampleSelection(len(population.sample_ids), ids, ids)
    out.mkdir(parents=True)
    records_path = out / f"{mvbench.DATASET_ID}.records.jsonl"
    records_sha = qm.write_jsonl_atomic(records_path, records)
    manifest = {
        "schema_version": qm.MATERIALIZATION_SCHEMA_VERSION, "record_type": "quality_materialization", "dataset_id": mvbench.DATASET_ID,
        "revision": media_map.revision, "media_map_sha256": media_map.sha256,
        "selection": {"algorithm": ALGORITHM, "group_preimage": "canonical JSON of archive name / path, member path, media type, time window",
                      "group_order": "source_contract_sha256 ascending", "within_group_order": "task, question index, sample id",
                      **selection.to_record()},
        "repeated_media": {"groups": len(groups), "samples": len(records), "group_records": groups,
                           "group_ids_sha256": canonical_json_sha256([g["source_contract_sha256"] for g in groups])},
        "records_file": {"path": records_path.name, "sha256": records_sha},
        "records_sha256": canonical_json_sha256(records),
        "source_files": [{"name": p.name, "bytes": p.stat().st_size, "sha256": qm.sha256_file(p)} for p in population.source_files],
        "evaluation_subset": mvbench.evaluation_subset(records), "pending_media_plan": mvbench.pending_plan(records),
        "materialization_status": "media_materialization_pending",
    }
    qm.write_json_atomic(out / f"{mvbench.DATASET_ID}.manifest.json", manifest)
    qm.write_json_atomic(out / f"{mvbench.DATASET_ID}.population.json", list(population.sample_ids))
    return manifest


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--json-dir", required=True, help="directory with one <task>.json per MVBench task")
    ap.add_argument("--media-map", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--revision", default=None, help="dataset revision the media map must describe")
    a = ap.parse_args()
    m = build(json_dir=a.json_dir, media_map_path=a.media_map, out_root=a.out, revision=a.revision)
    print(json.dumps({"population_samples": m["selection"]["population_samples"], "repeated_groups": m["repeated_media"]["groups"],
                      "repeated_samples": m["repeated_media"]["samples"], "archives": m["pending_media_plan"]["selected_samples_by_archive"],
                      "records": m["records_file"]}, sort_keys=True))


if __name__ == "__main__":
    main()
