"""Independent check of materialised quality data: the selection is recomputed from the
population ids, the record list must match it, and every media file is re-hashed
(reference: ``scripts/verify_quality_data.py``).

    python -m prism_infer_b200.utils.verify_quality_data --manifest m.json --records r.jsonl --population ids.json --root data/
"""

from __future__ import annotations

import argparse
import json
import sys

from ..analysis import quality_materialization as qm


def verify(manifest: dict, records: list[dict], population_ids: list, root: str) -> dict:
    sel = manifest["selection"]
    again = qm.select_sample_ids(population_ids, dataset_id=manifest["dataset_id"], revision=manifest["revision"], seed=sel["seed"],
                                 development_samples=sel["development"]["samples"], final_samples=sel["final"]["samples"])
    if again.to_record() != {k: sel[k] for k in ("population_samples", "development", "final")}:
        raise ValueError("the recorded selection cannot be reproduced from the population ids")
    qm.validate_selected_records(records, again.final_ids)
    if qm.canonical_json_sha256(records) != manifest["records_sha256"]:
        raise ValueError("records file differs from the manifest")
    return qm.verify_materialized_records(records, root)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--manifest", required=True)
    ap.add_argument("--records", required=True)
    ap.add_argument("--population", required=True, help="JSON list of all sample ids of the dataset split")
    ap.add_argument("--root", required=True)
    args = ap.parse_args()
    with open(args.manifest) as fh:
        manifest = json.load(fh)
    with open(args.records) as fh:
        records = [json.loads(line) for line in fh if line.strip()]
    with open(args.population) as fh:
        population = json.load(fh)
    print(json.dumps(verify(manifest, records, population, args.root)))


if __name__ == "__main__":
    try:
        main()
    except (ValueError, OSError) as exc:
        print(f"verification failed: {exc}", file=sys.stderr)
        sys.exit(1)
