"""Materialise the selected quality subset of a dataset from local parquet shards (reference
``scripts/materialize_quality_data.py``).

The raw dataset (parquet shards with embedded image bytes, fetched beforehand by whatever means
the machine has) is read twice, in batches: first only the id column of every shard, from which
the deterministic SHA-256-rank selection picks the development and final subsets; then the
selected rows only, whose images are written content-addressed under the output root.  The
results are a records JSONL (the input of ``benchmarks/bench_working_set_quality.py``), and a
manifest that names the source shards by digest, the selection and the media, so that
``utils/verify_quality_data.py`` can re-check everything later.

Two row layouts are known: ``docvqa`` (columns ``questionId``, ``question``, ``answers``, ``image``)
and ``muirbench`` (``idx``, ``question``, ``options``, ``answer``, ``image_list`` ...).  Shards must be
named ``<split>-00000-of-0000N.parquet`` and be complete: a missing shard is an error, not a
smaller population.

    python -m prism_infer_b200.utils.materialize_quality_data --layout muirbench --dataset-id muirbench \
        --revision <hf revision> --raw-dir data/raw/muirbench --split test --final 200 --development 20 --out data/quality
"""

from __future__ import annotations

import argparse
import json
import re
from pathlib import Path
from typing import Any, Iterator, Mapping, Sequence

from ..analysis import quality_materialization as qmat

SHARD_NAME = re.compile(r"^(?P<split>[A-Za-z_]+)-(?P<index>\d{5})-of-(?P<total>\d{5})\.parquet$")
LAYOUTS = {
    "docvqa": {"id": "questionId", "columns": ("questionId", "question", "answers", "image", "question_types", "docId")},
    "muirbench": {"id": "idx", "columns": ("idx", "task", "image_relation", "image_type", "question", "options", "answer", "image_list",
                                            "counterpart_idx")},
}


def discover_complete_shards(directory: str | Path, split: str) -> list[Path]:
    found = []
    for p in sorted(Path(directory).glob(f"{split}-*-of-*.parquet")):
        m = SHARD_NAME.fullmatch(p.name)
        if m is None or m.group("split") != split:
            raise ValueError(f"invalid parquet shard name: {p}")
        found.append((int(m.group("index")), int(m.group("total")), p))
    if not found:
        raise FileNotFoundError(f"no {split} parquet shards in {directory}")
    totals = {t for _, t, _ in found}
    if len(totals) != 1:
        raise ValueError(f"inconsistent shard totals in {directory}: {sorted(totals)}")
    total = totals.pop()
    if [i for i, _, _ in found] != list(range(total)):
        raise ValueError(f"incomplete {split} shards in {directory}: expected {total}, found indices {[i for i, _, _ in found]}")
    return [p for _, _, p in found]


def parquet_rows(paths: Sequence[Path], columns: Sequence[str], batch_size: int) -> Iterator[dict[str, Any]]:
    import pyarrow.parquet as pq

    for path in paths:
        f = pq.ParquetFile(path)
        have = set(f.schema_arrow.names)
        for batch in f.iter_batches(batch_size=batch_size, columns=[c for c in columns if c in have]):
            yield from batch.to_pylist()


def _image_bytes(value: Any, sample_id: str) -> bytes:
    if isinstance(value, Mapping) and isinstance(value.get("bytes"), (bytes, bytearray)):
        return bytes(value["bytes"])
    if isinstance(value, (bytes, bytearray)):
        return bytes(value)
    raise ValueError(f"sample {sample_id} has no embedded image bytes")


def convert_row(layout: str, row: Mapping[str, Any], *, root: str | Path, dataset_id: str) -> dict[str, Any]:
    """One selected raw row -> evaluator record with materialised media."""
    sid = qmat.canonical_sample_id(row.get(LAYOUTS[layout]["id"]))
    question = row.get("question")
    if not isinstance(question, str) or not question:
        raise ValueError(f"{dataset_id} {sid} has no question")
    if layout == "docvqa":
        answers = row.get("answers")
        if not isinstance(answers, list) or not answers or not all(isinstance(a, str) and a for a in answers):
            raise ValueError(f"{dataset_id} {sid} has invalid answers")
        media = [qmat.materialize_image(_image_bytes(row.get("image"), sid), root=root, dataset_id=dataset_id)]
        return {"sample_id": sid, "question": question, "answers": list(answers), "question_types": list(row.get("question_types") or []),
                "document": {"doc_id": row.get("docId")}, "media": media}
    options, answer, images = row.get("options"), row.get("answer"), row.get("image_list")
    if not isinstance(options, list) or not options or not all(isinstance(o, str) for o in options):
        raise ValueError(f"{dataset_id} {sid} has invalid options")
    if answer not in {chr(65 + i) for i in range(len(options))}:
        raise ValueError(f"{dataset_id} {sid} answer {answer!r} is outside its options")
    if not isinstance(images, list) or not images:
        raise ValueError(f"{dataset_id} {sid} has an invalid image_list")
    media = [qmat.materialize_image(_image_bytes(im, sid), root=root, dataset_id=dataset_id) for im in images]
    return {"sample_id": sid, "task": row.get("task"), "image_relation": row.get("image_relation"), "image_type": row.get("image_type"),
            "question": question, "options": list(options), "answer": answer, "counterpart_idx": row.get("counterpart_idx"), "media": media}


def materialize(*, layout: str, dataset_id: str, revision: str, raw_dir: str | Path, split: str, out_root: str | Path, seed: int,
                development: int, final: int, batch_size: int = 64) -> dict[str, Any]:
    if layout not in LAYOUTS:
        raise ValueError(f"unknown layout {layout!r}; known: {sorted(LAYOUTS)}")
    spec = LAYOUTS[layout]
    shards = discover_complete_shards(raw_dir, split)
    ids = [r[spec["id"]] for r in parquet_rows(shards, (spec["id"],), batch_size * 16)]
    selection = qmat.select_sample_ids(ids, dataset_id=dataset_id, revision=revision, seed=seed, development_samples=development,
                                       final_samples=final)
    wanted = set(selection.final_ids)
    by_id: dict[str, dict[str, Any]] = {}
    for row in parquet_rows(shards, spec["columns"], batch_size):
        sid = qmat.canonical_sample_id(row.get(spec["id"]))
        if sid in wanted:
            by_id[sid] = convert_row(layout, row, root=out_root, dataset_id=dataset_id)
    records = [by_id[s] for s in selection.final_ids]  # selection order
    out = Path(out_root)
    records_path = out / f"{dataset_id}.records.jsonl"
    records_sha = qmat.write_jsonl_atomic(records_path, records)
    manifest = qmat.materialization_manifest(dataset_id=dataset_id, revision=revision, seed=seed, selection=selection, records=records)
    manifest["layout"] = layout
    manifest["records_file"] = {"path": records_path.name, "sha256": records_sha}
    manifest["source_files"] = [{"name": p.name, "bytes": p.stat().st_size, "sha256": qmat.sha256_file(p)} for p in shards]
    qmat.write_json_atomic(out / f"{dataset_id}.population.json", [qmat.canonical_sample_id(i) for i in ids])  # input of verify_quality_data
    manifest["verification"] = qmat.verify_materialized_records(records, out_root)
    qmat.write_json_atomic(out / f"{dataset_id}.manifest.json", manifest)
    return manifest


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layout", choices=sorted(LAYOUTS), required=True)
    ap.add_argument("--dataset-id", required=True)
    ap.add_argument("--revision", required=True)
    ap.add_argument("--raw-dir", required=True)
    ap.add_argument("--split", default="test")
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=20260801)
    ap.add_argument("--development", type=int, default=20)
    ap.add_argument("--final", type=int, default=200)
    ap.add_argument("--batch-size", type=int, default=64)
    a = ap.parse_args()
    m = materialize(layout=a.layout, dataset_id=a.dataset_id, revision=a.revision, raw_dir=a.raw_dir, split=a.split, out_root=a.out,
                    seed=a.seed, development=a.development, final=a.final, batch_size=a.batch_size)
    print(json.dumps({"dataset_id": a.dataset_id, "population": m["selection"]["population_samples"],
                      "final": m["selection"]["final"]["samples"], "media_files": m["verification"]["unique_media_files"],
                      "records": m["records_file"]}))


if __name__ == "__main__":
    main()
