"""Extract the media of selected MVBench questions from the dataset's ZIP archives into a content-addressed
tree and complete the records (reference: ``scripts/materialize_mvbench_media.py``).

Archives are read from ``--archive-dir`` (files named as in the media map) or, with ``--endpoint``, member by
member over HTTP range requests, so a 1 GB archive costs only the bytes of the selected clips.  Members that an
archive does not hold are marked excluded; sources that need a separate licence are excluded with
``--exclude-manual``.  The run can be repeated: extracted files are reused when their bytes match.

    python -m prism_infer_b200.utils.materialize_mvbench_media --root data/quality/mvbench_repeated \
        --archive-dir raw/mvbench/video [--only star.zip] [--inventory-only] [--exclude-manual]
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Any

from ..analysis import mvbench
from ..analysis import quality_materialization as qm
from ..analysis.identity import canonical_json_sha256


def _read_jsonl(path: Path) -> list[dict[str, Any]]:
    rows = [json.loads(line) for line in path.read_text(encoding="utf-8").splitlines() if line.strip()]
    if not rows or not all(isinstance(r, dict) for r in rows):
        raise ValueError(f"expected a non-empty JSONL file of objects: {path}")
    return rows


def archive_url(endpoint: str, repository: str, revision: str, repository_path: str) -> str:
    endpoint = endpoint.rstrip("/")
    if not endpoint.startswith(("https://", "http://")):
        raise ValueError("the endpoint must be an http(s) URL")
    return f"{endpoint}/datasets/{repository}/resolve/{revision}/{repository_path}?download=true"


def _open_archive(name: str, spec: dict[str, Any], *, archive_dir: str | None, endpoint: str | None, repository: str | None,
                  revision: str, check_archive_sha256: bool):
    if archive_dir is not None:
        path = Path(archive_dir) / name
        if not path.is_file():
            return None
        if path.stat().st_size != int(spec["bytes"]):
            raise ValueError(f"{path}: {path.stat().st_size} bytes, the media map records {spec['bytes']}")
        if check_archive_sha256 and qm.sha256_file(path) != spec["sha256"]:
            raise ValueError(f"{path}: content differs from the media map's sha256")
        return path
    if endpoint is None or repository is None:
        raise ValueError("give --archive-dir, or --endpoint with --repository")
    from ..analysis.http_range_reader import HTTPRangeReader

    return HTTPRangeReader(archive_url(endpoint, repository, revision, spec["repository_path"]), expected_size=int(spec["bytes"]))


def materialize(*, root: str | Path, archive_dir: str | None = None, endpoint: str | None = None, repository: str | None = None,
                only: list[str] | None = None, inventory_only: bool = False, exclude_manual: bool = False,
                check_archive_sha256: bool = False) -> dict[str, Any]:
    root = Path(root)
    manifest_path = root / f"{mvbench.DATASET_ID}.manifest.json"
    manifest = json.loads(manifest_path.read_text(encoding="utf-8"))
    records_path = root / manifest["records_file"]["path"]
    if qm.sha256_file(records_path) != manifest["records_file"]["sha256"]:
        raise ValueError("the records file differs from the manifest; refusing to extend it")
    records = _read_jsonl(records_path)
    by_archive: dict[str, list[dict[str, Any]]] = {}
    for r in records:
        for m in r["media"]:
            if m.get("archive") is not None and m.get("materialization_status") == mvbench.PENDING_ARCHIVE:
                by_archive.setdefault(m["archive"]["name"], []).append(m)
    report: dict[str, Any] = {"archives": {}, "skipped_archives": []}
    for name in sorted(by_archive):
        if only and name not in only:
            continue
        medias = by_archive[name]
        source = _open_archive(name, medias[0]["archive"], archive_dir=archive_dir, endpoint=endpoint, repository=repository,
                               revision=manifest["revision"], check_archive_sha256=check_archive_sha256)
        if source is None:
            report["skipped_archives"].append(name)
            continue
        with mvbench.ArchiveExtractor(source, name=name, root=root) as ex:
            report["archives"][name] = ex.inventory(medias)
            if not inventory_only:
                for m in medias:
                    ex.materialize(m)
        if hasattr(source, "range_requests"):
            report["archives"][name]["range_requests"] = source.range_requests
            report["archives"][name]["range_response_bytes"] = source.range_response_bytes
    if inventory_only:
        return report
    if exclude_manual:
        report["excluded_manual_sources"] = mvbench.exclude_manual_sources(records)
    manifest["records_file"]["sha256"] = qm.write_jsonl_atomic(records_path, records)
    manifest["records_sha256"] = canonical_json_sha256(records)
    subset = mvbench.evaluation_subset(records)
    manifest["evaluation_subset"] = subset
    manifest["pending_media_plan"] = mvbench.pending_plan(records)
    manifest["media_sha256"] = sorted({m["sha256"] for r in records for m in r["media"] if m.get("sha256")})
    manifest["materialization_status"] = ("media_materialization_in_progress" if subset["status"] == "pending"
                                          else "complete_with_protocol_exclusions" if subset["excluded_samples"] else "complete")
    report["manifest_sha256"] = qm.write_json_atomic(manifest_path, manifest)
    report["evaluation_subset"] = {k: subset[k] for k in ("status", "eligible_samples", "excluded_samples", "pending_samples")}
    return report


def verify(root: str | Path) -> dict[str, int]:
    """Re-hash every extracted file (videos and frames) against the records."""
    root = Path(root)
    manifest = json.loads((root / f"{mvbench.DATASET_ID}.manifest.json").read_text(encoding="utf-8"))
    records = _read_jsonl(root / manifest["records_file"]["path"])
    if canonical_json_sha256(records) != manifest["records_sha256"]:
        raise ValueError("records differ from the manifest")
    files = nbytes = 0
    seen: set[str] = set()
    for r in records:
        for m in r["media"]:
            if m.get("materialization_status") != mvbench.COMPLETE:
                continue
            parts = m["frames"] if m["media_type"] == "frames" else [m]
            if m["media_type"] == "frames" and m["sha256"] != canonical_json_sha256(
                    [{"archive_member_path": p["archive_member_path"], "sha256": p["sha256"]} for p in parts]):
                raise ValueError(f"frame manifest of {r['sample_id']!r} does not hash to its identity")
            for p in parts:
                if p["sha256"] in seen:
                    continue
                seen.add(p["sha256"])
                path = qm.safe_materialized_path(root, p["materialized_path"])
                if qm.sha256_file(path) != p["sha256"]:
                    raise OSError(f"content hash mismatch: {path}")
                files += 1
                nbytes += path.stat().st_size
    return {"records": len(records), "unique_media_files": files, "bytes": nbytes}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--root", required=True, help="directory written by build_mvbench_repeated_subset")
    ap.add_argument("--archive-dir", default=None)
    ap.add_argument("--endpoint", default=None, help="e.g. https://huggingface.co (member-wise range reads)")
    ap.add_argument("--repository", default=None, help="dataset repository, e.g. OpenGVLab/MVBench")
    ap.add_argument("--only", action="append", default=None, help="archive name; may be repeated")
    ap.add_argument("--inventory-only", action="store_true")
    ap.add_argument("--exclude-manual", action="store_true")
    ap.add_argument("--check-archive-sha256", action="store_true")
    ap.add_argument("--verify", action="store_true", help="only re-hash what has been extracted")
    a = ap.parse_args()
    if a.verify:
        print(json.dumps(verify(a.root), sort_keys=True))
        return
    print(json.dumps(materialize(root=a.root, archive_dir=a.archive_dir, endpoint=a.endpoint, repository=a.repository, only=a.only,
                                 inventory_only=a.inventory_only, exclude_manual=a.exclude_manual,
                                 check_archive_sha256=a.check_archive_sha256), sort_keys=True))


if __name__ == "__main__":
    main()
