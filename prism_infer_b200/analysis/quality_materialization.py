"""Deterministic sample selection and content-addressed media materialisation for the quality
runs (behaviour of the reference's ``prism_infer/analysis/quality_materialization.py:46-640``).

* Selection: samples are ranked by ``sha256(dataset_id + revision + sample_id + str(seed))``
  (ties by id); the development subset is a prefix of the final subset, so results on the
  small set are a subset of the big one.
* Materialisation: media bytes are stored under ``<root>/<dataset>/<sha256>.<ext>`` through a
  temporary file and a rename; the record keeps the digest, size and (for images) format and
  dimensions.  Verification re-hashes every file and the selection.
No dataset is downloaded here; callers hand in rows they have read themselves.
"""

from __future__ import annotations

import hashlib
import io
import json
import os
from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .identity import canonical_json_sha256
from .schema_constants import SHA256_HEX_LENGTH, is_lower_hex

MATERIALIZATION_SCHEMA_VERSION = 1
SELECTION_PREIMAGE_ENCODING = "utf8(dataset_id + revision + sample_id + decimal_seed)"
IMAGE_SUFFIX = {"PNG": ".png", "JPEG": ".jpg", "WEBP": ".webp", "BMP": ".bmp", "GIF": ".gif"}


def sha256_bytes(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def sha256_file(path: str | Path, chunk: int = 1 << 20) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        while True:
            block = fh.read(chunk)
            if not block:
                return h.hexdigest()
            h.update(block)


def canonical_sample_id(value: object) -> str:
    if isinstance(value, bool) or not isinstance(value, (str, int)):
        raise ValueError(f"sample id must be a string or an integer, got {value!r}")
    text = str(value)
    if not text:
        raise ValueError("sample id must not be empty")
    return text


def selection_sha256(*, dataset_id: str, revision: str, sample_id: str, seed: int) -> str:
    if not dataset_id or not revision or not sample_id:
        raise ValueError("selection identity fields must be non-empty")
    if isinstance(seed, bool) or not isinstance(seed, int) or seed <= 0:
        raise ValueError("selection seed must be a positive integer")
    return sha256_bytes(f"{dataset_id}{revision}{sample_id}{seed}".encode())


def selected_ids_sha256(sample_ids: Sequence[object]) -> str:
    ids = [canonical_sample_id(s) for s in sample_ids]
    if len(set(ids)) != len(ids):
        raise ValueError("selected sample ids must be unique")
    return canonical_json_sha256(ids)


@dataclass(frozen=True)
class SampleSelection:
    population_samples: int
    development_ids: tuple[str, ...]
    final_ids: tuple[str, ...]

    def to_record(self) -> dict[str, Any]:
        def part(ids: tuple[str, ...]) -> dict[str, Any]:
            return {"samples": len(ids), "sample_ids": list(ids), "selected_sample_ids_sha256": selected_ids_sha256(ids)}

        return {"population_samples": self.population_samples, "development": part(self.development_ids), "final": part(self.final_ids)}


def select_sample_ids(sample_ids: Sequence[object], *, dataset_id: str, revision: str, seed: int, development_samples: int,
                      final_samples: int) -> SampleSelection:
    ids = [canonical_sample_id(s) for s in sample_ids]
    if len(set(ids)) != len(ids):
        raise ValueError(f"{dataset_id} contains duplicate sample ids")
    for name, n in (("development_samples", development_samples), ("final_samples", final_samples)):
        if isinstance(n, bool) or not isinstance(n, int) or n <= 0:
            raise ValueError(f"{name} must be a positive integer")
    if development_samples > final_samples:
        raise ValueError("development_samples cannot exceed final_samples")
    if final_samples > len(ids):
        raise ValueError(f"{dataset_id}: {final_samples} samples requested, {len(ids)} available")
    ranked = sorted(ids, key=lambda s: (selection_sha256(dataset_id=dataset_id, revision=revision, sample_id=s, seed=seed), s))
    final = tuple(ranked[:final_samples])
    return SampleSelection(len(ids), final[:development_samples], final)


def image_metadata(payload: bytes) -> tuple[str, int, int]:
    from PIL import Image

    with Image.open(io.BytesIO(payload)) as im:
        im.verify()
    with Image.open(io.BytesIO(payload)) as im:
        fmt, (w, h) = im.format or "", im.size
    if fmt not in IMAGE_SUFFIX:
        raise ValueError(f"unsupported image format {fmt!r}")
    return fmt, w, h


def atomic_write_bytes(path: Path, payload: bytes) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    with open(tmp, "wb") as fh:
        fh.write(payload)
        fh.flush()
        os.fsync(fh.fileno())
    os.replace(tmp, path)


def materialize_image(payload: bytes, *, root: str | Path, dataset_id: str) -> dict[str, Any]:
    """Store one image by content; returns its media record (relative path, digest, geometry)."""
    fmt, w, h = image_metadata(payload)
    digest = sha256_bytes(payload)
    rel = Path(dataset_id) / f"{digest}{IMAGE_SUFFIX[fmt]}"
    dest = Path(root) / rel
    if dest.exists():
        if sha256_file(dest) != digest:
            raise OSError(f"existing file does not match its content address: {dest}")
    else:
        atomic_write_bytes(dest, payload)
    return {"materialized_path": rel.as_posix(), "sha256": digest, "bytes": len(payload), "format": fmt, "width": w, "height": h}


def safe_materialized_path(root: str | Path, relative: str) -> Path:
    base = Path(root).resolve()
    path = (base / relative).resolve()
    if base != path and base not in path.parents:
        raise ValueError(f"materialized path escapes the root: {relative!r}")
    return path


def validate_selected_records(records: Sequence[Mapping[str, Any]], expected_ids: Sequence[str]) -> None:
    got = [canonical_sample_id(r.get("sample_id")) for r in records]
    if got != [canonical_sample_id(s) for s in expected_ids]:
        raise ValueError("materialized records do not match the selection (ids or order differ)")
    for r in records:
        media = r.get("media")
        if not isinstance(media, list) or not media:
            raise ValueError(f"record {r.get('sample_id')!r} has no media")
        for m in media:
            if not is_lower_hex(m.get("sha256"), SHA256_HEX_LENGTH) or not isinstance(m.get("materialized_path"), str):
                raise ValueError(f"record {r.get('sample_id')!r} has an invalid media entry")


def verify_materialized_records(records: Sequence[Mapping[str, Any]], root: str | Path) -> dict[str, int]:
    """Re-hash every media file; raises on the first mismatch.  Returns counts."""
    files = nbytes = 0
    seen: set[str] = set()
    for r in records:
        for m in r["media"]:
            if m["sha256"] in seen:
                continue
            seen.add(m["sha256"])
            path = safe_materialized_path(root, m["materialized_path"])
            if sha256_file(path) != m["sha256"]:
                raise OSError(f"content hash mismatch: {path}")
            files += 1
            nbytes += path.stat().st_size
    return {"records": len(records), "unique_media_files": files, "bytes": nbytes}


def materialization_manifest(*, dataset_id: str, revision: str, seed: int, selection: SampleSelection,
                             records: Sequence[Mapping[str, Any]]) -> dict[str, Any]:
    validate_selected_records(records, selection.final_ids)
    return {"schema_version": MATERIALIZATION_SCHEMA_VERSION, "record_type": "quality_materialization", "dataset_id": dataset_id,
            "revision": revision, "selection": {"algorithm": "sha256-rank", "preimage": SELECTION_PREIMAGE_ENCODING, "seed": seed,
                                                **selection.to_record()},
            "records_sha256": canonical_json_sha256(list(records)),
            "media_sha256": sorted({m["sha256"] for r in records for m in r["media"]})}


def write_json_atomic(path: str | Path, value: object) -> str:
    data = json.dumps(value, indent=1, sort_keys=True, ensure_ascii=True).encode() + b"\n"
    atomic_write_bytes(Path(path), data)
    return sha256_bytes(data)


def write_jsonl_atomic(path: str | Path, records: Sequence[Mapping[str, Any]]) -> str:
    data = b"".join(json.dumps(r, sort_keys=True, ensure_ascii=True).encode() + b"\n" for r in records)
    atomic_write_bytes(Path(path), data)
    return sha256_bytes(data)
