"""MVBench metadata, repeated-media selection and archive extraction for the video quality runs.

Behaviour of the reference's MVBench path (``prism_infer/analysis/quality_materialization.py:155-168,
326-452``, ``scripts/build_mvbench_repeated_subset.py:41-108``, ``scripts/materialize_mvbench_media.py:95-283``),
written around three small pieces:

* ``Population``: the task JSON files of the dataset plus a *media map* (which archive and which
  directory inside it holds a task's clips, whether the task cuts a time window out of the clip,
  whether the source needs a separate licence).  One record per question; its media entry starts as
  *pending* and names the exact archive member it needs.
* ``repeated_media_groups``: questions are grouped by the exact source they look at (archive, member,
  media type, time window); groups of two or more questions are the repeated-visual-context subset.
* ``ArchiveExtractor``: copies the needed members out of a ZIP archive (any seekable file object: a
  local file or an HTTP range reader) into a content-addressed tree, one file per video, one file per
  frame of a frame directory; a frame directory is identified by the hash of its ordered
  (member, digest) list.  Members that the archive does not have are marked excluded, never invented.
Nothing here downloads by itself and nothing decodes video.
"""

from __future__ import annotations

import hashlib
import json
import math
import os
import zipfile
from collections.abc import Mapping, Sequence
from dataclasses import dataclass, field
from pathlib import Path, PurePosixPath
from typing import Any, BinaryIO

from .identity import canonical_json_sha256
from .quality_materialization import sha256_file

DATASET_ID = "mvbench_test"
SAMPLE_ID_SEPARATOR = "|"
VIDEO_SUFFIXES = frozenset({".avi", ".gif", ".mkv", ".mov", ".mp4", ".webm"})
FRAME_SUFFIXES = frozenset({".bmp", ".jpeg", ".jpg", ".png", ".webp"})
COPY_CHUNK = 1 << 20

PENDING_ARCHIVE = "pending_archive_extraction"
PENDING_MANUAL = "pending_manual_source"
COMPLETE = "complete"
EXCLUDED_MISSING = "excluded_missing_frozen_archive_member"
EXCLUDED_LICENCE = "excluded_manual_ntu_rgbd_license_required"


def sample_id(task: str, video: str, question_index: int) -> str:
    """``task|video|index``: the same clip can be asked about several times in one task."""
    if not task or not video:
        raise ValueError("MVBench task and video must be non-empty")
    if SAMPLE_ID_SEPARATOR in task or SAMPLE_ID_SEPARATOR in video:
        raise ValueError(f"MVBench task / video must not contain {SAMPLE_ID_SEPARATOR!r}")
    if isinstance(question_index, bool) or not isinstance(question_index, int) or question_index < 0:
        raise ValueError("MVBench question index must be a non-negative integer")
    return SAMPLE_ID_SEPARATOR.join((task, video, str(question_index)))


def _finite_number(value: object) -> bool:
    return not isinstance(value, bool) and isinstance(value, (int, float)) and math.isfinite(float(value))


@dataclass(frozen=True)
class TaskMedia:
    """Where one task's clips live."""

    task: str
    archive: str | None          # None: not redistributed, the user has to obtain it
    prefix: str                  # directory of the clips inside the archive
    media_type: str              # "video" (one file) or "frames" (a directory of images)
    windowed: bool               # questions carry a start / end time
    availability: str = "archive_available"

    @classmethod
    def parse(cls, task: str, spec: Mapping[str, Any], archives: Mapping[str, Any]) -> "TaskMedia":
        archive = spec.get("archive")
        if archive is not None and not isinstance(archives.get(archive), Mapping):
            raise ValueError(f"MVBench task {task!r} names an archive the media map does not describe: {archive!r}")
        prefix = spec.get("media_prefix")
        if not isinstance(prefix, str) or not prefix:
            raise ValueError(f"MVBench task {task!r} has no media_prefix")
        kind = spec.get("media_type")
        if kind not in ("video", "frames"):
            raise ValueError(f"MVBench task {task!r} has media_type {kind!r}; expected 'video' or 'frames'")
        return cls(task, archive, prefix, kind, bool(spec.get("uses_temporal_bound")),
                   str(spec.get("availability", "archive_available")))


@dataclass
class MediaMap:
    revision: str
    archives: dict[str, dict[str, Any]]
    tasks: dict[str, TaskMedia]
    raw: dict[str, Any] = field(repr=False, default_factory=dict)

    @classmethod
    def parse(cls, value: Mapping[str, Any]) -> "MediaMap":
        archives, tasks = value.get("archives"), value.get("tasks")
        if not isinstance(archives, Mapping):
            raise ValueError("MVBench media map has no archives")
        if not isinstance(tasks, Mapping) or not tasks:
            raise ValueError("MVBench media map has no tasks")
        for name, a in archives.items():
            if not isinstance(a, Mapping) or not isinstance(a.get("repository_path"), str) or not _finite_number(a.get("bytes")) \
                    or not isinstance(a.get("sha256"), str):
                raise ValueError(f"MVBench archive {name!r} needs repository_path, bytes and sha256")
        revision = value.get("dataset_revision")
        if not isinstance(revision, str) or not revision:
            raise ValueError("MVBench media map has no dataset_revision")
        return cls(revision, {k: dict(v) for k, v in archives.items()},
                   {t: TaskMedia.parse(t, s, archives) for t, s in tasks.items()}, dict(value))

    @classmethod
    def load(cls, path: str | Path) -> "MediaMap":
        value = json.loads(Path(path).read_text(encoding="utf-8"))
        if not isinstance(value, dict):
            raise ValueError(f"expected a JSON object: {path}")
        return cls.parse(value)

    @property
    def sha256(self) -> str:
        return canonical_json_sha256(self.raw)


def question_record(row: Mapping[str, Any], *, index: int, media: TaskMedia, archives: Mapping[str, Any]) -> dict[str, Any]:
    """One question as the evaluator reads it; the media entry is pending until extraction."""
    where = f"MVBench {media.task}[{index}]"
    video, question, candidates, answer = (row.get(k) for k in ("video", "question", "candidates", "answer"))
    if not isinstance(video, str) or not video:
        raise ValueError(f"{where} has no video")
    if not isinstance(question, str) or not question:
        raise ValueError(f"{where} has no question")
    if not isinstance(candidates, list) or not candidates or not all(isinstance(c, str) and c for c in candidates):
        raise ValueError(f"{where} has invalid candidates")
    if not isinstance(answer, str) or answer not in candidates:
        raise ValueError(f"{where}: the answer is not one of the candidates")
    window = None
    if media.windowed:
        start, end = row.get("start"), row.get("end")
        if not (_finite_number(start) and _finite_number(end) and float(start) >= 0.0 and float(end) > float(start)):
            raise ValueError(f"{where} has an invalid time window")
        window = {"start": float(start), "end": float(end)}
    entry: dict[str, Any] = {
        "source_path": video,
        "archive_member_path": (PurePosixPath(media.prefix) / video).as_posix(),
        "media_type": media.media_type,
        "materialization_status": PENDING_MANUAL if media.archive is None else PENDING_ARCHIVE,
        "materialized_path": None,
        "sha256": None,
    }
    if media.archive is not None:
        a = archives[media.archive]
        entry["archive"] = {"name": media.archive, "repository_path": a["repository_path"], "bytes": a["bytes"], "sha256": a["sha256"]}
    return {
        "sample_id": sample_id(media.task, video, index), "task": media.task, "question_index": index, "question": question,
        "candidates": list(candidates), "answer": answer, "answer_index": candidates.index(answer), "temporal_bound": window,
        "subtitle": row.get("subtitle"), "source_availability": media.availability, "media": [entry],
    }


@dataclass
class Population:
    sample_ids: list[str]
    records: dict[str, dict[str, Any]]
    source_files: list[Path]

    @classmethod
    def load(cls, json_dir: str | Path, media_map: MediaMap) -> "Population":
        """Every ``<task>.json`` under ``json_dir``; the task set must equal the media map's."""
        paths = sorted(Path(json_dir).glob("*.json"))
        found = {p.stem for p in paths}
        if found != set(media_map.tasks):
            raise ValueError(f"MVBench task files differ from the media map: missing={sorted(set(media_map.tasks) - found)}, "
                             f"extra={sorted(found - set(media_map.tasks))}")
        ids: list[str] = []
        records: dict[str, dict[str, Any]] = {}
        for path in paths:
            rows = json.loads(path.read_text(encoding="utf-8"))
            if not isinstance(rows, list) or not rows:
                raise ValueError(f"MVBench task file must hold a non-empty list: {path}")
            for i, row in enumerate(rows):
                if not isinstance(row, Mapping):
                    raise ValueError(f"MVBench {path.stem}[{i}] is not an object")
                rec = question_record(row, index=i, media=media_map.tasks[path.stem], archives=media_map.archives)
                if rec["sample_id"] in records:
                    raise ValueError(f"duplicate MVBench sample id {rec['sample_id']!r}")
                ids.append(rec["sample_id"])
                records[rec["sample_id"]] = rec
        return cls(ids, records, paths)


# ------------------------------------------------------------------ repeated-media selection
def source_contract(record: Mapping[str, Any]) -> dict[str, Any]:
    """What a question looks at, exactly: two questions share visual context iff these are equal."""
    media = record.get("media")
    if not isinstance(media, list) or len(media) != 1 or not isinstance(media[0], Mapping):
        raise ValueError("a repeated-media group needs records with exactly one media source")
    m = media[0]
    archive = m.get("archive")
    if archive is not None and not isinstance(archive, Mapping):
        raise ValueError("the archive entry of a media source must be an object")
    member = m.get("archive_member_path")
    if not isinstance(member, str) or not member:
        raise ValueError("media source without an archive member path")
    if m.get("media_type") not in ("frames", "video"):
        raise ValueError(f"unsupported media type {m.get('media_type')!r}")
    return {"archive_name": archive.get("name") if archive else None,
            "archive_repository_path": archive.get("repository_path") if archive else None,
            "archive_member_path": member, "media_type": m["media_type"], "temporal_bound": record.get("temporal_bound")}


def repeated_media_groups(records: Sequence[Mapping[str, Any]]) -> tuple[list[dict[str, Any]], list[dict[str, Any]]]:
    """All groups of at least two questions over the same source.  Groups in ascending order of their
    contract hash, questions inside a group by (task, question index, sample id).  Returns the selected
    records in that order and one summary per group."""
    by_group: dict[str, list[Mapping[str, Any]]] = {}
    contracts: dict[str, dict[str, Any]] = {}
    for r in records:
        c = source_contract(r)
        gid = canonical_json_sha256(c)
        by_group.setdefault(gid, []).append(r)
        contracts[gid] = c
    chosen: list[dict[str, Any]] = []
    groups: list[dict[str, Any]] = []
    for gid in sorted(by_group):
        rows = by_group[gid]
        if len(rows) < 2:
            continue
        rows = sorted(rows, key=lambda r: (str(r.get("task", "")), int(r.get("question_index", -1)), str(r.get("sample_id", ""))))
        ids = [str(r["sample_id"]) for r in rows]
        chosen += [dict(r) for r in rows]
        groups.append({"source_contract_sha256": gid, "source_contract": contracts[gid], "samples": len(ids), "sample_ids": ids,
                       "sample_ids_sha256": canonical_json_sha256(ids)})
    if not groups:
        raise ValueError("no two MVBench questions share their media")
    return chosen, groups


# ------------------------------------------------------------------ archive extraction
class ArchiveExtractor:
    """Copies members of one ZIP archive into ``<root>/media/mvbench_test/<aa>/<sha256><suffix>``.

    ``source`` is a path or any seekable binary file object.  A member is extracted once however many
    questions use it; an existing destination must already hold the same bytes."""

    def __init__(self, source: str | Path | BinaryIO, *, name: str, root: str | Path) -> None:
        self.name = name
        self.root = Path(root)
        self.zip = zipfile.ZipFile(source)
        self._index = {i.filename: i for i in self.zip.infolist() if not i.is_dir()}
        self._done: dict[str, dict[str, Any]] = {}

    def close(self) -> None:
        self.zip.close()

    def __enter__(self) -> "ArchiveExtractor":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def members_for(self, media: Mapping[str, Any]) -> list[zipfile.ZipInfo]:
        member = media["archive_member_path"]
        if media["media_type"] == "frames":
            prefix = member.rstrip("/") + "/"
            return [self._index[n] for n in sorted(self._index) if n.startswith(prefix)]
        info = self._index.get(member)
        return [info] if info is not None else []

    def inventory(self, medias: Sequence[Mapping[str, Any]]) -> dict[str, Any]:
        """What an extraction of these media entries would read, without reading it."""
        unique: dict[str, zipfile.ZipInfo] = {}
        missing = []
        for m in medias:
            infos = self.members_for(m)
            if not infos:
                missing.append(m["archive_member_path"])
            unique.update({i.filename: i for i in infos})
        return {"selected_samples": len(medias), "unique_members": len(unique), "missing_members": sorted(missing),
                "selected_compressed_bytes": sum(i.compress_size for i in unique.values()),
                "selected_uncompressed_bytes": sum(i.file_size for i in unique.values())}

    def _extract(self, info: zipfile.ZipInfo, media_type: str) -> dict[str, Any]:
        suffix = PurePosixPath(info.filename).suffix.lower()
        if suffix not in (FRAME_SUFFIXES if media_type == "frames" else VIDEO_SUFFIXES):
            raise ValueError(f"archive member {info.filename!r} is not a {media_type} file")
        staging_dir = self.root / ".staging"
        staging_dir.mkdir(parents=True, exist_ok=True)
        staging = staging_dir / (hashlib.sha256(f"{self.name}\0{info.filename}".encode()).hexdigest() + f"{suffix}.tmp{os.getpid()}")
        h, n = hashlib.sha256(), 0
        try:
            with self.zip.open(info, "r") as src, open(staging, "wb") as dst:
                while chunk := src.read(COPY_CHUNK):
                    dst.write(chunk)
                    h.update(chunk)
                    n += len(chunk)
            if n != info.file_size:
                raise OSError(f"archive member {info.filename}: {n} bytes read, {info.file_size} recorded")
            digest = h.hexdigest()
            rel = PurePosixPath("media") / DATASET_ID / digest[:2] / f"{digest}{suffix}"
            dest = self.root / Path(rel)
            if dest.exists():
                if dest.stat().st_size != n or sha256_file(dest) != digest:
                    raise ValueError(f"existing file does not match its content address: {dest}")
            else:
                dest.parent.mkdir(parents=True, exist_ok=True)
                os.replace(staging, dest)
            return {"archive_member_path": info.filename, "materialized_path": rel.as_posix(), "sha256": digest, "bytes": n}
        finally:
            staging.unlink(missing_ok=True)

    def materialize(self, media: dict[str, Any]) -> None:
        """Fill one media entry in place: complete with its identity, or excluded when the member is absent."""
        infos = self.members_for(media)
        if not infos:
            media.update({"materialization_status": EXCLUDED_MISSING, "materialized_path": None, "sha256": None,
                          "exclusion_reason": "the archive of the recorded dataset revision does not contain this member"})
            return
        parts = []
        for info in infos:
            if info.filename not in self._done:
                self._done[info.filename] = self._extract(info, media["media_type"])
            parts.append(self._done[info.filename])
        if media["media_type"] == "frames":
            identity = [{"archive_member_path": p["archive_member_path"], "sha256": p["sha256"]} for p in parts]
            media.update({"materialization_status": COMPLETE, "identity_kind": "canonical_frame_manifest_sha256", "materialized_path": None,
                          "sha256": canonical_json_sha256(identity), "bytes": sum(p["bytes"] for p in parts), "frames": parts})
        else:
            if len(parts) != 1:
                raise ValueError("a video source must be exactly one archive member")
            media.update({"materialization_status": COMPLETE, "identity_kind": "file_sha256", "materialized_path": parts[0]["materialized_path"],
                          "sha256": parts[0]["sha256"], "bytes": parts[0]["bytes"]})


def exclude_manual_sources(records: Sequence[dict[str, Any]]) -> int:
    """Sources that need a separately licensed download leave the evaluation subset, visibly."""
    n = 0
    for r in records:
        for m in r["media"]:
            if m.get("archive") is None and m.get("materialization_status") == PENDING_MANUAL:
                m.update({"materialization_status": EXCLUDED_LICENCE,
                          "exclusion_reason": "the recorded source requires separately licensed NTU RGB+D media"})
                n += 1
    return n


def evaluation_subset(records: Sequence[Mapping[str, Any]]) -> dict[str, Any]:
    """Which samples can be evaluated: all media complete.  Pending media keep the whole artifact pending;
    excluded media remove their sample and are listed with the reason."""
    eligible, excluded, pending = [], [], []
    for r in records:
        states = [m.get("materialization_status") for m in r["media"]]
        if all(s == COMPLETE and m.get("sha256") for s, m in zip(states, r["media"])):
            eligible.append(str(r["sample_id"]))
        elif any(isinstance(s, str) and s.startswith("excluded_") for s in states):
            excluded.append({"sample_id": str(r["sample_id"]), "reasons": sorted({s for s in states if isinstance(s, str) and s.startswith("excluded_")})})
        else:
            pending.append(str(r["sample_id"]))
    return {"status": "pending" if pending else "complete", "eligible_samples": len(eligible), "eligible_sample_ids_sha256": canonical_json_sha256(eligible),
            "excluded_samples": len(excluded), "excluded": excluded, "pending_samples": len(pending)}


def pending_plan(records: Sequence[Mapping[str, Any]]) -> dict[str, Any]:
    """Archives still to be read, with the bytes a full download of each would take."""
    by_archive: dict[str, int] = {}
    size: dict[str, int] = {}
    manual = 0
    for r in records:
        for m in r["media"]:
            status = m.get("materialization_status")
            if m.get("sha256") is not None or (isinstance(status, str) and status.startswith("excluded_")):
                continue
            a = m.get("archive")
            if a is None:
                manual += 1
            else:
                by_archive[a["name"]] = by_archive.get(a["name"], 0) + 1
                size[a["name"]] = int(a["bytes"])
    return {"selected_samples_by_archive": dict(sorted(by_archive.items())), "manual_source_samples": manual,
            "full_archive_download_bytes": sum(size.values())}
