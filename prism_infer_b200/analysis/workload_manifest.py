"""Contract of a benchmark workload manifest (``benchmarks/workloads/system_cases.json`` and user-written ones).

A manifest names cases; a case is a list of requests; a request has a type, a prompt and the visual inputs of its
type, described so that every run materialises the same pixels:

* ``{"width", "height", "seed"}`` uniform noise from a seeded generator, or ``{"width", "height", "color": [r, g, b]}``
  a flat colour;
* ``image_file`` requests point at a file (``path`` relative to the manifest, ``sha256``, ``width``, ``height``,
  ``source_url``) whose bytes are checked when it is loaded;
* a request may carry an ``evaluation``: a caption or free-text task with several reference answers taken from a
  named ``reference_sources`` entry (dataset, split, annotation file and its content hash), scored with
  ``analysis/reference_quality.py``.

Behaviour of the reference's validator (``prism_infer/analysis/benchmark_schema.py:104-412``), expressed as one
walker over typed field tables instead of one function per field kind."""

from __future__ import annotations

import json
from collections.abc import Mapping
from pathlib import Path
from typing import Any

from .reference_quality import normalize_reference_text
from .schema_constants import SHA256_HEX_LENGTH, is_lower_hex

WORKLOAD_SCHEMA_VERSION = 1
REQUEST_TYPES = ("text", "image", "image_file", "images", "interleaved_images", "video")
TASKS = ("caption", "free_text_qa")
IMAGE_MARKER = "<image>"


class ManifestError(ValueError):
    pass


def _need(obj: Any, key: str, kind: str, path: str) -> Any:
    """``kind``: str (non-empty), posint, sha256, list (non-empty), obj."""
    if not isinstance(obj, Mapping):
        raise ManifestError(f"{path} must be an object")
    if key not in obj:
        raise ManifestError(f"{path}.{key} is missing")
    v = obj[key]
    ok = {"str": isinstance(v, str) and bool(v),
          "posint": isinstance(v, int) and not isinstance(v, bool) and v > 0,
          "sha256": is_lower_hex(v, SHA256_HEX_LENGTH),
          "list": isinstance(v, list) and bool(v),
          "obj": isinstance(v, Mapping)}[kind]
    if not ok:
        raise ManifestError(f"{path}.{key} = {v!r} is not a valid {kind}")
    return v


def _synthetic_image(spec: Any, path: str) -> None:
    _need(spec, "width", "posint", path)
    _need(spec, "height", "posint", path)
    if ("seed" in spec) == ("color" in spec):
        raise ManifestError(f"{path} needs exactly one of 'seed' (noise) and 'color' (flat)")
    if "seed" in spec:
        s = spec["seed"]
        if isinstance(s, bool) or not isinstance(s, int) or s < 0:
            raise ManifestError(f"{path}.seed must be a non-negative integer")
        return
    color = spec["color"]
    if not isinstance(color, list) or len(color) != 3 or any(isinstance(c, bool) or not isinstance(c, int) or not 0 <= c <= 255 for c in color):
        raise ManifestError(f"{path}.color must be three integers in 0..255")


def _file_image(spec: Any, path: str) -> None:
    for key, kind in (("path", "str"), ("source_url", "str"), ("sha256", "sha256"), ("width", "posint"), ("height", "posint")):
        _need(spec, key, kind, path)
    if Path(spec["path"]).is_absolute() or ".." in Path(spec["path"]).parts:
        raise ManifestError(f"{path}.path must stay below the manifest's directory")


def _image_list(request: Mapping[str, Any], key: str, path: str) -> int:
    items = _need(request, key, "list", path)
    for i, spec in enumerate(items):
        _synthetic_image(spec, f"{path}.{key}[{i}]")
    return len(items)


def _sources(manifest: Mapping[str, Any]) -> dict[str, str]:
    """``reference_sources`` -> ``{source id: task}``."""
    raw = manifest.get("reference_sources", {})
    if not isinstance(raw, Mapping):
        raise ManifestError("manifest.reference_sources must be an object")
    tasks = {}
    for sid, src in raw.items():
        path = f"manifest.reference_sources.{sid}"
        if not isinstance(sid, str) or not sid:
            raise ManifestError("reference source ids are non-empty strings")
        for key in ("dataset", "split", "task", "source_url", "annotation_file"):
            _need(src, key, "str", path)
        _need(src, "content_sha256", "sha256", path)
        if src["task"] not in TASKS:
            raise ManifestError(f"{path}.task must be one of {TASKS}")
        tasks[sid] = src["task"]
    return tasks


def _evaluation(ev: Any, path: str, sources: Mapping[str, str]) -> None:
    task = _need(ev, "task", "str", path)
    if task not in TASKS:
        raise ManifestError(f"{path}.task must be one of {TASKS}")
    sid = _need(ev, "reference_source", "str", path)
    if sid not in sources:
        raise ManifestError(f"{path}.reference_source names the unknown source {sid!r}")
    if sources[sid] != task:
        raise ManifestError(f"{path}.task is {task!r}, its source {sid!r} is a {sources[sid]!r} source")
    _need(ev, "image_id", "posint", path)
    seen = set()
    for i, ref in enumerate(_need(ev, "references", "list", path)):
        rp = f"{path}.references[{i}]"
        aid = _need(ref, "annotation_id", "posint", rp)
        if aid in seen:
            raise ManifestError(f"{path} lists annotation {aid} twice")
        seen.add(aid)
        if not normalize_reference_text(_need(ref, "text", "str", rp)):
            raise ManifestError(f"{rp}.text has no word left after normalisation")


def _request(req: Any, path: str, sources: Mapping[str, str]) -> None:
    kind = _need(req, "type", "str", path)
    prompt = _need(req, "prompt", "str", path)
    if kind not in REQUEST_TYPES:
        raise ManifestError(f"{path}.type {kind!r} is not one of {REQUEST_TYPES}")
    if req.get("evaluation") is not None:
        _evaluation(req["evaluation"], f"{path}.evaluation", sources)
    if kind == "image":
        _synthetic_image(_need(req, "image", "obj", path), f"{path}.image")
    elif kind == "image_file":
        _file_image(_need(req, "image", "obj", path), f"{path}.image")
    elif kind == "images":
        _image_list(req, "images", path)
    elif kind == "interleaved_images":
        n = _image_list(req, "images", path)
        if prompt.count(IMAGE_MARKER) != n:
            raise ManifestError(f"{path}.prompt has {prompt.count(IMAGE_MARKER)} {IMAGE_MARKER} markers for {n} images")
    elif kind == "video":
        _image_list(req, "frames", path)
        shapes = {(f["width"], f["height"]) for f in req["frames"]}
        if len(shapes) != 1:
            raise ManifestError(f"{path}.frames must all have the same size")


def validate_workload_manifest(manifest: Any) -> Mapping[str, Any]:
    if not isinstance(manifest, Mapping):
        raise ManifestError("a workload manifest is an object")
    if manifest.get("schema_version") != WORKLOAD_SCHEMA_VERSION:
        raise ManifestError(f"unsupported workload schema_version {manifest.get('schema_version')!r}")
    _need(manifest, "name", "str", "manifest")
    sources = _sources(manifest)
    ids = set()
    for i, case in enumerate(_need(manifest, "cases", "list", "manifest")):
        path = f"manifest.cases[{i}]"
        cid = _need(case, "id", "str", path)
        if cid in ids:
            raise ManifestError(f"case id {cid!r} appears twice")
        ids.add(cid)
        for j, req in enumerate(_need(case, "requests", "list", path)):
            _request(req, f"{path}.requests[{j}]", sources)
    return manifest


def load_workload_manifest(path: str | Path) -> dict[str, Any]:
    value = json.loads(Path(path).read_text(encoding="utf-8"))
    validate_workload_manifest(value)
    return value
