"""Shared pieces of the benchmark scripts: what was measured (source identity), on what (GPU
identity, read-only), with which requests (case manifests, batch expansion, synthetic media,
exact content-reuse workloads) and how much device memory the process held (reference
``benchmarks/harness.py``, ``benchmarks/multimodal_cache_workload.py`` and the per-process NVML
sampler of ``benchmarks/bench_external_prism.py:79-157``).

Keeping these in one module keeps the records of different runners comparable: they name the
source tree, the GPU and the workload in the same way.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import threading
import time
from copy import deepcopy
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Mapping, Sequence

import numpy as np

REPO_ROOT = Path(__file__).resolve().parents[1]
SOURCE_SUFFIXES = (".py", ".cu", ".cuh", ".h", ".json")
MEDIA_KEYS = ("image", "images", "video")


# ---------------------------------------------------------------------------- source identity
@dataclass(frozen=True)
class SourceIdentity:
    commit: str | None      # git HEAD, when the tree is a checkout
    dirty: bool | None      # uncommitted changes to tracked files
    tree_sha256: str        # digest over the package, benchmark and bench sources as they are on disk
    files: int

    def to_record(self) -> dict[str, Any]:
        return asdict(self)


def source_tree_sha256(root: str | Path = REPO_ROOT) -> tuple[str, int]:
    """Digest of (relative path, content) of every source file under the package and the
    benchmarks: identifies the code also where no ``.git`` travels with it."""
    root = Path(root)
    paths = sorted(p for top in ("prism_infer_b200", "benchmarks") if (root / top).is_dir()
                   for p in (root / top).rglob("*") if p.is_file() and p.suffix in SOURCE_SUFFIXES and "build" not in p.parts)
    paths += [p for p in (root / "bench.py", root / "__graft_entry__.py") if p.is_file()]
    h = hashlib.sha256()
    for p in paths:
        h.update(p.relative_to(root).as_posix().encode() + b"\0")
        h.update(hashlib.sha256(p.read_bytes()).digest())
    return h.hexdigest(), len(paths)


def collect_source_identity(root: str | Path = REPO_ROOT) -> SourceIdentity:
    def git(*args: str) -> str | None:
        try:
            r = subprocess.run(["git", "-C", str(root), *args], capture_output=True, text=True, timeout=20)
        except (OSError, subprocess.TimeoutExpired):
            return None
        return r.stdout.strip() if r.returncode == 0 else None

    commit = git("rev-parse", "HEAD")
    status = git("status", "--porcelain", "--untracked-files=no") if commit else None
    digest, n = source_tree_sha256(root)
    return SourceIdentity(commit, None if status is None else bool(status), digest, n)


# ------------------------------------------------------------------------------- GPU identity
GPU_QUERY = ("index", "name", "uuid", "driver_version", "memory.total", "clocks.max.sm", "clocks.max.memory", "power.limit")


@dataclass(frozen=True)
class GpuIdentity:
    index: int
    name: str
    uuid: str
    driver_version: str
    memory_total_mib: float | None
    sm_max_mhz: float | None
    memory_max_mhz: float | None
    power_limit_w: float | None
    compute_capability: str | None = None
    multiprocessors: int | None = None

    def to_record(self) -> dict[str, Any]:
        return asdict(self)


def _float(raw: str) -> float | None:
    try:
        return float(raw)
    except ValueError:
        return None


def parse_gpu_query(csv_text: str) -> list[GpuIdentity]:
    """Rows of ``nvidia-smi --query-gpu=<GPU_QUERY> --format=csv,noheader,nounits``."""
    out = []
    for line in csv_text.strip().splitlines():
        cells = [c.strip() for c in line.split(",")]
        if len(cells) != len(GPU_QUERY):
            raise ValueError(f"unexpected nvidia-smi row: {line!r}")
        out.append(GpuIdentity(int(cells[0]), cells[1], cells[2], cells[3], _float(cells[4]), _float(cells[5]), _float(cells[6]),
                               _float(cells[7])))
    return out


def collect_gpu_identity(device_index: int = 0) -> GpuIdentity | None:
    """Reads the GPU's identity; changes nothing.  ``None`` without a GPU."""
    try:
        r = subprocess.run(["nvidia-smi", f"--query-gpu={','.join(GPU_QUERY)}", "--format=csv,noheader,nounits"],
                           capture_output=True, text=True, timeout=30)
    except (OSError, subprocess.TimeoutExpired):
        return None
    if r.returncode != 0 or not r.stdout.strip():
        return None
    rows = parse_gpu_query(r.stdout)
    visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    physical = device_index
    if visible and all(v.strip().isdigit() for v in visible.split(",")):
        ids = [int(v) for v in visible.split(",")]
        physical = ids[device_index] if device_index < len(ids) else device_index
    gpu = next((g for g in rows if g.index == physical), rows[0])
    try:
        import torch

        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(device_index)
            gpu = GpuIdentity(**{**asdict(gpu), "compute_capability": f"{p.major}.{p.minor}", "multiprocessors": p.multi_processor_count})
    except Exception:  # identity stays the nvidia-smi view
        pass
    return gpu


# --------------------------------------------------------------------------- workload manifests
def find_workload_case(manifest: Mapping[str, Any], case_id: str) -> dict[str, Any]:
    for case in manifest["cases"]:
        if case["id"] == case_id:
            return case
    raise ValueError(f"unknown case {case_id!r}; available cases: {[c['id'] for c in manifest['cases']]}")


def expand_case_batch(case: Mapping[str, Any], batch_size: int) -> tuple[dict[str, Any], int, int]:
    """Repeat the case's whole request list until it has ``batch_size`` requests ->
    ``(expanded case, source size, replication factor)``."""
    n = len(case["requests"])
    if batch_size < n or batch_size % n:
        raise ValueError(f"batch size must be a positive multiple of the source case size: case={case['id']}, source={n}, "
                         f"requested={batch_size}")
    k = batch_size // n
    out = deepcopy(dict(case))
    out["requests"] = [deepcopy(r) for _ in range(k) for r in case["requests"]]
    return out, n, k


def make_image(spec: Mapping[str, Any]) -> np.ndarray:
    """``{"width", "height"}`` plus either ``"color": [r, g, b]`` (flat) or ``"seed"`` (uniform noise)."""
    h, w = int(spec["height"]), int(spec["width"])
    if "seed" in spec:
        return np.random.default_rng(int(spec["seed"])).integers(0, 256, (h, w, 3), dtype=np.uint8)
    return np.broadcast_to(np.asarray(spec.get("color", (128, 128, 128)), dtype=np.uint8), (h, w, 3)).copy()


def load_file_image(spec: Mapping[str, Any], base: str | Path) -> np.ndarray:
    """An ``image_file`` spec: the file below ``base`` whose bytes hash to ``sha256`` and whose size is as recorded."""
    import hashlib
    import io

    from PIL import Image

    data = (Path(base) / spec["path"]).read_bytes()
    if hashlib.sha256(data).hexdigest() != spec["sha256"]:
        raise ValueError(f"{spec['path']}: content differs from the manifest's sha256")
    with Image.open(io.BytesIO(data)) as im:
        arr = np.asarray(im.convert("RGB"))
    if arr.shape[:2] != (int(spec["height"]), int(spec["width"])):
        raise ValueError(f"{spec['path']}: {arr.shape[1]}x{arr.shape[0]} pixels, the manifest records {spec['width']}x{spec['height']}")
    return arr


def load_manifest(path: str | Path) -> dict[str, Any]:
    """Read and validate a workload manifest (``analysis/workload_manifest.py``)."""
    from prism_infer_b200.analysis.workload_manifest import load_workload_manifest

    return load_workload_manifest(path)


def materialize_requests(case: Mapping[str, Any], base: str | Path | None = None) -> list[dict[str, Any]]:
    """Case requests -> payloads for ``LLM.generate_mixed`` (``type`` in text / image / images /
    interleaved_images / video; an ``image_file`` request becomes an ``image`` payload read below ``base``)."""
    out = []
    for r in case["requests"]:
        kind = r["type"]
        p: dict[str, Any] = {"type": "image" if kind == "image_file" else kind, "prompt": r["prompt"]}
        if kind == "image":
            p["image"] = make_image(r["image"])
        elif kind == "image_file":
            if base is None:
                raise ValueError("an image_file request needs the manifest's directory")
            p["image"] = load_file_image(r["image"], base)
        elif kind in ("images", "interleaved_images"):
            p["images"] = [make_image(s) for s in r["images"]]
        elif kind == "video":
            p["video"] = [make_image(s) for s in r["frames"]]
        elif kind != "text":
            raise ValueError(f"unknown request type {kind!r}")
        out.append(p)
    return out


def describe_case_inputs(case: Mapping[str, Any]) -> dict[str, Any]:
    """Shapes and counts without creating any pixels."""
    shapes, images, videos, frames = [], 0, 0, 0
    for r in case["requests"]:
        specs: Sequence[Mapping[str, Any]] = ()
        if r["type"] in ("image", "image_file"):
            specs, images = [r["image"]], images + 1
        elif r["type"] in ("images", "interleaved_images"):
            specs, images = r["images"], images + len(r["images"])
        elif r["type"] == "video":
            specs, videos, frames = r["frames"], videos + 1, frames + len(r["frames"])
        shapes.append({"type": r["type"], "visual_shapes": [[int(s["height"]), int(s["width"]), 3] for s in specs]})
    return {"input_shapes": shapes, "images": images, "videos": videos, "video_frames": frames}


# --------------------------------------------------------------------- content-reuse workloads
def _mark(image: np.ndarray, variant: int) -> np.ndarray:
    """A copy whose top-left 8 x 8 block encodes ``variant`` as 64 black / white pixels: distinct
    content, same shape."""
    out = np.array(image, copy=True)
    bits = np.array([(variant >> b) & 1 for b in range(64)], dtype=np.uint8).reshape(8, 8) * 255
    out[:8, :8, :] = bits[:, :, None]
    return out


def _copy_media(value: Any, variant: int | None) -> Any:
    if isinstance(value, (list, tuple)):
        items = [np.array(v, copy=True) for v in value]
        if variant is not None and items:
            items[0] = _mark(items[0], variant)
        return items
    return np.array(value, copy=True) if variant is None else _mark(np.asarray(value), variant)


def build_multimodal_cache_workload(payloads: Sequence[Mapping[str, Any]], *, repeat_rate: float,
                                    vary_questions: bool) -> tuple[list[dict[str, Any]], dict[str, Any]]:
    """Give exactly ``round(n * repeat_rate)`` of the ``n`` multimodal payloads byte-identical
    media (in fresh arrays, so only content addressing can recognise them) and every other one
    a unique marker; repeats are spread evenly over the sequence."""
    if not 0.0 <= repeat_rate <= 1.0:
        raise ValueError(f"repeat_rate must be in [0, 1], got {repeat_rate}")
    n = sum(1 for p in payloads if any(k in p for k in MEDIA_KEYS))
    repeats = round(n * repeat_rate)
    out, i = [], 0
    for p in payloads:
        q = dict(p)
        if not any(k in p for k in MEDIA_KEYS):
            out.append(q)
            continue
        repeated = (i + 1) * repeats // n > i * repeats // n
        for k in MEDIA_KEYS:
            if k in p:
                q[k] = _copy_media(p[k], None if repeated else i + 1)
        if vary_questions:
            q["prompt"] = f"{str(p['prompt']).rstrip()}\nAnswer request variant {i + 1} concisely."
        out.append(q)
        i += 1
    return out, {"media_requests": n, "requested_repeat_rate": repeat_rate, "repeated_media_requests": repeats,
                 "unique_media_requests": n - repeats, "realized_repeat_rate": repeats / n if n else None,
                 "media_object_policy": "fresh_arrays_per_request", "unique_media_policy": "binary_marker_in_first_frame",
                 "question_policy": "different_suffix" if vary_questions else "original_question"}


# ------------------------------------------------------------------------ process GPU memory
class GpuMemorySampler:
    """Background thread that samples this process's device memory through NVML (read-only)
    every ``period_s`` and keeps the peak.  ``nvml`` is injectable for tests."""

    def __init__(self, device_index: int = 0, pid: int | None = None, period_s: float = 0.01, nvml: Any = None) -> None:
        self.device_index, self.pid, self.period_s = device_index, pid or os.getpid(), period_s
        self._nvml = nvml
        self.samples = 0
        self.peak_bytes = 0
        self.last_bytes = 0
        self.error: str | None = None
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _read(self, handle: Any) -> int:
        procs = self._nvml.nvmlDeviceGetComputeRunningProcesses(handle)
        return sum(int(p.usedGpuMemory or 0) for p in procs if int(p.pid) == self.pid)

    def _run(self) -> None:
        try:
            self._nvml.nvmlInit()
            handle = self._nvml.nvmlDeviceGetHandleByIndex(self.device_index)
            while not self._stop.is_set():
                self.last_bytes = self._read(handle)
                self.peak_bytes = max(self.peak_bytes, self.last_bytes)
                self.samples += 1
                self._stop.wait(self.period_s)
        except Exception as exc:  # a sampler must never take the benchmark down
            self.error = f"{type(exc).__name__}: {exc}"
        finally:
            try:
                self._nvml.nvmlShutdown()
            except Exception:
                pass

    def __enter__(self) -> "GpuMemorySampler":
        if self._nvml is None:
            try:
                import pynvml

                self._nvml = pynvml
            except Exception as exc:
                self.error = f"NVML unavailable: {exc}"
                return self
        self._thread = threading.Thread(target=self._run, name="gpu-memory-sampler", daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc: Any) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5.0)

    def to_record(self) -> dict[str, Any]:
        return {"pid": self.pid, "device_index": self.device_index, "period_s": self.period_s, "samples": self.samples,
                "peak_bytes": self.peak_bytes, "last_bytes": self.last_bytes, "error": self.error}


def provenance(device_index: int = 0) -> dict[str, Any]:
    """Block that a benchmark record carries under ``"provenance"``."""
    gpu = collect_gpu_identity(device_index)
    return {"source": collect_source_identity().to_record(), "gpu": None if gpu is None else gpu.to_record(),
            "unix_time": time.time()}
