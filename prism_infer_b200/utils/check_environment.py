"""``python -m prism_infer_b200.utils.check_environment``: what this machine offers and whether a planned run can start.

The report covers the Python distributions the package leans on, the in-tree kernel library (present, loadable, built
for which sources), the CUDA devices with their free memory, the run that is planned (execution backend, KV mode,
tensor-parallel size, page budget) and, with ``--model``, the checkpoint directory (required files, safetensors shards,
that its configuration is a Qwen3-VL one and which sharded dimensions the tensor-parallel size has to divide).
Failures make the exit status non-zero; warnings do not.  ``--json`` prints the machine-readable report only.  Nothing is
loaded onto a GPU.  The reference ships the same kind of tool as ``scripts/check_environment.py``.

    python -m prism_infer_b200.utils.check_environment --model /path/to/Qwen3-VL-8B-Instruct --tensor-parallel-size 8 \\
        --execution-backend cuda_graph --compression-mode scaled_fp8_kv --min-free-gib 40
"""

from __future__ import annotations

import argparse
import hashlib
import importlib
import importlib.metadata
import json
import os
import sys
from pathlib import Path
from typing import Any

GIB = float(1 << 30)
CORE_DISTRIBUTIONS = ("torch", "numpy", "safetensors")
OPTIONAL_DISTRIBUTIONS = ("transformers", "tokenizers", "pillow", "fastapi", "uvicorn", "pydantic", "pyarrow", "opencv-python-headless")
CHECKPOINT_FILES = ("config.json",)
CHECKPOINT_FILES_RECOMMENDED = ("tokenizer_config.json", "preprocessor_config.json")


def distribution_versions(names) -> dict[str, str | None]:
    out = {}
    for name in names:
        try:
            out[name] = importlib.metadata.version(name)
        except importlib.metadata.PackageNotFoundError:
            out[name] = None
    return out


def sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        for chunk in iter(lambda: fh.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def inspect_checkpoint(model: str | None, tp: int) -> tuple[dict[str, Any], list[str], list[str]]:
    """Files, identity and tensor-parallel divisibility of a checkpoint directory -> (report, errors, warnings)."""
    if not model:
        return {"status": "not_checked", "path": None}, [], []
    if model.startswith("random:"):
        from ..config import resolve_arch
        from ..models.architecture import validate_tensor_parallel

        errors: list[str] = []
        try:
            arch = resolve_arch(model)
            validate_tensor_parallel(arch, tp)
        except Exception as exc:  # unknown preset or a size the preset cannot be split into
            errors.append(f"{model}: {exc}")
        return {"status": "fail" if errors else "pass", "path": model, "kind": "random-init preset"}, errors, []
    path = Path(model).expanduser()
    rep: dict[str, Any] = {"status": "fail", "path": str(path)}
    if not path.is_dir():
        return rep, [f"model directory does not exist: {path}"], []
    errors, warnings = [], []
    missing = [n for n in CHECKPOINT_FILES if not (path / n).is_file()]
    if missing:
        errors.append(f"checkpoint is missing {', '.join(missing)}")
    absent = [n for n in CHECKPOINT_FILES_RECOMMENDED if not (path / n).is_file()]
    if absent:
        warnings.append(f"checkpoint has no {', '.join(absent)}: prompts will use the built-in id tokenizer / patch processor")
    shards = sorted(path.glob("*.safetensors"))
    if not shards:
        errors.append("checkpoint holds no *.safetensors file")
    config: dict[str, Any] = {}
    if (path / "config.json").is_file():
        try:
            config = json.loads((path / "config.json").read_text(encoding="utf-8"))
        except (OSError, json.JSONDecodeError) as exc:
            errors.append(f"config.json cannot be read: {exc}")
    model_type, archs = config.get("model_type"), config.get("architectures") or []
    if config and model_type != "qwen3_vl" and not any("Qwen3VL" in str(a) for a in archs):
        errors.append(f"config.json does not describe a Qwen3-VL model (model_type={model_type!r}, architectures={archs!r})")
    if config and not errors:
        from ..models.architecture import Qwen3VLArch, validate_tensor_parallel

        try:
            arch = Qwen3VLArch.from_hf_config(config)
            validate_tensor_parallel(arch, tp)
            rep["text"] = {"layers": arch.text.num_layers, "hidden": arch.text.hidden_size, "heads": arch.text.num_heads,
                           "kv_heads": arch.text.num_kv_heads, "head_dim": arch.text.head_dim, "vocabulary": arch.text.vocab_size}
            rep["vision"] = {"depth": arch.vision.depth, "hidden": arch.vision.hidden_size, "heads": arch.vision.num_heads}
        except Exception as exc:
            errors.append(f"configuration rejected: {exc}")
    rep.update({"status": "fail" if errors else "pass", "model_type": model_type, "architectures": list(archs),
                "config_sha256": sha256_file(path / "config.json") if (path / "config.json").is_file() else None,
                "weight_files": len(shards), "weight_gib": round(sum(s.stat().st_size for s in shards) / GIB, 3),
                "missing_files": missing + absent})
    return rep, errors, warnings


def inspect_cuda(torch_module: Any) -> dict[str, Any]:
    """Devices and the memory free for this process; no context is created on devices that are not queried."""
    rep: dict[str, Any] = {"available": bool(torch_module.cuda.is_available()), "torch_cuda_version": torch_module.version.cuda,
                           "device_count": 0, "devices": []}
    if not rep["available"]:
        return rep
    rep["device_count"] = torch_module.cuda.device_count()
    for i in range(rep["device_count"]):
        props = torch_module.cuda.get_device_properties(i)
        free, total = torch_module.cuda.mem_get_info(i)
        rep["devices"].append({"index": i, "name": props.name, "capability": list(torch_module.cuda.get_device_capability(i)),
                               "multiprocessors": props.multi_processor_count, "free_gib": round(free / GIB, 3),
                               "total_gib": round(total / GIB, 3)})
    return rep


def inspect_kernel_library() -> tuple[dict[str, Any], list[str]]:
    from ..ops import build, native

    lib = Path(build.LIB)
    rep: dict[str, Any] = {"path": str(lib), "present": lib.is_file(), "loadable": False}
    problems = []
    if lib.is_file():
        rep["bytes"] = lib.stat().st_size
        newer = [s for s in sorted(Path(build.CSRC).glob("*.cu*")) if s.stat().st_mtime > lib.stat().st_mtime]
        rep["sources_newer_than_library"] = [s.name for s in newer]
        if newer:
            problems.append(f"kernel sources changed after the library was built ({', '.join(s.name for s in newer[:4])}): "
                            "run python -m prism_infer_b200.ops.build")
    rep["loadable"] = bool(native.available())
    return rep, problems


def build_report(args: argparse.Namespace) -> tuple[dict[str, Any], list[str], list[str]]:
    errors: list[str] = []
    warnings: list[str] = []
    core, optional = distribution_versions(CORE_DISTRIBUTIONS), distribution_versions(OPTIONAL_DISTRIBUTIONS)
    lacking = [n for n, v in core.items() if v is None]
    if lacking:
        errors.append(f"missing core distributions: {', '.join(lacking)}")
    for name, version in optional.items():
        if version is None:
            warnings.append(f"optional distribution {name} is not installed")
    report: dict[str, Any] = {"python": sys.version.split()[0], "platform": sys.platform, "distributions": {**core, **optional},
                              "planned_run": {"execution_backend": args.execution_backend, "compression_mode": args.compression_mode,
                                              "tensor_parallel_size": args.tensor_parallel_size, "require_cuda": args.require_cuda}}
    try:
        torch_module = importlib.import_module("torch")
    except Exception as exc:
        errors.append(f"cannot import torch: {type(exc).__name__}: {exc}")
        report["status"] = "fail"
        return report, errors, warnings
    report["cuda"] = cuda = inspect_cuda(torch_module)
    report["kernel_library"], stale = inspect_kernel_library()
    warnings.extend(stale)
    from ..runtime_capabilities import probe_runtime_capabilities, validate_runtime_capabilities

    probe = probe_runtime_capabilities(require_cuda=args.require_cuda)
    cap: dict[str, Any] = {"observed": {k: (list(v) if isinstance(v, tuple) else v) for k, v in probe.__dict__.items() if k != "problems"}}
    try:
        validate_runtime_capabilities(args.require_cuda, execution_backend=args.execution_backend,
                                      compression_mode=args.compression_mode, report=probe)
        cap["status"] = "pass"
    except RuntimeError as exc:
        cap["status"] = "fail"
        errors.append(str(exc))
    report["capabilities"] = cap
    tp = args.tensor_parallel_size
    if tp > 1 and args.require_cuda and cuda["device_count"] < tp:
        errors.append(f"tensor_parallel_size={tp} needs {tp} visible CUDA devices, {cuda['device_count']} found")
    if args.min_free_gib is not None:
        short = [d for d in cuda["devices"][:max(1, tp)] if d["free_gib"] < args.min_free_gib]
        if not cuda["devices"]:
            errors.append("--min-free-gib needs at least one visible CUDA device")
        for d in short:
            errors.append(f"GPU {d['index']} has {d['free_gib']:.1f} GiB free; {args.min_free_gib:.1f} GiB asked for")
    report["model"], model_errors, model_warnings = inspect_checkpoint(args.model, tp)
    errors.extend(model_errors)
    warnings.extend(model_warnings)
    if report["model"].get("weight_gib") and cuda["devices"]:
        per_rank = report["model"]["weight_gib"] / max(1, tp)
        if per_rank > min(d["free_gib"] for d in cuda["devices"][:max(1, tp)]):
            errors.append(f"the weights need about {per_rank:.1f} GiB per rank, more than a device has free")
    report["status"] = "fail" if errors else "pass"
    report["errors"], report["warnings"] = list(errors), list(warnings)
    return report, errors, warnings


def print_human(report: dict[str, Any]) -> None:
    w = sys.stdout.write
    w(f"python {report['python']} on {report['platform']}\n")
    for name, version in report["distributions"].items():
        w(f"  {name:<26} {version or 'not installed'}\n")
    cuda = report.get("cuda", {})
    w(f"CUDA available: {cuda.get('available')} (torch built for CUDA {cuda.get('torch_cuda_version')}), {cuda.get('device_count', 0)} device(s)\n")
    for d in cuda.get("devices", []):
        w(f"  [{d['index']}] {d['name']} sm_{d['capability'][0]}{d['capability'][1]} {d['multiprocessors']} SMs "
          f"{d['free_gib']:.1f} / {d['total_gib']:.1f} GiB free\n")
    lib = report.get("kernel_library", {})
    w(f"kernel library: {'present' if lib.get('present') else 'missing'}, {'loadable' if lib.get('loadable') else 'not loadable'} ({lib.get('path')})\n")
    run = report["planned_run"]
    w(f"planned run: backend {run['execution_backend']}, KV mode {run['compression_mode']}, {run['tensor_parallel_size']} rank(s): "
      f"{report.get('capabilities', {}).get('status', 'not checked')}\n")
    model = report.get("model", {})
    if model.get("path"):
        w(f"model {model['path']}: {model['status']}")
        if "weight_gib" in model:
            w(f", {model['weight_files']} safetensors file(s), {model['weight_gib']} GiB")
        w("\n")
    for msg in report.get("warnings", []):
        w(f"warning: {msg}\n")
    for msg in report.get("errors", []):
        w(f"ERROR: {msg}\n")
    w(f"result: {report['status'].upper()}\n")


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=os.environ.get("PRISM_MODEL_PATH"), help="checkpoint directory or a random:<preset> name")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--execution-backend", default="cuda_graph", choices=("eager", "cuda_graph", "compile", "compile_graph"))
    ap.add_argument("--compression-mode", default="scaled_fp8_kv")
    ap.add_argument("--min-free-gib", type=float, default=None, help="free memory every rank's device must have")
    ap.add_argument("--allow-cpu", dest="require_cuda", action="store_false", help="do not fail when no CUDA device is visible")
    ap.add_argument("--json", action="store_true", help="print the report as JSON only")
    args = ap.parse_args(argv)
    if args.tensor_parallel_size < 1:
        ap.error("--tensor-parallel-size must be positive")
    return args


def main(argv=None) -> int:
    args = parse_args(argv)
    report, errors, _ = build_report(args)
    if args.json:
        print(json.dumps(report, indent=1, sort_keys=True, default=str))
    else:
        print_human(report)
    return 1 if errors else 0


if __name__ == "__main__":
    raise SystemExit(main())
