"""Fail-closed start-up probe (reference ``prism_infer/runtime_capabilities.py:18-197``).

The B200 build needs: PyTorch in the tested window, a CUDA device of compute capability
10.x, the in-tree kernel library, CUDA graphs, the E4M3 dtype and pinned host memory.
Nothing degrades silently: ``validate_runtime_capabilities`` raises with every unmet
requirement listed.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

MIN_TORCH = (2, 5)
MAX_TORCH_EXCLUSIVE = (2, 13)


@dataclass
class CapabilityReport:
    torch_version: str
    cuda_available: bool
    device_name: str | None = None
    compute_capability: tuple[int, int] | None = None
    kernel_library: bool = False
    fp8_dtype: bool = False
    cuda_graphs: bool = False
    problems: list[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return not self.problems


def _version_tuple(v: str) -> tuple[int, int]:
    parts = v.split("+")[0].split(".")
    return int(parts[0]), int(parts[1])


def probe_runtime_capabilities(require_cuda: bool = True) -> CapabilityReport:
    from .ops import native

    rep = CapabilityReport(torch.__version__, torch.cuda.is_available())
    tv = _version_tuple(torch.__version__)
    if not MIN_TORCH <= tv < MAX_TORCH_EXCLUSIVE:
        rep.problems.append(f"torch {torch.__version__} outside the supported window "
                            f"[{MIN_TORCH[0]}.{MIN_TORCH[1]}, {MAX_TORCH_EXCLUSIVE[0]}.{MAX_TORCH_EXCLUSIVE[1]})")
    rep.fp8_dtype = hasattr(torch, "float8_e4m3fn")
    if not rep.fp8_dtype:
        rep.problems.append("torch.float8_e4m3fn is missing")
    rep.kernel_library = native.available()
    if rep.cuda_available:
        rep.device_name = torch.cuda.get_device_name(0)
        rep.compute_capability = torch.cuda.get_device_capability(0)
        rep.cuda_graphs = hasattr(torch.cuda, "CUDAGraph")
        if rep.compute_capability[0] != 10:
            rep.problems.append(f"kernels are built for sm_100a; found compute capability {rep.compute_capability}")
        if not rep.kernel_library:
            rep.problems.append("libprism_b200.so is missing: run python -m prism_infer_b200.ops.build")
        if not rep.cuda_graphs:
            rep.problems.append("torch.cuda.CUDAGraph is unavailable")
    elif require_cuda:
        rep.problems.append("no CUDA device")
    return rep


def validate_runtime_capabilities(require_cuda: bool = True, *, execution_backend: str = "eager",
                                  compression_mode: str = "off", report: CapabilityReport | None = None) -> CapabilityReport:
    """Raise before any tokenizer, process or model side effect when the selected run cannot work
    here.  ``execution_backend`` and ``compression_mode`` add the requirements only that path has
    (graph capture, the E4M3 dtype); ``report`` injects a probe result (tests)."""
    rep = report or probe_runtime_capabilities(require_cuda)
    problems = list(rep.problems)
    if require_cuda and execution_backend in ("cuda_graph", "compile_graph") and rep.cuda_available and not rep.cuda_graphs:
        problems.append(f"execution backend {execution_backend!r} needs CUDA graphs")
    if "fp8" in compression_mode and not rep.fp8_dtype:
        problems.append(f"compression mode {compression_mode!r} needs torch.float8_e4m3fn")
    if problems:
        raise RuntimeError("runtime capability check failed: " + "; ".join(dict.fromkeys(problems)))
    return rep


def validate_tensor_parallel_environment(arch, tp: int, device_count: int, *, world_size: int = 1) -> None:
    """Hardware and sharding checks of a tensor-parallel run, before any process is spawned or
    communicator created (reference ``prism_infer/engine/llm_engine.py:117-143``): enough visible
    devices, an externally launched world of exactly ``tp`` ranks, every sharded dimension divisible."""
    from .models.architecture import validate_tensor_parallel

    validate_tensor_parallel(arch, tp)
    if tp <= 1:
        return
    if world_size > 1 and world_size != tp:
        raise RuntimeError(f"tensor_parallel_size={tp} but the launcher started WORLD_SIZE={world_size} ranks")
    if tp > device_count:
        raise RuntimeError(f"tensor_parallel_size={tp} requires at least {tp} visible CUDA devices, "
                           f"but only {device_count} are available")
