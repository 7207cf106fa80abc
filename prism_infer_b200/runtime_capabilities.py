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


def validate_runtime_capabilities(require_cuda: bool = True) -> CapabilityReport:
    rep = probe_runtime_capabilities(require_cuda)
    if not rep.ok:
        raise RuntimeError("runtime capability check failed: " + "; ".join(rep.problems))
    return rep
