"""Symmetric device memory across the tensor-parallel ranks of one node.

Every rank allocates an identically laid out region with ``cudaMalloc`` (through the kernel
library), exports it with CUDA IPC, and maps all peers' regions, which yields plain peer
pointers kernels can store to and load from over NVLink.  Handles travel through
``torch.distributed.all_gather_object`` once at start-up; nothing else uses the process
group on the fused paths.  The reference has no such layer (NCCL only).

Region layout (bytes)::

    0     flags of exchange slot 0   u64[8]      256   flags of slot 1   u64[8]
    512   flags of the arg-max exchange u64[8]   768   step epoch word   u64
    1024  CTA counter slot 0  i32                1280  CTA counter slot 1  i32
    1344  CTA counter of the vision all-gather  1536  vision flags: 2 sets x 4 outputs x u64[8]
    4096  arg-max values f32[8][BMAX]            then  arg-max ids i64[8][BMAX]
    2048  prefill reduce-scatter flags: 2 slots x u64[8]   2176  prefill all-gather flags: 2 slots x u64[8]
    2304  CTA counters of the prefill scatter GEMM and of the reduce + norm + all-gather kernel
    SLAB0 / SLAB1: two slab buffers of  tp * S_MAX * T_MAX * H  8-byte {fp32 value, sequence} words each
    VIS: 2 sets x 4 outputs x VIS_T_MAX x H bf16 (gathered merger outputs of the vision tower)
    PRE: 2 slots x (reduce-scatter slabs tp x ceil(PRE_T_MAX / tp) x H bf16, all-gathered rows PRE_T_MAX x H bf16)
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ..ops import native

T_MAX = 128
S_MAX = 4
B_MAX = 512
OFF_FLAGS = (0, 256)
OFF_ARGMAX_FLAGS = 512
OFF_EPOCH = 768
OFF_COUNTER = (1024, 1280)
OFF_VIS_COUNTER = 1344
OFF_VIS_FLAGS = 1536          # 8 arrays (2 buffer sets x 4 outputs) of u64[8]
VIS_OUTPUTS = 4               # main merger + up to three DeepStack mergers
VIS_T_MAX = 4096              # merged visual tokens per vision-tower call on the fused path
OFF_PRE_RS_FLAGS = (2048, 2112)
OFF_PRE_AG_FLAGS = (2176, 2240)
OFF_PRE_COUNTER = (2304, 2368)  # scatter GEMM, reduce + norm + all-gather kernel
PRE_T_MAX = 8192              # prefill tokens per step on the fused tensor-parallel path
OFF_ARGMAX_VAL = 4096
OFF_ARGMAX_ID = OFF_ARGMAX_VAL + 8 * B_MAX * 4
OFF_SLABS = (OFF_ARGMAX_ID + 8 * B_MAX * 8 + 4095) // 4096 * 4096
POINTS_PER_STEP = 128
ARGMAX_POINT = POINTS_PER_STEP - 1


def _pre_bytes(size: int, hidden: int) -> tuple[int, int]:
    """(reduce-scatter slab bytes, all-gather bytes) of one prefill slot."""
    rows = -(-PRE_T_MAX // size)
    return size * rows * hidden * 2, PRE_T_MAX * hidden * 2


def _region_bytes(size: int, hidden: int, slab_bytes: int) -> int:
    rs, ag = _pre_bytes(size, hidden)
    return OFF_SLABS + 2 * slab_bytes + 2 * VIS_OUTPUTS * VIS_T_MAX * hidden * 2 + 2 * (rs + ag)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise native.NativeError(f"{what} failed with cudaError {rc}")


class _DevView:
    """Exposes a raw device range to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


@dataclass
class SymmetricRegion:
    rank: int
    size: int
    hidden: int
    local_ptr: int
    peer_ptrs: list[int]          # device addresses of every rank's region as seen from this rank
    nbytes: int
    slab_bytes: int

    @classmethod
    def create(cls, rank: int, size: int, hidden: int, group=None) -> "SymmetricRegion":
        import torch.distributed as dist

        lib = native.lib()
        slab_bytes = size * S_MAX * T_MAX * hidden * 8
        nbytes = _region_bytes(size, hidden, slab_bytes)
        out = ctypes.c_void_p()
        _check(lib.prism_ipc_alloc(nbytes, ctypes.byref(out)), "prism_ipc_alloc")
        handle = (ctypes.c_char * 64)()
        _check(lib.prism_ipc_get_handle(out, ctypes.cast(handle, ctypes.c_void_p)), "prism_ipc_get_handle")
        handles: list[bytes] = [b""] * size
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        peers: list[int] = []
        for r in range(size):
            if r == rank:
                peers.append(out.value)
                continue
            mapped = ctypes.c_void_p()
            buf = (ctypes.c_char * 64).from_buffer_copy(handles[r])
            _check(lib.prism_ipc_open_handle(ctypes.cast(buf, ctypes.c_void_p), ctypes.byref(mapped)), "prism_ipc_open_handle")
            peers.append(mapped.value)
        dist.barrier(group=group)
        return cls(rank, size, hidden, out.value, peers, nbytes, slab_bytes)

    @classmethod
    def create_emulated(cls, size: int, hidden: int) -> list["SymmetricRegion"]:
        """All ranks' regions on the current device (single-GPU tests of the fused kernels)."""
        lib = native.lib()
        slab_bytes = size * S_MAX * T_MAX * hidden * 8
        nbytes = _region_bytes(size, hidden, slab_bytes)
        ptrs = []
        for _ in range(size):
            out = ctypes.c_void_p()
            _check(lib.prism_ipc_alloc(nbytes, ctypes.byref(out)), "prism_ipc_alloc")
            ptrs.append(out.value)
        return [cls(r, size, hidden, ptrs[r], list(ptrs), nbytes, slab_bytes) for r in range(size)]

    # ---- typed local views ---------------------------------------------------------
    def local_bytes(self) -> torch.Tensor:
        return torch.as_tensor(_DevView(self.local_ptr, self.nbytes), device="cuda")

    def slabs(self, slot: int, groups: int, tokens: int) -> torch.Tensor:
        """Local view ``[groups, tokens, hidden, 2]`` (fp32 value, int32 sequence as raw bits) at the
        start of slab buffer ``slot``; ``[..., 0]`` are the values."""
        n = groups * tokens * self.hidden
        raw = self.local_bytes()[OFF_SLABS + slot * self.slab_bytes: OFF_SLABS + slot * self.slab_bytes + n * 8]
        return raw.view(torch.float32).view(groups, tokens, self.hidden, 2)

    def vis_offset(self, buffer_set: int, output: int) -> int:
        return OFF_SLABS + 2 * self.slab_bytes + (buffer_set * VIS_OUTPUTS + output) * VIS_T_MAX * self.hidden * 2

    def vis_rows(self, buffer_set: int, output: int, rows: int) -> torch.Tensor:
        """Local bf16 view ``[rows, hidden]`` of one gathered vision output."""
        off = self.vis_offset(buffer_set, output)
        raw = self.local_bytes()[off: off + rows * self.hidden * 2]
        return raw.view(torch.bfloat16).view(rows, self.hidden)

    def pre_offsets(self, slot: int) -> tuple[int, int]:
        """Byte offsets of (reduce-scatter slabs, all-gathered rows) of prefill slot ``slot``."""
        rs, ag = _pre_bytes(self.size, self.hidden)
        base = OFF_SLABS + 2 * self.slab_bytes + 2 * VIS_OUTPUTS * VIS_T_MAX * self.hidden * 2 + slot * (rs + ag)
        return base, base + rs

    def pre_rows(self, slot: int, rows: int) -> torch.Tensor:
        """Local bf16 view ``[rows, hidden]`` of the all-gathered activations of a prefill slot."""
        off = self.pre_offsets(slot)[1]
        raw = self.local_bytes()[off: off + rows * self.hidden * 2]
        return raw.view(torch.bfloat16).view(rows, self.hidden)

    # ---- pointer tables for the launchers ------------------------------------------------
    def ptr_array(self, offset: int):
        arr = (ctypes.c_void_p * 8)()
        for r in range(self.size):
            arr[r] = self.peer_ptrs[r] + offset
        return arr

    def local(self, offset: int) -> int:
        return self.local_ptr + offset

    def close(self) -> None:
        lib = native.lib()
        for r, p in enumerate(self.peer_ptrs):
            if r != self.rank and p != self.local_ptr:
                lib.prism_ipc_close_handle(ctypes.c_void_p(p))
        lib.prism_ipc_free(ctypes.c_void_p(self.local_ptr))
