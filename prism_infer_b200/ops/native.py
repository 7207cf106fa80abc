"""ctypes binding of ``libprism_b200.so`` (the sm_100a kernel library).

The library is built in-tree by ``prism_infer_b200.ops.build``.  On a machine with a CUDA
device a missing or unloadable library is a hard error: there is no silent PyTorch
fallback for CUDA tensors.  Every launcher returns ``0`` or an error code which is turned
into an exception here.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libprism_b200.so")

_lib = None
_lock = threading.Lock()
_launches = 0  # kernels launched through this binding (bench.py reports it)

_T = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "f": ctypes.c_float,
      "u": ctypes.c_ulonglong}

# name -> argument signature (p pointer, i int, l int64, f float, u uint64)
_SIGNATURES = {
    "prism_gemm_wx": "pppiiilllippliiiiiliipi",
    "prism_gemm_effective_splits": "ii",
    "prism_gemm_clear_tensor_maps": "",
    "prism_add_rmsnorm": "plipppppppiifpi",
    "prism_layernorm": "ppppiifpi",
    "prism_qk_norm_rope_store": "pplilpppppplpppppiiiiiiiifipi",
    "prism_swiglu": "pplipiipi",
    "prism_embed": "pppppiillpi",
    "prism_indexed_add": "pppiipi",
    "prism_pos_embed_add": "ppppiipi",
    "prism_vit_rope": "pppiiipi",
    "prism_paged_decode": "pppppppppppiiiiiiiiifipi",
    "prism_flash_attention": "plplppplppppppiiiiiiiiiifpi",
    "prism_kv_page_copy": "ppllippllpppiiiip",
    "prism_kv_compact": "pliplppppiiiip",
    "prism_sample": "pllipppiilupppipi",
    "prism_merge_candidates": "pppiipi",
    "prism_lm_head_fp8_plan": "p",
    "prism_lm_head_fp8_candidates": "ppplpliiilpppppi",
    "prism_gemm_wx_push": "ppiiillliilppiilppiipi",
    "prism_add_rmsnorm_wait": "plippppppiifpipipi",
    "prism_gemm_wx_scatter": "ppiiillippiilpppi",
    "prism_reduce_norm_allgather": "ppliiiiiiplppppfpplpppi",
    "prism_add_rmsnorm_packed": "plippppppiifpipi",
    "prism_flash_attention_tc": "plpplplpiiiiiiifpi",
    "prism_paged_prefill_tc": "plplpppppppiiippiiiiiiiiifpi",
    "prism_gemm_set_small_tile_smem_cap": "i",
    "prism_gemm_set_persistent_min_tokens": "i",
    "prism_gemm_set_persistent_rowmajor": "i",
    "prism_gemm_wx_allgather": "ppiiillllpippiilpppi",
    "prism_signal_peers": "piilp",
    "prism_scatter_rows": "pliiiippiilpppi",
    "prism_wait_flags": "pilpp",
    "prism_ipc_alloc": "lp",
    "prism_ipc_free": "p",
    "prism_ipc_get_handle": "pp",
    "prism_ipc_open_handle": "pp",
    "prism_ipc_close_handle": "p",
    "prism_epoch_advance": "plpi",
    "prism_argmax_exchange": "ppppppppiiiiipi",
    "prism_decode_layers": "pip",
    "prism_decode_layer_desc": "ppipppiiipppppppp",
    "prism_decode_layers_plan": "iiiip",
    "prism_decode_layer_desc_bytes": "",
    "prism_decode_layers_max_tokens": "",
    "prism_decode_layers_timeline_stamps": "",
    "prism_decode_layers_seq_step": "i",
}
_STATUS_UNITS = ("gemm", "norm", "attn", "attn_tc", "kvops", "sampler", "comm", "decode_layers", "lm_head_fp8")


class NativeError(RuntimeError):
    pass


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise NativeError(
                        f"{LIB_PATH} is missing: run `python -m prism_infer_b200.ops.build` "
                        "(CUDA tensors never fall back to PyTorch ops)"
                    )
                handle = ctypes.CDLL(LIB_PATH)
                for name, sig in _SIGNATURES.items():
                    try:
                        fn = getattr(handle, name)
                    except AttributeError:
                        continue
                    fn.argtypes = [_T[c] for c in sig]
                    fn.restype = ctypes.c_int
                _lib = handle
    return _lib


def has_symbol(name: str) -> bool:
    try:
        getattr(lib(), name)
        return True
    except (AttributeError, NativeError):
        return False


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def call(name: str, *args) -> None:
    """Invoke a launcher; raise on a non-zero return."""
    global _launches
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        detail = ""
        if rc > 0:
            try:
                detail = f" ({torch.cuda.cudart().cudaGetErrorString(rc)})"  # type: ignore[attr-defined]
            except Exception:  # pragma: no cover - best effort
                detail = " (cudaError)"
        raise NativeError(f"{name} failed with code {rc}{detail}")
    _launches += 1


def launch_count() -> int:
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def read_status(reset: bool = True) -> dict[str, tuple[int, int, int, int]]:
    """Device status words of every translation unit: ``{unit: (code, detail, block, count)}``.

    Code 0 is healthy; 1 = an mbarrier wait ran out, 2 = a peer-flag wait ran out,
    3 = a bounds check failed.  Kernels never trap, so the context stays usable.
    """
    out: dict[str, tuple[int, int, int, int]] = {}
    handle = lib()
    buf = (ctypes.c_int * 4)()
    for unit in _STATUS_UNITS:
        try:
            fn = getattr(handle, f"prism_status_{unit}")
        except AttributeError:
            continue
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int]
        fn.restype = ctypes.c_int
        rc = fn(ctypes.cast(buf, ctypes.c_void_p), 1 if reset else 0)
        if rc != 0:
            raise NativeError(f"prism_status_{unit} failed with cudaError {rc}")
        out[unit] = (buf[0], buf[1], buf[2], buf[3])
    return out


def check_status() -> None:
    bad = {k: v for k, v in read_status().items() if v[0] != 0}
    if bad:
        raise NativeError(f"device status reports failures: {bad}")
