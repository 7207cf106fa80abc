"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of this library may not allocate device memory at all (a serving loop with a
fixed memory plan, a plugin living inside another framework's pool, code running while a
CUDA graph is being captured).  ``prism_paged_decode_noalloc`` serves them: it keeps the
split-KV partial results in a fixed 4 MiB device array inside the library instead of in
scratch tensors the caller would have to allocate.  This test checks, on two calls in a
row that share that array, that it returns what the ordinary entry point returns, and that
a request beyond the built-in array is refused with a readable message.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""

import ctypes
import math

import pytest
import torch

from prism_infer_b200 import ops
from prism_infer_b200.ops import native

pytestmark = pytest.mark.gpu


def _symbol():
    lib = native.lib()
    fn = lib.prism_paged_decode_noalloc
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int] * 9 + [ctypes.c_float, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    err = lib.prism_noalloc_last_error
    err.argtypes = []
    err.restype = ctypes.c_char_p
    need = lib.prism_paged_decode_noalloc_scratch_bytes
    need.argtypes = [ctypes.c_int] * 4
    need.restype = ctypes.c_longlong
    return fn, err, need


def _call(fn, cache, q, bt, ctx, out, nsplit, B=None):
    B = q.shape[0] if B is None else B
    return fn(q.data_ptr(), cache.k(0).data_ptr(), cache.v(0).data_ptr(), cache.k_scale(0).data_ptr(),
              cache.v_scale(0).data_ptr(), bt.data_ptr(), ctx.data_ptr(), out.data_ptr(), B, q.shape[1],
              cache.num_kv_heads, q.shape[2], cache.page, bt.shape[1], cache.num_blocks, nsplit, cache.mode,
              1.0 / math.sqrt(q.shape[2]), torch.cuda.current_stream().cuda_stream)


def _case(seed, B, Hq, Hkv, D, page, blocks, mode, short_first=False):
    g = torch.Generator().manual_seed(seed)
    cache = ops.KVCache(1, blocks, Hkv, page, D, mode, "cuda")
    raw = torch.randn(2, 1, blocks, Hkv, page, D, generator=g)
    q8, scale = ops.quantize_fp8_rows(raw, True)
    cache.payload.copy_(q8)
    cache.scales.copy_(scale)
    ctx = torch.randint(1, 3 * page, (B,), generator=g, dtype=torch.int32)
    if short_first:
        ctx[0] = 5  # every split but the first is empty for this sequence
    maxblk = 4
    bt = torch.full((B, maxblk), -1, dtype=torch.int32)
    perm = torch.randperm(blocks, generator=g)
    c = 0
    for b in range(B):
        n = (int(ctx[b]) + page - 1) // page
        bt[b, :n] = perm[c:c + n].int()
        c += n
    q = (torch.randn(B, Hq, D, generator=g)).to(torch.bfloat16)
    return cache, q.cuda(), bt.cuda(), ctx.cuda()


def test_noalloc_decode_matches_regular_entry_point_twice(cuda_device):
    fn, err, need = _symbol()
    B, Hq, Hkv, D, page, nsplit = 6, 32, 8, 128, 256, 8
    assert need(B, Hq, D, nsplit) <= 4 << 20
    for seed in (1, 2):  # the second call reuses the array the first one left dirty
        cache, q, bt, ctx = _case(seed, B, Hq, Hkv, D, page, 24, ops.KV_FP8_SCALED)
        want = ops.paged_decode_attention(q, cache, 0, bt, ctx, nsplit=nsplit)
        out = torch.empty_like(q)
        rc = _call(fn, cache, q, bt, ctx, out, nsplit)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        diff = (out.float() - want.float()).abs()
        assert diff.max() < 2e-2 and diff.mean() < 2e-3, (diff.max(), diff.mean())
    # a third call with another batch and split count, so that the previous call's (max, sum)
    # words lie under this call's partial outputs, and one sequence whose later splits are empty
    B2, nsplit2 = 3, 5
    cache, q, bt, ctx = _case(7, B2, Hq, Hkv, D, page, 24, ops.KV_FP8_SCALED, short_first=True)
    want = ops.paged_decode_attention(q, cache, 0, bt, ctx, nsplit=nsplit2)
    out = torch.empty_like(q)
    assert _call(fn, cache, q, bt, ctx, out, nsplit2) == 0, err().decode()
    torch.cuda.synchronize()
    diff = (out.float() - want.float()).abs()
    assert diff.max() < 2e-2 and diff.mean() < 2e-3, (diff.max(), diff.mean())
    # a split count above the kernels' limit of 32 is clamped before the scratch is sized
    assert need(2, Hq, D, 1000) == need(2, Hq, D, 32)
    native.check_status()


def test_noalloc_decode_rejects_oversized_requests(cuda_device):
    fn, err, need = _symbol()
    B, Hq, Hkv, D, page, nsplit = 64, 32, 8, 128, 256, 32
    assert need(B, Hq, D, nsplit) > 4 << 20
    cache, q, bt, ctx = _case(3, 2, Hq, Hkv, D, page, 8, ops.KV_FP8_SCALED)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device="cuda")
    rc = _call(fn, cache, q, bt, ctx, out, nsplit, B=B)
    assert rc == -10
    msg = err().decode()
    assert "needs" in msg and "bytes" in msg
    # invalid head counts are refused with a code instead of dividing by zero on the host
    rc = fn(q.data_ptr(), cache.k(0).data_ptr(), cache.v(0).data_ptr(), cache.k_scale(0).data_ptr(),
            cache.v_scale(0).data_ptr(), bt.data_ptr(), ctx.data_ptr(), out.data_ptr(), 2, Hq, 0, D, page,
            bt.shape[1], cache.num_blocks, 4, cache.mode, 1.0, torch.cuda.current_stream().cuda_stream)
    assert rc == -13 and "Hkv" in err().decode()
