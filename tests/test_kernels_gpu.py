"""sm_100a kernels against the plain-PyTorch fp32 statement of the same op.

Every case runs the op twice through ``prism_infer_b200.ops``: on CUDA bf16 tensors (the
hand-written kernel) and on CPU fp32 tensors holding the same bf16-representable values
(the reference path).  Tolerances follow the reference's kernel tests
(tests/test_paged_decode_kernel.py:144-146, tests/test_scaled_fp8_kv_cache.py:399-472).
"""

import math

import pytest
import torch

from prism_infer_b200 import ops
from prism_infer_b200.ops import native

pytestmark = pytest.mark.gpu


def bf(x):
    return x.to(torch.bfloat16)


def rand_bf16(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return bf(torch.randn(*shape, generator=g) * scale)


def close(a, b, atol, rtol, what=""):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    assert bool((err <= lim).all()), f"{what}: max err {err.max().item():.4g}, worst ratio {(err / lim).max().item():.3g}"


@pytest.fixture(autouse=True)
def _status(cuda_device):
    yield
    torch.cuda.synchronize()
    native.check_status()


@pytest.mark.parametrize(
    "T,M,K",
    [(1, 256, 512), (16, 6144, 4096), (37, 512, 256), (128, 4096, 12288), (300, 1152, 4304), (1600, 4096, 4096),
     (5, 1000, 136), (2048, 768, 4096)],
)
def test_gemm_plain(cuda_device, T, M, K):
    x, w = rand_bf16(T, K, seed=1), rand_bf16(M, K, scale=K ** -0.5, seed=2)
    y = ops.linear(x.cuda(), w.cuda())
    ref = x.float() @ w.float().t()
    close(y, ref, 2e-2, 2e-2, f"gemm {T}x{M}x{K}")


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
def test_gemm_all_token_tiles(cuda_device, bn):
    T, M, K = 200, 384, 1024
    x, w = rand_bf16(T, K, seed=3), rand_bf16(M, K, scale=K ** -0.5, seed=4)
    y = ops.linear(x.cuda(), w.cuda(), bn=bn)
    close(y, x.float() @ w.float().t(), 2e-2, 2e-2, f"bn={bn}")


@pytest.mark.parametrize("stages", [1, 2, 3])
def test_gemm_short_pipelines(cuda_device, stages):
    T, M, K = 64, 256, 2048
    x, w = rand_bf16(T, K, seed=5), rand_bf16(M, K, scale=K ** -0.5, seed=6)
    y = ops.linear(x.cuda(), w.cuda(), stages=stages)
    close(y, x.float() @ w.float().t(), 2e-2, 2e-2, f"stages={stages}")


def test_gemm_epilogues(cuda_device):
    T, M, K = 70, 640, 1152
    x, w = rand_bf16(T, K, seed=7), rand_bf16(M, K, scale=K ** -0.5, seed=8)
    b, r = rand_bf16(M, seed=9), rand_bf16(T, M, seed=10)
    for act in (None, "gelu_tanh", "gelu"):
        y = ops.linear(x.cuda(), w.cuda(), bias=b.cuda(), act=act, residual=r.cuda())
        ref = ops.linear(x.float(), w.float(), bias=b.float(), act=act, residual=r.float())
        close(y, ref, 3e-2, 2e-2, f"epilogue {act}")


@pytest.mark.parametrize("T,M,K,splits", [(1, 4096, 4096, 4), (8, 512, 12288, 9), (16, 6144, 4096, 3), (130, 256, 512, 2),
                                          (130, 4096, 4096, 4), (256, 4096, 12288, 4), (400, 4096, 4096, 2), (511, 4096, 12288, 2),
                                          (228, 6144, 4096, 3)])
def test_gemm_split_k(cuda_device, T, M, K, splits):
    x, w = rand_bf16(T, K, seed=11), rand_bf16(M, K, scale=K ** -0.5, seed=12)
    parts = ops.linear_partial(x.cuda(), w.cuda(), splits, bn=16 if T <= 16 else 0)  # explicit tile: the tcgen05 kernel
    assert parts.shape[0] == ops.effective_splits(K, splits)
    close(parts.sum(0), x.float() @ w.float().t(), 1e-2, 1e-2, "split-k")


def test_short_prefill_row_parallel_splits_k_and_matches_dense(cuda_device):
    """129-511 tokens: the row-parallel projections return split-K partials whose sum, through the residual
    add + RMSNorm that consumes them, equals the dense projection path."""
    from prism_infer_b200.models.qwen3_vl import TPComm

    comm = TPComm()
    for T, M, K in ((228, 4096, 4096), (400, 4096, 12288), (511, 4096, 4096)):
        x, w = rand_bf16(T, K, seed=51).cuda(), rand_bf16(M, K, scale=K ** -0.5, seed=52).cuda()
        nw, res = bf(1 + 0.1 * torch.randn(M)).cuda(), rand_bf16(T, M, seed=53).cuda()
        dense, parts, ticket = comm.row_parallel(x, w)
        assert dense is None and ticket is None and parts.shape[0] == ops.choose_splits(M, K, T) > 1
        h, new_res = comm.add_rmsnorm(nw, 1e-6, dense, parts, ticket, res.clone())
        want_h, want_res = ops.add_rmsnorm(nw, 1e-6, x=ops.linear(x, w), residual=res.clone())
        close(new_res, want_res, 3e-2, 2e-2, f"residual T={T}")
        close(h, want_h, 6e-2, 3e-2, f"normed T={T}")


@pytest.mark.parametrize("T,I,K", [(1, 512, 256), (24, 12288, 4096), (700, 1536, 4096)])
def test_gemm_dual_swiglu(cuda_device, T, I, K):
    x, w = rand_bf16(T, K, seed=13), rand_bf16(2 * I, K, scale=K ** -0.5, seed=14)
    y = ops.gate_up_swiglu(x.cuda(), w.cuda())
    ref = ops.gate_up_swiglu(x.float(), w.float())
    close(y, ref, 2e-2, 3e-2, "dual swiglu")


def test_add_rmsnorm_variants(cuda_device):
    T, H = 9, 4096
    w = bf(1 + 0.1 * torch.randn(H))
    x, res = rand_bf16(T, H, seed=15), rand_bf16(T, H, seed=16)
    parts = torch.randn(3, T, H)
    extra, idx = rand_bf16(4, H, seed=17), torch.tensor([-1, 0, 1, -1, 2, 3, -1, -1, 0], dtype=torch.int32)
    for kw in (dict(x=x), dict(partials=parts)):
        for use_res in (False, True):
            for use_extra in (False, True):
                g = {k: v.cuda() for k, v in kw.items()}
                c = {k: v.float() for k, v in kw.items()}
                rg = res.clone().cuda() if use_res else None
                rc = res.float().clone() if use_res else None
                eg = dict(extra=extra.cuda(), extra_index=idx.cuda()) if use_extra else {}
                ec = dict(extra=extra.float(), extra_index=idx) if use_extra else {}
                ng, sg = ops.add_rmsnorm(w.cuda(), 1e-6, residual=rg, **g, **eg)
                nc, sc = ops.add_rmsnorm(w.float(), 1e-6, residual=rc, **c, **ec)
                close(sg, sc, 2e-2, 1e-2, "residual")
                close(ng, nc, 3e-2, 2e-2, "normed")


def test_layernorm_swiglu_embed(cuda_device):
    x = rand_bf16(33, 1152, seed=18)
    w, b = bf(1 + 0.1 * torch.randn(1152)), bf(0.1 * torch.randn(1152))
    close(ops.layernorm(x.cuda(), w.cuda(), b.cuda(), 1e-6), ops.layernorm(x.float(), w.float(), b.float(), 1e-6), 2e-2, 1e-2, "ln")
    gu = rand_bf16(7, 2 * 1536, seed=19)
    close(ops.swiglu(gu.cuda()), ops.swiglu(gu.float()), 1e-2, 1e-2, "swiglu")
    parts = torch.randn(2, 7, 2 * 1536)
    close(ops.swiglu(partials=parts.cuda()), ops.swiglu(partials=parts), 2e-2, 1e-2, "swiglu partials")
    table, vis = rand_bf16(100, 256, seed=20), rand_bf16(3, 256, seed=21)
    ids = torch.tensor([5, 99, 40, 41, 42, 7])
    vi = torch.tensor([-1, -1, 0, 1, 2, -1], dtype=torch.int32)
    yg = ops.embed(ids.cuda(), table[32:96].cuda(), visual=vis.cuda(), vis_index=vi.cuda(), vocab_start=32)
    yc = ops.embed(ids, table[32:96].float(), visual=vis.float(), vis_index=vi, vocab_start=32)
    close(yg, yc, 0, 0, "embed")


@pytest.mark.parametrize("mode", [ops.KV_BF16, ops.KV_FP8, ops.KV_FP8_SCALED])
@pytest.mark.parametrize("D,Hq,Hkv,section", [(128, 32, 8, (24, 20, 20)), (64, 4, 2, (8, 12, 12))])
def test_qk_norm_rope_store(cuda_device, mode, D, Hq, Hkv, section):
    T, page, blocks, L = 11, 16, 6, 2
    qkv = rand_bf16(T, (Hq + 2 * Hkv) * D, seed=22)
    qw, kw = bf(1 + 0.1 * torch.randn(D)), bf(1 + 0.1 * torch.randn(D))
    pos = torch.randint(0, 3000, (3, T), dtype=torch.int32)
    slots = torch.tensor([0, 1, 2, 17, -1, 40, 41, 95, 94, 3, 50], dtype=torch.int64)
    cg = ops.KVCache(L, blocks, Hkv, page, D, mode, "cuda")
    cc = ops.KVCache(L, blocks, Hkv, page, D, mode, "cpu", dtype=torch.float32)
    kwargs = dict(num_heads=Hq, num_kv_heads=Hkv, head_dim=D, theta=5e6, section=section, eps=1e-6, layer=1)
    for src in ("bf16", "partials"):
        if src == "bf16":
            qg = ops.qk_norm_rope_store(qkv=qkv.cuda(), partials=None, positions=pos.cuda(), q_weight=qw.cuda(),
                                        k_weight=kw.cuda(), slots=slots.cuda(), cache=cg, **kwargs)
        else:
            parts = torch.stack((qkv.float() * 0.25, qkv.float() * 0.75)).cuda()
            qg = ops.qk_norm_rope_store(qkv=None, partials=parts, positions=pos.cuda(), q_weight=qw.cuda(),
                                        k_weight=kw.cuda(), slots=slots.cuda(), cache=cg, **kwargs)
        qc = ops.qk_norm_rope_store(qkv=qkv.float(), partials=None, positions=pos, q_weight=qw.float(),
                                    k_weight=kw.float(), slots=slots, cache=cc, **kwargs)
        close(qg, qc, 4e-2, 2e-2, "q")
        tol = 4e-2 if mode == ops.KV_BF16 else 0.3
        for kv in (0, 1):
            close(cg.dequant(kv, 1), cc.dequant(kv, 1), tol, 0.07, f"cache kv={kv} mode={mode}")
        if mode == ops.KV_FP8_SCALED:
            close(cg.scales, cc.scales, 1e-4, 2e-2, "scales")
        assert float(cg.dequant(0, 0).abs().sum()) == 0.0  # other layer untouched


def test_scaled_fp8_store_matches_reference_quantiser(cuda_device):
    """Payload bit-equal and scales equal to the reference quantiser when fed bf16 k/v directly."""
    T, Hkv, D, page = 13, 8, 128, 16
    k, v = rand_bf16(T, Hkv, D, seed=23), rand_bf16(T, Hkv, D, scale=3.0, seed=24)
    slots = torch.arange(T, dtype=torch.int64) + 5
    cg = ops.KVCache(1, 4, Hkv, page, D, ops.KV_FP8_SCALED, "cuda")
    cg.payload.view(torch.uint8).fill_(0x7F)
    ops.store_kv(k.cuda(), v.cuda(), slots.cuda(), cg, 0)
    for kv, x in ((0, k), (1, v)):
        q, scale = ops.quantize_fp8_rows(x, True)
        blk, off = slots // page, slots % page
        got = cg.payload[kv, 0].cpu().view(torch.uint8)[blk, :, off]
        assert torch.equal(got, q.view(torch.uint8)), "payload bits differ"
        torch.testing.assert_close(cg.scales[kv, 0].cpu()[blk, :, off], scale, rtol=1e-6, atol=1e-7)
    # untouched slots keep their sentinel
    assert int(cg.payload[0, 0].cpu().view(torch.uint8)[0, 0, 0, 0]) == 0x7F


def _fill_cache(mode, L, blocks, Hkv, page, D, seed):
    cc = ops.KVCache(L, blocks, Hkv, page, D, mode, "cpu", dtype=torch.float32)
    g = torch.Generator().manual_seed(seed)
    raw = torch.randn(2, L, blocks, Hkv, page, D, generator=g)
    if mode == ops.KV_BF16:
        cc.payload.copy_(bf(raw).float())
    else:
        q, s = ops.quantize_fp8_rows(raw, mode == ops.KV_FP8_SCALED)
        cc.payload.copy_(q)
        if s is not None:
            cc.scales.copy_(s)
    cg = ops.KVCache(L, blocks, Hkv, page, D, mode, "cuda")
    cg.payload.copy_(cc.payload.to(cg.payload.dtype) if mode == ops.KV_BF16 else cc.payload)
    if cc.scales is not None:
        cg.scales.copy_(cc.scales)
    return cg, cc


@pytest.mark.parametrize("mode", [ops.KV_BF16, ops.KV_FP8, ops.KV_FP8_SCALED])
@pytest.mark.parametrize("D,Hq,Hkv,page", [(128, 32, 8, 256), (128, 4, 1, 256), (64, 4, 2, 16)])
@pytest.mark.parametrize("nsplit", [1, 4, 0])
@pytest.mark.parametrize("use_mma", [False, True])
def test_paged_decode(cuda_device, mode, D, Hq, Hkv, page, nsplit, use_mma):
    B, blocks = 5, 24
    cg, cc = _fill_cache(mode, 1, blocks, Hkv, page, D, seed=25)
    maxblk = 6
    ctx = torch.tensor([1, page + 3, 3 * page, 0, 2 * page - 1], dtype=torch.int32)
    bt = torch.full((B, maxblk), -1, dtype=torch.int32)
    perm = torch.randperm(blocks, generator=torch.Generator().manual_seed(26))
    c = 0
    for b in range(B):
        n = (int(ctx[b]) + page - 1) // page
        bt[b, :n] = perm[c:c + n].int()
        c += n
    q = rand_bf16(B, Hq, D, seed=27)
    yg = ops.paged_decode_attention(q.cuda(), cg, 0, bt.cuda(), ctx.cuda(), nsplit=nsplit, use_mma=use_mma)
    yc = ops.paged_decode_attention(q.float(), cc, 0, bt, ctx)
    err = (yg.float().cpu() - yc).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3, (err.max(), err.mean())


@pytest.mark.parametrize("use_mma", [False, True])
def test_paged_attention_skips_out_of_range_pages_and_reports(cuda_device, use_mma):
    """A context longer than the page table can describe and a page id beyond the cache are not
    read: the kernels cut the context, treat the page as a hole and set the status word."""
    D, Hq, Hkv, page, blocks, maxblk = 64, 4, 2, 16, 4, 3
    cg, cc = _fill_cache(ops.KV_FP8_SCALED, 1, blocks, Hkv, page, D, seed=41)
    q = rand_bf16(2, Hq, D, seed=42)
    bt = torch.tensor([[0, 1, 2], [3, 7, 1]], dtype=torch.int32)       # 7 >= blocks
    ctx = torch.tensor([100, 40], dtype=torch.int32)                   # 100 > maxblk * page
    yg = ops.paged_decode_attention(q.cuda(), cg, 0, bt.cuda(), ctx.cuda(), nsplit=2, use_mma=use_mma)
    torch.cuda.synchronize()
    st = native.read_status()["attn"]
    assert st[0] == 3 and st[3] >= 2, st
    bt_ok = torch.tensor([[0, 1, 2], [3, -1, 1]], dtype=torch.int32)
    yc = ops.paged_decode_attention(q.float(), cc, 0, bt_ok, torch.tensor([48, 40], dtype=torch.int32))
    err = (yg.float().cpu() - yc).abs()
    assert err.max() < 2e-2, err.max()
    # paged prefill: same guards (a skipped page contributes zero keys / values there, as any hole does)
    cu = torch.tensor([0, 3, 5], dtype=torch.int32)
    qp = rand_bf16(5, Hq, D, seed=43)
    kv = torch.tensor([35, 24], dtype=torch.int32)
    bt2 = torch.tensor([[0, 9, 2], [3, 1, -1]], dtype=torch.int32)     # 9 >= blocks
    yg = ops.paged_prefill_attention(qp.cuda(), cg, 0, cu.cuda(), kv.cuda(), bt2.cuda(), 3)
    torch.cuda.synchronize()
    st = native.read_status()["attn"]
    assert st[0] == 3, st
    bt2_hole = torch.tensor([[0, -1, 2], [3, 1, -1]], dtype=torch.int32)
    yh = ops.paged_prefill_attention(qp.cuda(), cg, 0, cu.cuda(), kv.cuda(), bt2_hole.cuda(), 3)
    torch.cuda.synchronize()
    assert native.read_status()["attn"][0] == 0
    assert torch.isfinite(yg.float()).all() and torch.equal(yg, yh)


@pytest.mark.parametrize("hd,Hq,Hkv", [(128, 8, 2), (64, 4, 2), (72, 16, 16), (32, 4, 4)])
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_attention(cuda_device, hd, Hq, Hkv, causal):
    lens = [5, 64, 130, 1, 257]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    packed = rand_bf16(T, (Hq + 2 * Hkv) * hd, seed=28)
    def views(t):
        return (t[:, : Hq * hd].view(T, Hq, hd), t[:, Hq * hd:(Hq + Hkv) * hd].view(T, Hkv, hd),
                t[:, (Hq + Hkv) * hd:].view(T, Hkv, hd))
    pg = packed.cuda()
    yg = ops.varlen_attention(*views(pg), cu.cuda(), max(lens), causal=causal)
    yc = ops.varlen_attention(*views(packed.float()), cu, max(lens), causal=causal)
    err = (yg.float().cpu() - yc).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3, (err.max(), err.mean())


@pytest.mark.parametrize("mode", [ops.KV_BF16, ops.KV_FP8_SCALED])
@pytest.mark.parametrize("D,Hq,Hkv,page", [(128, 8, 2, 256), (64, 4, 2, 16)])
def test_paged_prefill(cuda_device, mode, D, Hq, Hkv, page):
    blocks = 40
    cg, cc = _fill_cache(mode, 1, blocks, Hkv, page, D, seed=29)
    q_lens = [70, 1, 33]
    kv_lens = torch.tensor([70, page + 5, 2 * page + 33], dtype=torch.int32)
    cu = torch.tensor([0, 70, 71, 104], dtype=torch.int32)
    maxblk = 8
    bt = torch.full((3, maxblk), -1, dtype=torch.int32)
    perm = torch.randperm(blocks, generator=torch.Generator().manual_seed(30))
    c = 0
    for s in range(3):
        n = (int(kv_lens[s]) + page - 1) // page
        bt[s, :n] = perm[c:c + n].int()
        c += n
    q = rand_bf16(104, Hq, D, seed=31)
    yg = ops.paged_prefill_attention(q.cuda(), cg, 0, cu.cuda(), kv_lens.cuda(), bt.cuda(), max(q_lens))
    yc = ops.paged_prefill_attention(q.float(), cc, 0, cu, kv_lens, bt, max(q_lens))
    err = (yg.float().cpu() - yc).abs()
    assert err.max() < 3e-2 and err.mean() < 3e-3, (err.max(), err.mean())


def _cu(lens):
    out = torch.zeros(len(lens) + 1, dtype=torch.int32)
    out[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
    return out


@pytest.mark.parametrize("mode", [ops.KV_BF16, ops.KV_FP8, ops.KV_FP8_SCALED])
def test_paged_prefill_gathered_keys_on_the_tensor_cores(cuda_device, mode):
    """Head dimension 128 with key ranges given: the keys are gathered from their pages and the tcgen05 kernel
    runs over them.  Against the fp32 oracle, and against the page-reading kernel on the same inputs: a chunk with
    a long history (several key tiles, query rows past one 128-row tile), a single new token, a sequence without
    history and one whose history ends inside a page."""
    D, Hq, Hkv, page, blocks = 128, 8, 2, 256, 24
    cg, cc = _fill_cache(mode, 1, blocks, Hkv, page, D, seed=61)
    q_lens = [200, 1, 70, 130]
    kv = [3 * page + 200, page + 5, 70, 2 * page - 3]
    kv_lens = torch.tensor(kv, dtype=torch.int32)
    cu, cu_kv = _cu(q_lens), _cu(kv)
    maxblk = 6
    bt = torch.full((4, maxblk), -1, dtype=torch.int32)
    perm = torch.randperm(blocks, generator=torch.Generator().manual_seed(62))
    c = 0
    for s in range(4):
        n = (kv[s] + page - 1) // page
        bt[s, :n] = perm[c:c + n].int()
        c += n
    T = sum(q_lens)
    q = rand_bf16(T, Hq, D, seed=63)
    qg = q.cuda()
    args = (cg, 0, cu.cuda(), kv_lens.cuda(), bt.cuda(), max(q_lens))
    yt = ops.paged_prefill_attention(qg, *args, cu_seqlens_kv=cu_kv.cuda(), total_kv=sum(kv), max_kv_len=max(kv))
    ym = ops.paged_prefill_attention(qg, *args)
    torch.cuda.synchronize()
    assert native.read_status()["attn_tc"][0] == 0
    yc = ops.paged_prefill_attention(q.float(), cc, 0, cu, kv_lens, bt, max(q_lens))
    err = (yt.float().cpu() - yc).abs()
    assert err.max() < 3e-2 and err.mean() < 3e-3, (err.max(), err.mean())
    both = (yt.float() - ym.float()).abs()
    assert both.max() < 2e-2 and both.mean() < 1e-3, (both.max(), both.mean())


def test_paged_prefill_gather_skips_out_of_range_pages_and_reports(cuda_device):
    """A page id beyond the cache gives zero key rows (as a hole does) and sets the status word; nothing is read
    out of range."""
    D, Hq, Hkv, page, blocks = 128, 4, 1, 16, 6
    cg, _ = _fill_cache(ops.KV_FP8_SCALED, 1, blocks, Hkv, page, D, seed=64)
    q_lens, kv = [3, 2], [35, 24]
    cu, cu_kv = _cu(q_lens), _cu(kv)
    q = rand_bf16(5, Hq, D, seed=65).cuda()
    kvl = torch.tensor(kv, dtype=torch.int32).cuda()
    kw = dict(cu_seqlens_kv=cu_kv.cuda(), total_kv=sum(kv), max_kv_len=max(kv))
    bad = torch.tensor([[0, 9, 2], [3, 1, -1]], dtype=torch.int32)       # 9 >= blocks
    yb = ops.paged_prefill_attention(q, cg, 0, cu.cuda(), kvl, bad.cuda(), 3, **kw)
    torch.cuda.synchronize()
    st = native.read_status()["attn_tc"]
    assert st[0] == 3, st
    hole = torch.tensor([[0, -1, 2], [3, 1, -1]], dtype=torch.int32)
    yh = ops.paged_prefill_attention(q, cg, 0, cu.cuda(), kvl, hole.cuda(), 3, **kw)
    torch.cuda.synchronize()
    assert native.read_status()["attn_tc"][0] == 0
    assert torch.isfinite(yb.float()).all() and torch.equal(yb, yh)


def test_kv_copy_and_compaction(cuda_device):
    L, blocks, Hkv, page, D = 3, 10, 2, 16, 64
    cg, cc = _fill_cache(ops.KV_FP8_SCALED, L, blocks, Hkv, page, D, seed=32)
    ops.kv_page_copy(cg, cg, [0, 1], [5, 6], [16, 7])
    ops.kv_page_copy(cc, cc, [0, 1], [5, 6], [16, 7])
    src = torch.tensor([3, 17, 18, 40, 41, 47], dtype=torch.int64)
    dst = torch.tensor([0, 1, 2, 3, 16, 17], dtype=torch.int64)  # overlaps the sources
    ops.kv_compact(cg, src.cuda(), dst.cuda())
    ops.kv_compact(cc, src, dst)
    assert torch.equal(cg.payload.cpu().view(torch.uint8), cc.payload.view(torch.uint8))
    assert torch.equal(cg.scales.cpu(), cc.scales)
    # swap out to a pinned host pool and back
    host = ops.KVCache(L, 4, Hkv, page, D, ops.KV_FP8_SCALED, "cpu", pin_memory=True)
    ops.kv_page_copy(cg, host, [5, 2], [0, 3])
    torch.cuda.synchronize()
    assert torch.equal(host.payload[:, :, 0].view(torch.uint8), cc.payload[:, :, 5].view(torch.uint8))
    cg.payload.view(torch.uint8)[:, :, 9] = 0
    ops.kv_page_copy(host, cg, [3], [9])
    torch.cuda.synchronize()
    assert torch.equal(cg.payload[:, :, 9].cpu().view(torch.uint8), cc.payload[:, :, 2].view(torch.uint8))
    assert torch.equal(cg.scales[:, :, 9].cpu(), cc.scales[:, :, 2])


def test_sampler(cuda_device):
    B, V = 6, 151936
    logits = torch.randn(B, V)
    logits[2, 777] = logits[2, 90000] = 50.0  # tie -> lowest id
    tok = ops.sample(logits.cuda())
    assert tok.cpu().tolist() == logits.argmax(-1).tolist() and tok[2].item() == 777
    slabs = torch.stack((logits * 0.5, logits * 0.5)).cuda()
    val = torch.empty(B, device="cuda")
    tok2 = ops.sample(slabs, vocab_offset=1000, out_val=val)
    assert (tok2.cpu() - 1000).tolist() == logits.argmax(-1).tolist()
    close(val, logits.max(-1).values, 1e-5, 1e-5, "max value")
    # temperature sampling follows softmax(logits / T)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(4096, 1)
    temp = torch.full((4096,), 0.7)
    draws = ops.sample(small.cuda(), temp.cuda(), seed=1234)
    freq = torch.bincount(draws.cpu(), minlength=4).float() / 4096
    want = torch.softmax(small[0] / 0.7, -1)
    assert (freq - want).abs().max() < 0.03, (freq, want)
    mixed = ops.sample(small.cuda(), torch.zeros(4096).cuda())
    assert int(mixed.sum()) == 0


def test_vision_pointwise(cuda_device):
    from prism_infer_b200.models.position import vision_patch_coords, vision_pos_embed_plan
    grid = [(1, 6, 8), (2, 4, 4)]
    idx, wt = vision_pos_embed_plan(grid, 16, 2)
    N = idx.shape[1]
    x, table = rand_bf16(N, 128, seed=33), rand_bf16(256, 128, seed=34)
    yg = ops.pos_embed_add(x.clone().cuda(), table.cuda(), idx.cuda(), wt.cuda())
    yc = ops.pos_embed_add(x.float().clone(), table.float(), idx, wt)
    close(yg, yc, 3e-2, 1e-2, "pos embed")
    heads, hd = 4, 32
    qkv = rand_bf16(N, 3 * heads * hd, seed=35)
    coords = vision_patch_coords(grid, 2).int()
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2).float() / (hd // 2)))
    rg = ops.vit_rope(qkv.clone().cuda(), coords.cuda(), inv.cuda(), heads, hd)
    rc = ops.vit_rope(qkv.float().clone(), coords, inv, heads, hd)
    close(rg, rc, 3e-2, 1e-2, "vit rope")


@pytest.mark.parametrize("T,M,K", [(3000, 2000, 320), (6272, 1152, 1152), (777, 4304, 1152)])
def test_gemm_persistent_matches_tiled_kernel(cuda_device, T, M, K):
    """The persistent form (several tiles per CTA, two TMEM accumulators) gives the same bits as
    the one-tile-per-CTA kernel for every epilogue, and both match the fp32 reference."""
    x, w = rand_bf16(T, K, seed=21).cuda(), rand_bf16(M, K, scale=K ** -0.5, seed=22).cuda()
    b, r = rand_bf16(M, seed=23).cuda(), rand_bf16(T, M, seed=24).cuda()
    for kw in (dict(), dict(bias=b, act="gelu_tanh"), dict(bias=b, residual=r)):
        got = ops.linear(x, w, **kw)            # T >= 512: persistent kernel
        want = ops.linear(x, w, bn=256, **kw)   # explicit tile size: one tile per CTA
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"persistent vs tiled differ for {list(kw)}"
    close(got, ops.linear(x.float().cpu(), w.float().cpu(), bias=b.float().cpu(), residual=r.float().cpu()), 3e-2, 2e-2, "persistent")


def test_gemm_persistent_dual_swiglu(cuda_device):
    T, I, K = 2500, 1280, 512  # 10 x 20 tiles of 128 tokens: more tiles than SMs
    x, w = rand_bf16(T, K, seed=25).cuda(), rand_bf16(2 * I, K, scale=K ** -0.5, seed=26).cuda()
    got = ops.gate_up_swiglu(x, w)
    want = ops.gate_up_swiglu(x, w, bn=128)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    close(got, ops.gate_up_swiglu(x.float().cpu(), w.float().cpu()), 2e-2, 3e-2, "persistent dual")


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("lens,Hq,Hkv", [((300, 129, 64), 8, 2), ((1616,), 32, 8), ((1, 127, 128, 700), 4, 4)])
def test_tcgen05_flash_attention_matches_fp32_reference(cuda_device, causal, lens, Hq, Hkv, monkeypatch):
    """Head dimension 128, K/V read as strided views of a packed projection, ragged segments."""
    D = 128
    T = sum(lens)
    g = torch.Generator().manual_seed(len(lens) * 7 + Hq)
    qkv = (torch.randn(T, (Hq + 2 * Hkv) * D, generator=g) * 0.7).to(torch.bfloat16)
    heads = qkv.view(T, Hq + 2 * Hkv, D)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32)
    ref = ops.varlen_attention(heads[:, :Hq].float(), heads[:, Hq:Hq + Hkv].float(), heads[:, Hq + Hkv:].float(), cu, max(lens),
                               causal=causal)
    dev = heads.cuda()
    q = dev[:, :Hq].contiguous()
    monkeypatch.setattr(ops, "ATTN_TC_ENABLED", True)
    got = ops.varlen_attention(q, dev[:, Hq:Hq + Hkv], dev[:, Hq + Hkv:], cu.cuda(), max(lens), causal=causal)
    torch.cuda.synchronize()
    close(got, ref, 2e-2, 2e-2, f"tcgen05 attention causal={causal} lens={lens}")
    monkeypatch.setattr(ops, "ATTN_TC_ENABLED", False)
    legacy = ops.varlen_attention(q, dev[:, Hq:Hq + Hkv], dev[:, Hq + Hkv:], cu.cuda(), max(lens), causal=causal)
    close(got, legacy.float().cpu(), 2e-2, 2e-2, "tcgen05 vs mma.sync attention")


@pytest.mark.parametrize("lens", [(784, 784, 100), (196,), (130, 1, 257)])
def test_tcgen05_flash_attention_head_dim_72(cuda_device, lens, monkeypatch):
    """Vision-tower shape: 16 heads x 72 read as views of the packed QKV rows; the kernel pads the
    head to 80 columns with zeros supplied by the TMA unit."""
    H, D = 16, 72
    N = sum(lens)
    g = torch.Generator().manual_seed(N)
    qkv = (torch.randn(N, 3 * H * D, generator=g) * 0.8).to(torch.bfloat16)
    hv = qkv.view(N, 3, H, D)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32)
    ref = ops.varlen_attention(hv[:, 0].float(), hv[:, 1].float(), hv[:, 2].float(), cu, max(lens), causal=False)
    dev = hv.cuda()
    monkeypatch.setattr(ops, "ATTN_TC_ENABLED", True)
    got = ops.varlen_attention(dev[:, 0], dev[:, 1], dev[:, 2], cu.cuda(), max(lens), causal=False)
    torch.cuda.synchronize()
    close(got, ref, 2e-2, 2e-2, f"tcgen05 attention hd 72 lens={lens}")


@pytest.mark.parametrize("B,V,H", [(1, 151936, 4096), (4, 151936, 4096), (3, 5000, 256), (2, 1024, 8192)])
def test_fp8_candidate_lm_head_finds_the_exact_argmax(cuda_device, B, V, H):
    """Greedy token through the E4M3 candidate head + exact bf16 rerank equals the arg-max of the fp32 logits of the
    bf16 head; near ties (the two best logits closer than the rerank's summation-order noise) may pick either."""
    g = torch.Generator().manual_seed(B * 7 + H)
    w = (torch.randn(V, H, generator=g) * H ** -0.5).to(torch.bfloat16).cuda()
    x = (torch.randn(B, H, generator=g) * 3.0).to(torch.bfloat16).cuda()
    # plant clear and narrow winners: rows aligned with the activations
    for b in range(B):
        w[(1000 + 37 * b) % V] = (x[b].float() / x[b].float().norm() * (2.0 + b)).to(torch.bfloat16)
    codes, scale = ops.quantize_lm_head_fp8(w)
    deq = codes.view(torch.float8_e4m3fn).float() * scale[:, None]
    assert float((deq - w.float()).abs().max() / w.float().abs().max()) < 0.07
    got = ops.lm_head_fp8_greedy(x, codes, scale, w, vocab_offset=11)
    torch.cuda.synchronize()
    native.check_status()
    logits = x.float() @ w.float().t()
    want = logits.argmax(-1)
    top2 = logits.topk(2, dim=-1).values
    for b in range(B):
        if float(top2[b, 0] - top2[b, 1]) > 1e-3:
            assert int(got[b]) == int(want[b]) + 11, (b, int(got[b]), int(want[b]))
        else:
            assert float(logits[b, int(got[b]) - 11]) >= float(top2[b, 1]) - 1e-3
