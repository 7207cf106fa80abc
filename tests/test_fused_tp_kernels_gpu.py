"""Fused row-parallel GEMM -> exchange -> add+RMSNorm kernels.

On one GPU every rank's symmetric region is allocated on the same device and the ranks run
one after another in one stream (all pushes before any wait), which exercises the exact
kernels, pointer tables, slab indexing and sequence numbers without two kernels ever
waiting on each other.  The multi-GPU form (real peer memory over NVLink) runs when at
least two devices are visible.
"""

import pytest
import torch

from prism_infer_b200 import ops
from prism_infer_b200.ops import native

pytestmark = pytest.mark.gpu


def close(a, b, atol, rtol, what):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    assert bool((err <= lim).all()), f"{what}: max err {err.max().item():.4g}, worst ratio {(err / lim).max().item():.3g}"


@pytest.mark.parametrize("tp,T,K", [(2, 1, 2048), (4, 8, 1024), (2, 96, 512), (8, 24, 512), (8, 3, 1536)])
def test_push_gemm_then_wait_norm_emulated_ranks(cuda_device, tp, T, K):
    from prism_infer_b200.parallel import symm
    from prism_infer_b200.parallel.comm import FusedComm

    H = 4096
    ops.set_pdl(False)
    regions = symm.SymmetricRegion.create_emulated(tp, H)
    comms = [FusedComm(r, tp, H, region=regions[r]) for r in range(tp)]
    g = torch.Generator().manual_seed(tp * 100 + T)
    xs = [(torch.randn(T, K, generator=g)).to(torch.bfloat16).cuda() for _ in range(tp)]
    ws = [(torch.randn(H, K, generator=g) * (K * tp) ** -0.5).to(torch.bfloat16).cuda() for _ in range(tp)]
    weight = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    res0 = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    try:
        for step in range(3):  # several steps: sequence numbers grow, slots alternate
            for c in comms:
                c.begin_step()
            for point_pair in range(2):
                tickets = [c.row_parallel(xs[r], ws[r])[2] for r, c in enumerate(comms)]
                assert all(t is not None for t in tickets)
                want = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
                outs = []
                for r, c in enumerate(comms):
                    res = res0.clone()
                    normed, new_res = c.add_rmsnorm(weight, 1e-6, None, None, tickets[r], res)
                    outs.append((normed, new_res))
                torch.cuda.synchronize()
                ref_n, ref_r = ops.add_rmsnorm(weight.float().cpu(), 1e-6, x=want.cpu(), residual=res0.float().cpu().clone())
                for normed, new_res in outs:
                    assert (new_res.float().cpu() - ref_r).abs().max() < 5e-2
                    assert (normed.float().cpu() - ref_n).abs().max() < 8e-2
                # every rank computed bit-identical results (fixed summation order)
                for normed, new_res in outs[1:]:
                    assert torch.equal(normed, outs[0][0]) and torch.equal(new_res, outs[0][1])
        native.check_status()
    finally:
        for reg in regions:
            native.lib().prism_ipc_free(__import__("ctypes").c_void_p(reg.local_ptr))


def test_wait_that_never_completes_reports_status_and_returns(cuda_device):
    """Slabs nobody wrote: the bounded poll runs out, the status word says so, the context
    stays usable.  (The wait limit is about two seconds.)"""
    from prism_infer_b200.parallel import symm
    from prism_infer_b200.parallel.comm import FusedComm

    H = 4096
    ops.set_pdl(False)
    regions = symm.SymmetricRegion.create_emulated(2, H)
    c = FusedComm(0, 2, H, region=regions[0])
    c.begin_step()
    weight = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    res = torch.zeros(1, H, dtype=torch.bfloat16, device="cuda")
    native.read_status(reset=True)
    c.add_rmsnorm(weight, 1e-6, None, None, (0, 0, 2, 1), res)  # nobody pushed for point 0
    torch.cuda.synchronize()
    status = native.read_status(reset=True)
    assert status["norm"][0] == 2, status  # PRISM_ERR_PEER_TIMEOUT
    y = ops.rmsnorm(torch.ones(2, H, dtype=torch.bfloat16, device="cuda"), weight, 1e-6)  # context still works
    assert torch.isfinite(y.float()).all()
    for reg in regions:
        native.lib().prism_ipc_free(__import__("ctypes").c_void_p(reg.local_ptr))


def test_sharded_vision_tower_matches_single_rank(cuda_device):
    """Segment-sharded vision tower with the fused merger GEMM -> all-gather, ranks emulated
    on one device: every rank's pushes are issued before any rank waits."""
    import ctypes

    import numpy as np

    from prism_infer_b200.engine.vl_inputs import PatchProcessor
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.qwen3_vl import Qwen3VLModel
    from prism_infer_b200.models.weights import random_weights
    from prism_infer_b200.parallel import symm
    from prism_infer_b200.parallel.comm import FusedComm

    ops.set_pdl(False)
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    model = Qwen3VLModel(arch, device="cuda", dtype=torch.bfloat16)
    model.load(weights.items())
    proc = PatchProcessor(arch)
    rng = np.random.default_rng(0)
    parts = [proc.process_image(rng.integers(0, 256, (s, s, 3), dtype=np.uint8)) for s in (64, 96, 64)]
    vid = proc.process_video([rng.integers(0, 256, (64, 64, 3), dtype=np.uint8) for _ in range(6)])
    pixel_values = torch.cat([p for p, _ in parts] + [vid[0]]).cuda()
    grid = [g for _, g in parts] + [vid[1]]
    want_main, want_deep = model._vision_tower(pixel_values, grid, None, 0)
    total_tokens = want_main.shape[0]
    tp = 4
    H = arch.text.hidden_size
    regions = symm.SymmetricRegion.create_emulated(tp, H)
    comms = [FusedComm(r, tp, H, region=regions[r]) for r in range(tp)]
    model.tp = tp
    try:
        for call in range(3):  # alternate buffer sets across calls
            shards = model._vision_shards(grid)
            assert sum(rows for _, rows, _ in shards) == pixel_values.shape[0]
            for r, c in enumerate(comms):
                assert c.vision_begin(total_tokens)
                start, rows, sub = shards[r]
                if rows:
                    model._vision_tower(pixel_values[start:start + rows], sub, c, start // arch.vision.merge_unit)
            for c in comms:
                outs = c.vision_finish(1 + len(want_deep), total_tokens)
                assert torch.equal(outs[0], want_main)
                for got, want in zip(outs[1:], want_deep):
                    assert torch.equal(got, want)
        torch.cuda.synchronize()
        native.check_status()
    finally:
        model.tp = 1
        for reg in regions:
            native.lib().prism_ipc_free(ctypes.c_void_p(reg.local_ptr))


@pytest.mark.parametrize("tp,T,K", [(2, 700, 512), (4, 1616, 1024), (8, 1000, 512), (8, 520, 256)])
def test_prefill_scatter_gemm_then_reduce_norm_allgather_emulated_ranks(cuda_device, tp, T, K):
    """Row-parallel GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather for prefill-sized
    steps, ranks emulated one after another on one device (every rank's GEMM, then every rank's
    reduce, then the waits).  Two exchanges in a row: full residual first, sharded afterwards."""
    import ctypes

    from prism_infer_b200.parallel import symm
    from prism_infer_b200.parallel.comm import FusedComm

    H = 4096
    ops.set_pdl(False)
    regions = symm.SymmetricRegion.create_emulated(tp, H)
    comms = [FusedComm(r, tp, H, region=regions[r]) for r in range(tp)]
    g = torch.Generator().manual_seed(tp * 1000 + T)
    weight = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    extra = torch.randn(37, H, generator=g).to(torch.bfloat16).cuda()
    extra_index = torch.full((T,), -1, dtype=torch.int32)
    extra_index[5:42] = torch.arange(37, dtype=torch.int32)
    extra_index = extra_index.cuda()
    res_full = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    try:
        residual_ref = res_full.float().cpu()
        shards = [None] * tp
        for exchange in range(3):
            xs = [(torch.randn(T, K, generator=g)).to(torch.bfloat16).cuda() for _ in range(tp)]
            ws = [(torch.randn(H, K, generator=g) * (K * tp) ** -0.5).to(torch.bfloat16).cuda() for _ in range(tp)]
            tickets = [c.scatter_linear(xs[r], ws[r]) for r, c in enumerate(comms)]
            use_extra = exchange == 1
            outs = []
            for r, c in enumerate(comms):
                res = res_full if exchange == 0 else shards[r]
                h, shard = c.reduce_norm_allgather(tickets[r], weight, 1e-6, res, residual_is_shard=exchange > 0,
                                                   extra=extra if use_extra else None, extra_index=extra_index if use_extra else None,
                                                   wait=False)
                shards[r] = shard
                outs.append(h)
            for r, c in enumerate(comms):
                c.wait_allgather(tickets[r])
            torch.cuda.synchronize()
            native.check_status()
            # reference: bf16 partial per rank, summed in fp32, rounded, + residual (+ extra), RMSNorm
            partial = sum((x.float() @ w.float().t()).to(torch.bfloat16).float().cpu() for x, w in zip(xs, ws))
            delta = partial.to(torch.bfloat16).float()
            new_res = (residual_ref + delta).to(torch.bfloat16).float()
            if use_extra:
                idx = extra_index.cpu()
                sel = idx >= 0
                new_res[sel] = (new_res[sel] + extra.float().cpu()[idx[sel].long()]).to(torch.bfloat16).float()
            normed = (new_res * torch.rsqrt(new_res.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16).float() * weight.float().cpu()
            rpo = -(-T // tp)
            for r in range(tp):
                assert torch.equal(outs[r], outs[0]), "every rank holds the same gathered rows"
                rows = max(0, min(T, (r + 1) * rpo) - r * rpo)
                close(shards[r][:rows], new_res[r * rpo: r * rpo + rows], 6e-2, 2e-2, f"residual shard of rank {r}")
            close(outs[0], normed, 8e-2, 3e-2, f"gathered normalised rows, exchange {exchange}")
            residual_ref = torch.cat([shards[r][:max(0, min(T, (r + 1) * rpo) - r * rpo)].float().cpu() for r in range(tp)])
    finally:
        for reg in regions:
            native.lib().prism_ipc_free(ctypes.c_void_p(reg.local_ptr))


@pytest.mark.parametrize("tp,T,P", [(8, 32, 4), (8, 100, 3), (2, 128, 2), (4, 49, 1)])
def test_partial_rows_scatter_then_reduce_norm_allgather_emulated_ranks(cuda_device, tp, T, P):
    """The mid-size exchange (rows x ranks above 192, at most 128 rows): every rank's split-K partial
    rows are summed and sent as bf16 to the row's owner, which reduces over ranks, adds the residual,
    normalises and all-gathers.  Ranks emulated one after another on one device."""
    import ctypes

    from prism_infer_b200.parallel import symm
    from prism_infer_b200.parallel.comm import FusedComm

    H = 4096
    ops.set_pdl(False)
    regions = symm.SymmetricRegion.create_emulated(tp, H)
    comms = [FusedComm(r, tp, H, region=regions[r]) for r in range(tp)]
    g = torch.Generator().manual_seed(tp * 100 + T)
    weight = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    res_full = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    try:
        residual_ref = res_full.float().cpu()
        shards = [None] * tp
        for exchange in range(3):
            parts = [(torch.randn(P, T, H, generator=g) * 0.3).cuda() for _ in range(tp)]
            tickets = [c.scatter_partials(parts[r]) for r, c in enumerate(comms)]
            outs = []
            for r, c in enumerate(comms):
                res = res_full if exchange == 0 else shards[r]
                h, shard = c.reduce_norm_allgather(tickets[r], weight, 1e-6, res, residual_is_shard=exchange > 0, wait=False)
                shards[r] = shard
                outs.append(h)
            for r, c in enumerate(comms):
                c.wait_allgather(tickets[r])
            torch.cuda.synchronize()
            native.check_status()
            delta = sum(p.sum(0).to(torch.bfloat16).float().cpu() for p in parts).to(torch.bfloat16).float()
            new_res = (residual_ref + delta).to(torch.bfloat16).float()
            normed = (new_res * torch.rsqrt(new_res.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16).float() * weight.float().cpu()
            rpo = -(-T // tp)
            for r in range(tp):
                assert torch.equal(outs[r], outs[0]), "every rank holds the same gathered rows"
                rows = max(0, min(T, (r + 1) * rpo) - r * rpo)
                close(shards[r][:rows], new_res[r * rpo: r * rpo + rows], 6e-2, 2e-2, f"residual shard of rank {r}")
            close(outs[0], normed, 8e-2, 3e-2, f"gathered normalised rows, exchange {exchange}")
            residual_ref = torch.cat([shards[r][:max(0, min(T, (r + 1) * rpo) - r * rpo)].float().cpu() for r in range(tp)])
    finally:
        for reg in regions:
            native.lib().prism_ipc_free(ctypes.c_void_p(reg.local_ptr))
