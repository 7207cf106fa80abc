"""Fused tensor-parallel kernels against their roofline and against the NCCL baseline.

Launch with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/bench_fused_tp.py [--iters 200]

Cases (Qwen3-VL-8B shapes, tensor-parallel over N ranks):

* ``o_proj`` / ``down_proj`` row-parallel GEMM -> one-shot exchange -> residual add + RMSNorm
  (``prism_gemm_wx_push`` + ``prism_add_rmsnorm_packed``) for T in {1, 8, 32, 128} tokens,
  versus split-K GEMM + ``dist.all_reduce`` + add+RMSNorm.
* the prefill-sized form of the same exchange for 1616 and 4096 tokens: GEMM -> reduce-scatter
  (``prism_gemm_wx_scatter``) + reduce / residual / RMSNorm -> all-gather
  (``prism_reduce_norm_allgather``), versus GEMM + ``dist.all_reduce`` + add+RMSNorm.
* vision merger GEMM -> all-gather (``prism_gemm_wx_allgather``) for 196 and 1568 tokens,
  versus GEMM + ``dist.all_gather``.

Each number is device time (CUDA events around ``iters`` back-to-back iterations, max over
ranks); the GEMM -> exchange cases are captured into a CUDA graph first, like a decode step.  Roofline per iteration = max(local weight + activation bytes / measured HBM
bandwidth, bytes that must cross NVLink per rank / 770 GB/s, FLOPs / measured bf16 peak).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200 import ops  # noqa: E402
from prism_infer_b200.parallel.comm import FusedComm, NcclComm  # noqa: E402

NVLINK_GBS = 770.0


def timed(fn, iters: int, graph: bool = False) -> float:
    """Device time per call.  With ``graph`` the call is captured once into a CUDA graph and
    replayed, as the decode step does, so host launch cost does not hide the kernels."""
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fn()
            side.synchronize()
            dist.barrier()
            with torch.cuda.graph(g, stream=side):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        run = g.replay
        for _ in range(3):
            run()
    else:
        run = fn
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        run()
    e.record()
    torch.cuda.synchronize()
    ms = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peaks = json.load(open(peaks_path)) if os.path.exists(peaks_path) else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    H, I = 4096, 12288
    fused = FusedComm(rank, world, H)
    nccl = NcclComm(rank, world)
    ops.set_pdl(True)
    g = torch.Generator(device="cuda").manual_seed(rank)
    weight = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    rows = []
    for name, K in (("o_proj", H // world), ("down_proj", I // world)):
        w = (torch.randn(H, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        for T in (1, 8, 32, 128):
            x = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
            res = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")

            def run_fused():
                fused.begin_step()
                for _ in range(2):  # two exchange points per step, alternating slots
                    d, p, ticket = fused.row_parallel(x, w)  # falls back to the NCCL arm when tokens * tp is large
                    fused.add_rmsnorm(weight, 1e-6, d, p, ticket, res)

            def run_nccl():
                for _ in range(2):
                    d, p, t = nccl.row_parallel(x, w)
                    nccl.add_rmsnorm(weight, 1e-6, d, p, t, res)

            t_f = timed(run_fused, args.iters, graph=True) / 2
            t_n = timed(run_nccl, args.iters, graph=True) / 2
            local_bytes = H * K * 2 + T * K * 2
            link_bytes = T * H * 4 * (world - 1)  # fp32 partial rows pushed to every peer
            flops = 2.0 * T * H * K
            roof_ms = max(local_bytes / peaks["hbm_gbs"] / 1e6, link_bytes / NVLINK_GBS / 1e6, flops / peaks["bf16_tflops"] / 1e9)
            rows.append({"kernel": f"{name} GEMM->exchange->add+RMSNorm", "tp": world, "tokens": T, "fused_us": round(t_f * 1e3, 2),
                         "nccl_us": round(t_n * 1e3, 2), "roofline_us": round(roof_ms * 1e3, 3),
                         "frac_of_roofline": round(roof_ms / t_f, 4), "speedup_vs_nccl": round(t_n / t_f, 2)})
    # prefill-sized exchange: row-parallel GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather
    for name, K in (("o_proj", H // world), ("down_proj", I // world)):
        w = (torch.randn(H, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        for T in (1616, 4096):
            x = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
            res_full = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
            state = {"shard": None}

            def run_fused_prefill():
                ticket = fused.scatter_linear(x, w)
                res = res_full if state["shard"] is None else state["shard"]
                _, state["shard"] = fused.reduce_norm_allgather(ticket, weight, 1e-6, res, residual_is_shard=state["shard"] is not None)

            def run_nccl_prefill():
                d, p, t = nccl.row_parallel(x, w)
                nccl.add_rmsnorm(weight, 1e-6, d, p, t, res_full)

            t_f = timed(run_fused_prefill, max(20, args.iters // 4))
            t_n = timed(run_nccl_prefill, max(20, args.iters // 4))
            own_rows = -(-T // world)
            link_bytes = (world - 1) * own_rows * H * 2 * 2  # partial rows out to their owners, normalised rows out to every peer
            flops = 2.0 * T * H * K
            local_bytes = H * K * 2 + T * K * 2 + T * H * 2
            roof_ms = max(local_bytes / peaks["hbm_gbs"] / 1e6, link_bytes / NVLINK_GBS / 1e6, flops / peaks["bf16_tflops"] / 1e9)
            rows_out = {"kernel": f"{name} GEMM->reduce-scatter->add+RMSNorm->all-gather", "tp": world, "tokens": T,
                        "fused_us": round(t_f * 1e3, 2), "nccl_us": round(t_n * 1e3, 2), "roofline_us": round(roof_ms * 1e3, 3),
                        "frac_of_roofline": round(roof_ms / t_f, 4), "speedup_vs_nccl": round(t_n / t_f, 2)}
            if rank == 0:
                print(json.dumps(rows_out), flush=True)
    # vision merger fc2 GEMM -> all-gather
    md = 4608
    w2 = (torch.randn(H, md, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b2 = torch.zeros(H, dtype=torch.bfloat16, device="cuda")
    for total in (196, 1568):
        per = -(-total // world)
        t0 = min(total, rank * per)
        n = max(0, min(total, t0 + per) - t0)
        h = torch.randn(max(n, 1), md, generator=g, device="cuda").to(torch.bfloat16)

        def run_fused_vis():
            assert fused.vision_begin(total)
            if n:
                fused.allgather_linear(h[:n], w2, b2, 0, t0)
            fused.vision_finish(1, total)

        def run_nccl_vis():
            y = ops.linear(h[:n], w2, bias=b2) if n else torch.empty((0, H), dtype=torch.bfloat16, device="cuda")
            pad = torch.zeros((per, H), dtype=torch.bfloat16, device="cuda")
            pad[:n] = y
            parts = [torch.empty_like(pad) for _ in range(world)]
            dist.all_gather(parts, pad)

        t_f = timed(run_fused_vis, max(20, args.iters // 4))
        t_n = timed(run_nccl_vis, max(20, args.iters // 4))
        local_bytes = H * md * 2 + n * md * 2
        link_bytes = n * H * 2 * (world - 1)
        flops = 2.0 * n * H * md
        roof_ms = max(local_bytes / peaks["hbm_gbs"] / 1e6, link_bytes / NVLINK_GBS / 1e6, flops / peaks["bf16_tflops"] / 1e9)
        rows.append({"kernel": "merger fc2 GEMM->all-gather", "tp": world, "tokens": total, "fused_us": round(t_f * 1e3, 2),
                     "nccl_us": round(t_n * 1e3, 2), "roofline_us": round(roof_ms * 1e3, 3),
                     "frac_of_roofline": round(roof_ms / t_f, 4), "speedup_vs_nccl": round(t_n / t_f, 2)})
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
    torch.cuda.synchronize()
    from prism_infer_b200.ops import native

    status = native.read_status()
    bad = {k: v for k, v in status.items() if v[0]}
    if bad:
        print(f"rank {rank} device status: {bad}", flush=True)
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
