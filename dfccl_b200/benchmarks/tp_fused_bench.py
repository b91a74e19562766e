"""Fused tensor-parallel GEMMs vs the unfused library path (NCCL collective + cuBLAS GEMM).

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m dfccl_b200.benchmarks.tp_fused_bench --out tp.json

Shapes are the four linear layers of GPT-2 medium (d = 1024) under 2-way tensor parallelism with
sequence-parallel activations.  Times are CUDA-event device times, max over ranks.  The roofline of
a fused kernel is the slower of its FLOPs at the measured bf16 GEMM peak and the bytes it must move
over NVLink at the measured peer-copy bandwidth.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from dfccl_b200.ops.fused_linear import AllGatherGemm, GemmReduceScatter, TpGroup
from dfccl_b200.ops import gemm
from dfccl_b200.parallel import init_distributed


def timeit(fn, iters, world):
    """Device time per call.  A 2 ms kernel is queued first so that the host is well ahead of the GPU
    when the timed calls start: what is measured is the kernels, not Python's enqueue rate."""
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(4_000_000)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192, help="rows of the full activation (micro-batch x sequence)")
    ap.add_argument("--d-model", dest="d", type=int, default=1024, help="model width (the launcher module of torch treats a bare --d as an abbreviation of its own options)")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--peak-tflops", type=float, default=1658.4)
    ap.add_argument("--link-gbs", type=float, default=655.0)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    d = init_distributed()
    n, rank, dev = d.world, d.rank, d.device
    tp = TpGroup(d.comm, dist.group.WORLD if n > 1 else None, dev)
    M, D = a.tokens, a.d
    rows = M // n
    rowsOut = []
    # column-parallel layers: all-gather -> GEMM
    for name, n_out in (("qkv", 3 * D // n), ("mlp_up", 4 * D // n)):
        xs = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        w = torch.randn(n_out, D, device=dev, dtype=torch.bfloat16)
        op = AllGatherGemm(tp, rows, D, n_out)
        y = torch.empty(M, n_out, device=dev, dtype=torch.bfloat16)
        full = torch.empty(M, D, device=dev, dtype=torch.bfloat16)
        fused = timeit(lambda: op(xs, w, y), a.iters, n)

        def unfused():
            dist.all_gather_into_tensor(full, xs)
            torch.matmul(full, w.t(), out=y)
        base = timeit(unfused, a.iters, n)
        only = timeit(lambda: gemm.matmul_nt(full, w, y), a.iters, n)
        flops = 2.0 * M * n_out * D
        wire = (n - 1) * rows * D * 2
        roof = max(flops / (a.peak_tflops * 1e6), wire / (a.link_gbs * 1e3))
        rowsOut.append({"layer": name, "kind": "allgather->gemm", "M": M, "N": n_out, "K": D, "fused_us": fused, "nccl_plus_cublas_us": base,
                        "own_gemm_only_us": only, "roofline_us": roof, "fraction_of_roofline": roof / fused, "speedup_vs_unfused": base / fused})
    # row-parallel layers: GEMM -> reduce-scatter
    for name, k_full in (("attn_out", D), ("mlp_down", 4 * D)):
        kl = k_full // n
        x = torch.randn(M, kl, device=dev, dtype=torch.bfloat16)
        w = torch.randn(D, kl, device=dev, dtype=torch.bfloat16)
        op = GemmReduceScatter(tp, M, kl, D)
        ys = torch.empty(rows, D, device=dev, dtype=torch.bfloat16)
        part = torch.empty(M, D, device=dev, dtype=torch.bfloat16)
        fused = timeit(lambda: op(x, w, ys), a.iters, n)

        def unfused():
            torch.matmul(x, w.t(), out=part)
            dist.reduce_scatter_tensor(ys, part)
        base = timeit(unfused, a.iters, n)
        flops = 2.0 * M * D * kl
        wire = (n - 1) * rows * D * 2
        roof = max(flops / (a.peak_tflops * 1e6), wire / (a.link_gbs * 1e3))
        rowsOut.append({"layer": name, "kind": "gemm->reducescatter", "M": M, "N": D, "K": kl, "fused_us": fused, "nccl_plus_cublas_us": base,
                        "roofline_us": roof, "fraction_of_roofline": roof / fused, "speedup_vs_unfused": base / fused})
    ok = gemm.check_kernels()
    if rank == 0:
        for r in rowsOut:
            print(json.dumps(r), flush=True)
        print(json.dumps({"kernels_ok": ok, "world": n}))
        if a.out:
            json.dump({"world": n, "rows": rowsOut, "peak_tflops": a.peak_tflops, "link_gbs": a.link_gbs}, open(a.out, "w"), indent=1)
    d.destroy()


if __name__ == "__main__":
    main()
