"""Throughput of the hand-written tcgen05 GEMM kernels next to cuBLAS (one GPU).

    python -m dfccl_b200.benchmarks.gemm_bench                       # table over the sizes below
    python -m dfccl_b200.benchmarks.gemm_bench --once 8192 --kernel pair   # a few launches of one kernel (for a profiler)

Timing: CUDA events on the launching stream after warm-up; operands of every size but the smallest exceed the L2, and
a buffer larger than the L2 is rewritten between timed launches (``--flush 1``, default) so that no launch finds its
operands cached by the previous one.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

import torch

from .. import native as nv
from ..ops import gemm

SIZES = [(2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (16384, 4096, 1024), (8192, 4096, 4096), (4096, 3072, 1024),
         (8192, 1024, 4096)]


def _time(fn, iters: int, flush: torch.Tensor | None) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--flush", type=int, default=1)
    ap.add_argument("--once", type=int, default=0, help="run three launches of an N^3 product and exit")
    ap.add_argument("--kernel", default="pair", choices=["pair", "one"])
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    if a.once:
        os.environ["DFCCL_GEMM_PAIR"] = "1" if a.kernel == "pair" else "0"
        n = a.once
        x = torch.randn(n, n, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, n, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            gemm.matmul_nt(x, w, out)
        torch.cuda.synchronize()
        assert gemm.check_kernels()
        print("ok")
        return
    pairs = C.c_int()
    nv.check(nv.lib().dfcclGemmPairResident(C.byref(pairs)))
    flush = torch.zeros(160 << 20, device="cuda", dtype=torch.uint8) if a.flush else None
    rows = []
    for m, n, k in SIZES:
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * m * n * k
        os.environ["DFCCL_GEMM_PAIR"] = "1"
        t_pair = _time(lambda: gemm.matmul_nt(x, w, out), a.iters, flush)
        os.environ["DFCCL_GEMM_PAIR"] = "0"
        t_one = _time(lambda: gemm.matmul_nt(x, w, out), a.iters, flush)
        del os.environ["DFCCL_GEMM_PAIR"]
        t_lib = _time(lambda: torch.matmul(x, w.t(), out=out), a.iters, flush)
        rows.append({"m": m, "n": n, "k": k, "cta_pair_tflops": round(flops / t_pair / 1e9, 1), "one_cta_tflops": round(flops / t_one / 1e9, 1),
                     "cublas_tflops": round(flops / t_lib / 1e9, 1), "cta_pair_us": round(t_pair * 1e3, 1), "cublas_us": round(t_lib * 1e3, 1)})
        print(json.dumps(rows[-1]), flush=True)
    assert gemm.check_kernels()
    res = {"resident_cta_pairs": pairs.value, "l2_flushed_between_launches": bool(a.flush), "rows": rows}
    if a.out:
        with open(a.out, "w") as f:
            json.dump(res, f, indent=1)
    print(json.dumps({"resident_cta_pairs": pairs.value}))


if __name__ == "__main__":
    main()
