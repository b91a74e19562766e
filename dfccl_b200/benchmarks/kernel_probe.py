"""Single-GPU probe of the library's own kernels for profiling: the stream-ordered collective
kernel on a one-rank communicator (reduce / scale / cast data path over heap buffers, nothing to
wait for) and the fused optimizer kernel.  Sized above the L2 capacity, a few launches, so that a
profiler capture ends by itself.

    python -m dfccl_b200.benchmarks.kernel_probe --mbytes 256 --iters 3
    python -m dfccl_b200.benchmarks.kernel_probe --gemm 8192 8192 8192 --iters 20     # tcgen05 GEMM vs cuBLAS
    python -m dfccl_b200.benchmarks.kernel_probe --stream-ops --iters 200             # stream <-> resident kernel round trip
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from dfccl_b200 import native as nv
from dfccl_b200.utils import tensor_from_ptr


def gemm_probe(mnk, iters):
    """C[M,N] = A[M,K] B[N,K]^T in bf16: this library's tcgen05 kernel and cuBLAS (through torch.matmul).  Between
    timed launches a 256 MB buffer is rewritten so that no launch finds its operands in L2."""
    from dfccl_b200.ops.gemm import matmul_nt
    m, n, k = mnk
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    c = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    out = {"M": m, "N": n, "K": k}
    for name, fn in (("tcgen05", lambda: matmul_nt(a, b, c)), ("cublas", lambda: torch.matmul(a, b.t(), out=c))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(iters):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        us = tot * 1e3 / iters
        out[name] = {"us": us, "tflops": 2.0 * m * n * k / us / 1e6}
    ref = a.float() @ b.float().t()
    matmul_nt(a, b, c)
    out["max_rel_err"] = float((c.float() - ref).abs().max() / ref.abs().max())
    print(json.dumps(out))


def stream_ops_probe(iters):
    """Round trip stream -> resident kernel -> stream in its eight forms (see dfcclProbeStreamRoundTrip)."""
    L = nv.lib()
    names = {0: "memop_write+memop_wait", 1: "kernel_write+memop_wait", 2: "memop_write+kernel_wait", 3: "kernel_write+kernel_wait"}
    ns = (C.c_uint64 * 13)()
    if L.dfcclProbeMemoryOps(200, ns) == nv.SUCCESS:
        names_ops = ("ld_host", "st_host", "st_host+fence_sys", "st_dev+fence_sys", "st_dev+fence_gpu", "fence_sys", "atomic_dev", "ld_dev",
                     "st_dev+fence_acq_rel_sys", "st_dev+fence_acq_rel_gpu", "ld_dev_dependent", "st_release_sys", "timer_read")
        print(json.dumps({"control_path_op_ns": dict(zip(names_ops, [int(v) for v in ns]))}))
    for delay in (0, 10, 50):
        out = {}
        for mode in range(8):
            us = C.c_double(0)
            rc = L.dfcclProbeStreamRoundTrip(mode, iters, delay, C.byref(us))      # first call warms the kernels up
            rc = L.dfcclProbeStreamRoundTrip(mode, iters, delay, C.byref(us))
            out[names[mode & 3] + ("+host_mirror" if mode & 4 else "")] = round(us.value - delay, 2) if rc == nv.SUCCESS else f"error {rc}"
        print(json.dumps({"answer_delay_us": delay, "stream_round_trip_minus_delay_us": out}))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbytes", type=int, default=256)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--gemm", type=int, nargs=3, metavar=("M", "N", "K"), help="time the plain tcgen05 GEMM of this size instead")
    ap.add_argument("--stream-ops", action="store_true", help="time the stream <-> resident kernel round trip instead")
    a = ap.parse_args(argv)
    torch.cuda.set_device(0)
    nv.set_backend("cuda")
    L = nv.lib()
    if a.stream_ops:
        return stream_ops_probe(a.iters)
    if a.gemm:
        return gemm_probe(a.gemm, a.iters)
    (comm,) = nv.Comm.init_loopback(1, 0)
    n = a.mbytes * (1 << 20) // 2                    # bf16 elements
    p, q = comm.alloc(2 * n), comm.alloc(2 * n)
    x = tensor_from_ptr(p, (n,), torch.bfloat16, "cuda:0")
    x.normal_()
    st = torch.cuda.current_stream().cuda_stream
    out = {}
    for name, fn in (
        ("collective_kernel_1rank_bf16", lambda: nv.check(L.ncclAllReduce(p, q, n, nv.BFLOAT16, nv.AVG, comm.handle, st))),
    ):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / a.iters
        out[name] = {"us": us, "gbs_read_plus_write": 2 * 2 * n / us / 1e3}
    m = n // 2
    master = torch.randn(m, device="cuda")
    grad = torch.randn(m, device="cuda")
    mom = torch.zeros(m, device="cuda")
    par = torch.empty(m, dtype=torch.bfloat16, device="cuda")

    def sgd():
        nv.check(L.dfcclFusedSgdStep(master.data_ptr(), grad.data_ptr(), mom.data_ptr(), par.data_ptr(), m, nv.BFLOAT16,
                                     0.1, 0.9, 1e-4, 0, st))
    for _ in range(3):
        sgd()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        sgd()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    out["fused_sgd"] = {"us": us, "gbs": (3 * 4 + 2 * 4 + 2) * m / us / 1e3}
    mom2 = torch.zeros(m, device="cuda")

    def adamw(step=[0]):
        step[0] += 1
        nv.check(L.dfcclFusedAdamWStep(master.data_ptr(), grad.data_ptr(), mom.data_ptr(), mom2.data_ptr(), par.data_ptr(), m,
                                       nv.BFLOAT16, 1e-3, 0.9, 0.999, 1e-8, 0.01, step[0], st))
    for _ in range(3):
        adamw()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        adamw()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    out["fused_adamw"] = {"us": us, "gbs": (4 * 4 + 3 * 4 + 2) * m / us / 1e3}     # reads master, grad, m, v; writes master, m, v (fp32) + bf16 param
    print(json.dumps(out))
    comm.destroy()


if __name__ == "__main__":
    main()
