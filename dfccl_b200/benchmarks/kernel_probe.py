"""Single-GPU probe of the library's own kernels for profiling: the stream-ordered collective
kernel on a one-rank communicator (reduce / scale / cast data path over heap buffers, nothing to
wait for) and the fused optimizer kernel.  Sized above the L2 capacity, a few launches, so that a
profiler capture ends by itself.

    python -m dfccl_b200.benchmarks.kernel_probe --mbytes 256 --iters 3
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from dfccl_b200 import native as nv
from dfccl_b200.utils import tensor_from_ptr


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbytes", type=int, default=256)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    torch.cuda.set_device(0)
    nv.set_backend("cuda")
    L = nv.lib()
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
    print(json.dumps(out))
    comm.destroy()


if __name__ == "__main__":
    main()
