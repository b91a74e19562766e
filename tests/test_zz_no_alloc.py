"""The allocation-free entry point (``dfcclAllReduceNoAlloc``, csrc/include/dfccl_noalloc.h).

It serves callers that must not allocate device memory - a process whose GPU memory is
already fully reserved by its framework or capped by a quota, a latency-critical loop that
cannot take the device-wide synchronisation of cudaMalloc / cudaFree - by keeping all
scratch of the one-rank all-reduce in a static device array of the library.

The test calls it through its exported C symbol and compares with the regular entry point
(``ncclAllReduce`` on a one-rank communicator with a pre-multiplied-sum operator, which
stages the same buffers through allocated scratch), twice in a row with different data:
the second call finds the array exactly as the first one left it.  That nothing is allocated
is checked on the device's own count of free bytes (``cudaMemGetInfo``), which sees every
allocation in the process, around each call after a first one that has loaded the kernel.
This file sorts last
on purpose, so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nv():
    from dfccl_b200 import native
    native.lib()
    native.set_backend("cuda")
    return native


def _regular(nv, comm, x, scale, dt):
    """out = scale * x through the allocating path."""
    L = nv.lib()
    op = C.c_int()
    s = C.c_float(scale)
    nv.check(L.ncclRedOpCreatePreMulSum(C.byref(op), C.byref(s), nv.FLOAT32, 1, comm.handle))
    # the operator's scalar is given in fp32; the library folds it into the registration
    out = torch.empty_like(x)
    st = torch.cuda.current_stream().cuda_stream
    nv.check(L.ncclAllReduce(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), x.numel(), dt, op.value, comm.handle,
                             C.c_void_p(st)))
    torch.cuda.synchronize()
    nv.check(L.ncclRedOpDestroy(op.value, comm.handle))
    return out


@pytest.mark.parametrize("dt_name,tdt", [("FLOAT32", torch.float32), ("BFLOAT16", torch.bfloat16)])
def test_no_alloc_matches_regular_entry_point_twice(nv, dt_name, tdt):
    torch.cuda.set_device(0)
    L = nv.lib()
    dt = getattr(nv, dt_name)
    (comm,) = nv.Comm.init_loopback(1, 0)
    L.dfcclNoAllocStatus.argtypes = [C.POINTER(C.c_uint32)]
    g = torch.Generator(device="cpu").manual_seed(7)
    side = torch.cuda.Stream()                                   # a non-blocking stream: not ordered after the default one
    try:
        # first call on this device: set-up and kernel load (the only call allowed to change the free-byte count)
        w = torch.ones(64, dtype=tdt, device="cuda")
        assert L.dfcclAllReduceNoAlloc(C.c_void_p(w.data_ptr()), C.c_void_p(w.data_ptr()), 64, dt, C.c_float(1.0),
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)) == nv.SUCCESS
        torch.cuda.synchronize()
        for (n, scale), stream in zip(((1_000_003, 0.125), (4099, 3.0), (65_537, -1.5)),
                                      (torch.cuda.current_stream(), torch.cuda.current_stream(), side)):
            # calls in a row, different size and data; the last one on the non-blocking stream
            x = (torch.rand(n, generator=g) * 2 - 1).to(tdt).cuda()
            want = _regular(nv, comm, x, scale, dt)
            got = torch.empty_like(x)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc = L.dfcclAllReduceNoAlloc(C.c_void_p(x.data_ptr()), C.c_void_p(got.data_ptr()), n, dt, C.c_float(scale),
                                         C.c_void_p(stream.cuda_stream))
            assert rc == nv.SUCCESS
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before, "the entry point changed the device's free memory"
            status = C.c_uint32(99)
            assert L.dfcclNoAllocStatus(C.byref(status)) == nv.SUCCESS and status.value == 0
            tol = 1e-6 if tdt == torch.float32 else 1e-2
            torch.testing.assert_close(got.float(), want.float(), rtol=tol, atol=tol)
            torch.testing.assert_close(got.float(), x.float() * scale, rtol=tol, atol=tol)
        # in place, and the size limit
        y = torch.ones(1024, dtype=tdt, device="cuda")
        assert L.dfcclAllReduceNoAlloc(C.c_void_p(y.data_ptr()), C.c_void_p(y.data_ptr()), 1024, dt, C.c_float(2.0),
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)) == nv.SUCCESS
        torch.cuda.synchronize()
        assert bool((y == 2).all())
        too_many = (8 << 20) // y.element_size() + 1
        assert L.dfcclAllReduceNoAlloc(C.c_void_p(y.data_ptr()), C.c_void_p(y.data_ptr()), too_many, dt, C.c_float(1.0),
                                       None) == nv.INVALID_ARGUMENT
        assert L.dfcclAllReduceNoAlloc(None, C.c_void_p(y.data_ptr()), 8, dt, C.c_float(1.0), None) == nv.INVALID_ARGUMENT
    finally:
        comm.destroy()
