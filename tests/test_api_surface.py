"""The exported C API exactly as a user of the reference calls it (names and argument order of its public header),
through ctypes on the host backend: every symbol and its ``p``-prefixed twin exists, the communicator queries answer,
and the register-then-submit entry points of all six collectives run with C callbacks."""
import ctypes as C
import threading

import numpy as np
import pytest

from helpers import run_ranks

NCCL = ["ncclGetVersion", "ncclGetUniqueId", "ncclCommInitRank", "ncclCommInitAll", "ncclCommDestroy", "ncclCommAbort",
        "ncclGetErrorString", "ncclCommGetAsyncError", "ncclCommCount", "ncclCommCuDevice", "ncclCommUserRank",
        "ncclRedOpCreatePreMulSum", "ncclRedOpDestroy", "ncclReduce", "ncclBcast", "ncclBroadcast", "ncclAllReduce",
        "ncclReduceScatter", "ncclAllGather", "ncclSend", "ncclRecv", "ncclGroupStart", "ncclGroupEnd"]
OFCCL = ["ofcclInitRankCtx", "ofcclFinalizeRankCtx7StartHostThrds", "ofcclPrepareDone", "ofcclDestroy",
         "ofcclPrepareReduce", "ofcclRunReduce", "ofcclPrepareBcast", "ofcclRunBcast", "ofcclPrepareBroadcast",
         "ofcclRunBroadcast", "ofcclPrepareAllReduce", "ofcclRunAllReduce", "ofcclPrepareReduceScatter",
         "ofcclRunReduceScatter", "ofcclPrepareAllGather", "ofcclRunAllGather"]


def test_every_symbol_of_the_reference_header_is_exported_with_its_profiling_twin(native):
    L = native.lib()
    for name in NCCL + OFCCL:
        assert hasattr(L, name), name
        assert hasattr(L, "p" + name), "p" + name


def test_communicator_queries_and_error_strings(host_backend):
    nv = host_backend
    L = nv.lib()
    v = C.c_int()
    assert L.ncclGetVersion(C.byref(v)) == nv.SUCCESS and v.value >= 21200        # the fork point of the reference: 2.12
    comms = nv.Comm.init_loopback(3)
    for r, c in enumerate(comms):
        n, u, d, e = C.c_int(-1), C.c_int(-1), C.c_int(-7), C.c_int(-1)
        assert L.ncclCommCount(c.handle, C.byref(n)) == nv.SUCCESS and n.value == 3
        assert L.ncclCommUserRank(c.handle, C.byref(u)) == nv.SUCCESS and u.value == r
        assert L.ncclCommCuDevice(c.handle, C.byref(d)) == nv.SUCCESS
        assert L.ncclCommGetAsyncError(c.handle, C.byref(e)) == nv.SUCCESS and e.value == nv.SUCCESS
        assert L.pncclCommCount(c.handle, C.byref(n)) == nv.SUCCESS and n.value == 3
    assert L.ncclCommCount(None, C.byref(v)) != nv.SUCCESS
    texts = {nv.error_string(code) for code in range(0, 8)}
    assert len(texts) >= 6 and all(texts)                                          # distinct, non-empty descriptions
    for c in comms:
        c.destroy()


def test_register_then_submit_with_the_reference_names(host_backend):
    """ofcclPrepare* / ofcclRun* for Reduce, Bcast (in place), Broadcast, AllReduce, ReduceScatter and AllGather, each
    rank submitting in its own order, completions delivered through C callbacks with their argument pointers."""
    nv = host_backend
    L = nv.lib()
    world, n = 3, 3001
    vp, sz, i = C.c_void_p, C.c_size_t, C.c_int
    CB = C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p)
    L.ofcclInitRankCtx.argtypes = [C.POINTER(vp), i]
    L.ofcclPrepareReduce.argtypes = [sz, i, i, i, vp, i, vp]
    L.ofcclPrepareBcast.argtypes = [sz, i, i, vp, i, vp]
    L.ofcclPrepareBroadcast.argtypes = [sz, i, i, vp, i, vp]
    L.ofcclPrepareAllReduce.argtypes = [sz, i, i, vp, i, vp]
    L.ofcclPrepareReduceScatter.argtypes = [sz, i, i, vp, i, vp]
    L.ofcclPrepareAllGather.argtypes = [sz, i, vp, i, vp]
    for name in ("ofcclRunReduce", "ofcclRunBroadcast", "ofcclRunAllReduce", "ofcclRunReduceScatter", "ofcclRunAllGather"):
        getattr(L, name).argtypes = [vp, vp, i, CB, vp, vp]
    L.ofcclRunBcast.argtypes = [vp, i, CB, vp, vp]
    L.ofcclFinalizeRankCtx7StartHostThrds.argtypes = [vp]
    L.ofcclDestroy.argtypes = [vp]
    comms = nv.Comm.init_loopback(world)
    results = {}

    def body(r):
        comm = comms[r].handle
        ctx = vp()
        nv.check(L.ofcclInitRankCtx(C.byref(ctx), r))
        nv.check(L.ofcclPrepareReduce(n, nv.FLOAT32, nv.SUM, 1, comm, 0, ctx))
        nv.check(L.ofcclPrepareBcast(n, nv.FLOAT32, 2, comm, 1, ctx))
        nv.check(L.ofcclPrepareBroadcast(n, nv.FLOAT32, 0, comm, 2, ctx))
        nv.check(L.ofcclPrepareAllReduce(n, nv.FLOAT32, nv.MAX, comm, 3, ctx))
        nv.check(L.ofcclPrepareReduceScatter(n, nv.FLOAT32, nv.SUM, comm, 4, ctx))
        nv.check(L.ofcclPrepareAllGather(n, nv.FLOAT32, comm, 5, ctx))
        nv.check(L.ofcclFinalizeRankCtx7StartHostThrds(ctx))
        done, seen = threading.Event(), []
        tokens = (C.c_int * 6)(*range(100, 106))

        @CB
        def on_done(coll_id, args):
            seen.append((coll_id, C.cast(args, C.POINTER(C.c_int))[0]))
            if len(seen) == 6:
                done.set()
            return 0
        mk = lambda k, val: np.full(k, val, np.float32)
        send = {0: mk(n, r + 1), 2: mk(n, 10 * (r + 1)), 3: mk(n, float((r * 7) % 5)), 4: np.arange(world * n, dtype=np.float32) + r, 5: mk(n, r + 1)}
        recv = {0: mk(n, 0), 2: mk(n, 0), 3: mk(n, 0), 4: mk(n, 0), 5: mk(world * n, 0)}
        inplace = mk(n, 100 + r)
        runs = {0: L.ofcclRunReduce, 2: L.ofcclRunBroadcast, 3: L.ofcclRunAllReduce, 4: L.ofcclRunReduceScatter, 5: L.ofcclRunAllGather}
        order = [(k + r) % 6 for k in range(6)]                                    # a different order on every rank
        for cid in order:
            arg = C.cast(C.byref(tokens, 4 * cid), vp)
            if cid == 1:
                nv.check(L.ofcclRunBcast(inplace.ctypes.data, 1, on_done, arg, ctx))
            else:
                nv.check(runs[cid](send[cid].ctypes.data, recv[cid].ctypes.data, cid, on_done, arg, ctx))
        assert done.wait(60), seen
        assert sorted(seen) == [(c, 100 + c) for c in range(6)]
        results[r] = (recv, inplace)
        nv.check(L.ofcclDestroy(ctx))

    run_ranks(world, body, timeout=180)
    for c in comms:
        c.destroy()
    for r in range(world):
        recv, inplace = results[r]
        if r == 1:
            assert np.all(recv[0] == 6.0)                                           # Reduce to root 1: 1 + 2 + 3
        assert np.all(inplace == 102.0)                                             # Bcast from root 2, in place
        assert np.all(recv[2] == 10.0)                                              # Broadcast from root 0
        assert np.all(recv[3] == max((q * 7) % 5 for q in range(world)))            # AllReduce max
        np.testing.assert_array_equal(recv[4], sum(np.arange(world * n, dtype=np.float32)[r * n:(r + 1) * n] + q for q in range(world)))
        np.testing.assert_array_equal(recv[5], np.repeat(np.arange(1, world + 1, dtype=np.float32), n))
