"""Runtime behaviour on the host backend: arbitrary per-rank issue orders,
preemption, voluntary quit / relaunch, bounded waits, abort, host-side fault
injection, statistics, tracing, the stream-ordered nccl* interface, send / recv,
communicator split.  No test here needs (or touches) a GPU."""
import ctypes as C
import json
import os
import random
import threading
import time

import numpy as np
import pytest

from helpers import host_array, run_ranks


def _env(**kv):
    class _E:
        def __enter__(self):
            self.old = {k: os.environ.get(k) for k in kv}
            os.environ.update({k: str(v) for k, v in kv.items()})

        def __exit__(self, *a):
            for k, v in self.old.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
    return _E()


def test_disordered_issue_completes_and_preempts(host_backend):
    """Every rank submits the same set of collectives in its own random order, several
    iterations in a row: everything completes, results are right, and the daemons had
    to park collectives to get there."""
    nv = host_backend
    nranks, ncolls, iters = 4, 16, 6
    rng = random.Random(7)
    kinds = [rng.choice([nv.ALLREDUCE, nv.ALLGATHER, nv.REDUCESCATTER, nv.BROADCAST]) for _ in range(ncolls)]
    counts = [rng.choice([64, 1000, 4096, 33333]) for _ in range(ncolls)]
    comms = nv.Comm.init_loopback(nranks)
    stats = {}

    def body(r):
        c = comms[r]
        ctx = nv.RankCtx(r)
        bufs = []
        for i in range(ncolls):
            ctx.prepare(i, c, kinds[i], counts[i], nv.FLOAT32, root=i % nranks)
            sn = counts[i] * (nranks if kinds[i] == nv.REDUCESCATTER else 1)
            rn = counts[i] * (nranks if kinds[i] == nv.ALLGATHER else 1)
            sp, rp = c.alloc(sn * 4), c.alloc(rn * 4)
            bufs.append((sp, rp, host_array(sp, sn, np.float32), host_array(rp, rn, np.float32)))
        ctx.finalize()
        order_rng = random.Random(100 + r)
        for it in range(iters):
            order = list(range(ncolls))
            order_rng.shuffle(order)
            for i in order:
                bufs[i][2][:] = (r + 1) * (i + 1) + it
                ctx.run(i, bufs[i][0], bufs[i][1])
                if order_rng.random() < 0.3:
                    time.sleep(0.0005)
            assert ctx.wait_all(60000) == nv.SUCCESS
            for i in range(ncolls):
                out = bufs[i][3]
                vals = [(q + 1) * (i + 1) + it for q in range(nranks)]
                if kinds[i] in (nv.ALLREDUCE, nv.REDUCESCATTER):
                    assert np.all(out == sum(vals)), (i, out[:3], sum(vals))
                elif kinds[i] == nv.ALLGATHER:
                    assert np.all(out.reshape(nranks, -1) == np.array(vals, np.float32)[:, None])
                else:
                    assert np.all(out == vals[i % nranks])
        time.sleep(0.05)                           # device counters are folded in when the daemon parks
        stats[r] = ctx.stats()
        ctx.destroy()

    with _env(DFCCL_BASE_CTX_SWITCH_THRESHOLD=20, DFCCL_IDLE_QUIT_US=300):
        run_ranks(nranks, body, timeout=240)
    for c in comms:
        c.destroy()
    total = {k: sum(s[k] for s in stats.values()) for k in stats[0]}
    assert total["sqesSubmitted"] == total["cqesDelivered"] == nranks * ncolls * iters
    assert total["ctxSwitches"] > 0 and total["ctxLoads"] >= total["ctxSwitches"]
    assert total["waitTimeouts"] == 0


def test_voluntary_quit_and_relaunch(host_backend):
    nv = host_backend
    comms = nv.Comm.init_loopback(2)
    seen = {}

    def body(r):
        ctx = nv.RankCtx(r)
        ctx.prepare(0, comms[r], nv.ALLREDUCE, 256, nv.FLOAT32)
        ctx.finalize()
        p = comms[r].alloc(1024)
        v = host_array(p, 256, np.float32)
        for it in range(4):
            v[:] = 1.0
            ctx.run(0, p, p)
            assert ctx.wait(0, 20000) == nv.SUCCESS
            assert np.all(v == 2.0)
            time.sleep(0.05)             # far longer than the idle limit: the daemon leaves in between
        time.sleep(0.05)
        seen[r] = ctx.stats()
        ctx.destroy()

    with _env(DFCCL_IDLE_QUIT_US=100):
        run_ranks(2, body)
    for c in comms:
        c.destroy()
    assert seen[0]["daemonLaunches"] >= 4 and seen[0]["daemonVoluntaryQuits"] >= 3


def test_bounded_wait_reports_timeout_instead_of_hanging(host_backend):
    """Rank 1 never submits: rank 0's collective ends with a timeout status, the
    context stays usable for the error query, nothing hangs."""
    nv = host_backend
    comms = nv.Comm.init_loopback(2)
    out = {}
    gate = threading.Event()

    def body(r):
        ctx = nv.RankCtx(r)
        ctx.prepare(0, comms[r], nv.ALLREDUCE, 64, nv.FLOAT32)
        ctx.finalize()
        p = comms[r].alloc(256)
        if r == 0:
            fired = []
            t0 = time.time()
            ctx.run(0, p, p, lambda cid: fired.append(cid))
            out["rc"] = ctx.wait(0, 20000)
            out["dt"] = time.time() - t0
            out["fired"] = fired
            out["async"] = ctx.async_error()
            time.sleep(0.05)                       # device counters are folded in when the daemon parks
            out["stats"] = ctx.stats()
            gate.set()
        else:
            gate.wait(30)
        ctx.destroy()

    with _env(DFCCL_WAIT_TIMEOUT_MS=400):
        run_ranks(2, body)
    for c in comms:
        c.destroy()
    assert out["rc"] == nv.TIMEOUT and out["async"] == nv.TIMEOUT
    assert out["fired"] == [0]                     # the callback still runs exactly once
    assert 0.3 < out["dt"] < 10
    assert out["stats"]["waitTimeouts"] >= 1


def test_dropped_submission_times_out_on_the_peer(host_backend):
    nv = host_backend
    comms = nv.Comm.init_loopback(2)
    rcs = {}

    def body(r):
        ctx = nv.RankCtx(r)
        ctx.prepare(0, comms[r], nv.ALLGATHER, 32, nv.INT32)
        ctx.finalize()
        s, d = comms[r].alloc(128), comms[r].alloc(256)
        if r == 1:
            ctx.inject_fault(nv.FAULT_DROP_SQE, 1)      # accepted by the host side, never reaches the daemon
        ctx.run(0, s, d)
        rcs[r] = ctx.wait(0, 1500 if r == 1 else 20000)
        if r == 1:
            ctx.abort()                                  # its own submission can never complete
        ctx.destroy()

    with _env(DFCCL_WAIT_TIMEOUT_MS=300):
        run_ranks(2, body)
    for c in comms:
        c.destroy()
    assert rcs[0] == nv.TIMEOUT
    assert rcs[1] in (nv.TIMEOUT, nv.ABORTED)


def test_abort_releases_waiters(host_backend):
    nv = host_backend
    comms = nv.Comm.init_loopback(2)
    res = {}

    def body(r):
        ctx = nv.RankCtx(r)
        ctx.prepare(0, comms[r], nv.ALLREDUCE, 64, nv.FLOAT32)
        ctx.finalize()
        p = comms[r].alloc(256)
        if r == 0:
            ctx.run(0, p, p)
            threading.Timer(0.2, ctx.abort).start()
            res["rc"] = ctx.wait(0, 20000)
        ctx.destroy()

    run_ranks(2, body)
    for c in comms:
        c.destroy()
    assert res["rc"] == nv.ABORTED


def test_delayed_submissions_and_slow_poller_still_complete(host_backend):
    nv = host_backend
    comms = nv.Comm.init_loopback(3)

    def body(r):
        ctx = nv.RankCtx(r)
        for i in range(4):
            ctx.prepare(i, comms[r], nv.ALLREDUCE, 128, nv.FLOAT32)
        ctx.finalize()
        if r == 1:
            ctx.inject_fault(nv.FAULT_DELAY_SQE_US, 3000)
        if r == 2:
            ctx.inject_fault(nv.FAULT_FREEZE_POLLER, 5)
        ps = [comms[r].alloc(512) for _ in range(4)]
        for it in range(3):
            for i in (range(4) if r % 2 == 0 else reversed(range(4))):
                host_array(ps[i], 128, np.float32)[:] = 1
                ctx.run(i, ps[i], ps[i])
            assert ctx.wait_all(30000) == nv.SUCCESS
            assert all(np.all(host_array(p, 128, np.float32) == 3) for p in ps)
        ctx.destroy()

    run_ranks(3, body)
    for c in comms:
        c.destroy()


def test_usage_errors(host_backend):
    nv = host_backend
    (c,) = nv.Comm.init_loopback(1)
    ctx = nv.RankCtx(0)
    with pytest.raises(nv.DfcclError):
        ctx.prepare(5000, c, nv.ALLREDUCE, 8, nv.FLOAT32)           # id out of range
    with pytest.raises(nv.DfcclError):
        ctx.prepare(0, c, nv.ALLREDUCE, 8, nv.FLOAT32, root=3)      # bad root
    with pytest.raises(nv.DfcclError):
        ctx.prepare(0, c, nv.ALLGATHER, 8, nv.FLOAT32, out_dtype=nv.BFLOAT16)   # copies cannot cast
    with pytest.raises(nv.DfcclError):
        ctx.prepare(0, c, nv.ALLREDUCE, 8, nv.INT32, out_dtype=nv.FLOAT32)      # no such kernel
    ctx.prepare(0, c, nv.ALLREDUCE, 8, nv.FLOAT32)
    with pytest.raises(nv.DfcclError):
        ctx.prepare(0, c, nv.ALLREDUCE, 8, nv.FLOAT32)              # registered twice
    p = c.alloc(64)
    with pytest.raises(nv.DfcclError):
        ctx.run(0, p, p)                                            # not finalized
    ctx.finalize()
    with pytest.raises(nv.DfcclError):
        ctx.prepare(1, c, nv.ALLREDUCE, 8, nv.FLOAT32)              # after finalize
    with pytest.raises(nv.DfcclError):
        ctx.run(3, p, p)                                            # never prepared
    with pytest.raises(nv.DfcclError):
        ctx.run(0, 0, p)                                            # null buffer
    ctx.run(0, p, p)
    assert ctx.wait(0, 10000) == nv.SUCCESS
    ctx.destroy()
    c.free(p)
    c.destroy()


def test_queue_flow_control_with_many_outstanding_submissions(host_backend):
    """More registered collectives than a small queue would hold at once: submissions
    block only while the ring is full and all complete."""
    nv = host_backend
    n = 300
    (c,) = nv.Comm.init_loopback(1)
    ctx = nv.RankCtx(0)
    for i in range(n):
        ctx.prepare(i, c, nv.ALLREDUCE, 16, nv.FLOAT32, scale=2.0)
    ctx.finalize()
    p = c.alloc(64 * n)
    v = host_array(p, 16 * n, np.float32)
    for it in range(3):
        v[:] = 1.0
        for i in range(n):
            ctx.run(i, p + 64 * i, p + 64 * i)
        assert ctx.wait_all(30000) == nv.SUCCESS
        assert np.all(v == 2.0)
    st = ctx.stats()
    assert st["sqesSubmitted"] == 3 * n == st["cqesDelivered"]
    ctx.destroy()
    c.destroy()


def test_trace_dump_is_chrome_trace_json(host_backend, tmp_path):
    nv = host_backend
    with _env(DFCCL_TRACE=1):
        (c,) = nv.Comm.init_loopback(1)
        ctx = nv.RankCtx(0)
        ctx.prepare(0, c, nv.ALLREDUCE, 1024, nv.FLOAT32)
        ctx.finalize()
    p = c.alloc(4096)
    ctx.run(0, p, p)
    assert ctx.wait(0, 10000) == nv.SUCCESS
    time.sleep(0.05)
    out = tmp_path / "trace.json"
    ctx.trace_dump(str(out))
    ev = json.loads(out.read_text())["traceEvents"]
    names = {e["name"] for e in ev}
    assert {"sqe", "data", "done"} <= names
    assert ctx.stats()["deviceEvents"] >= 4
    ctx.destroy()
    c.destroy()


# ---------------------------------------------------------------- stream-ordered interface

def test_nccl_style_collectives_on_the_host_backend(host_backend):
    nv = host_backend
    L = nv.lib()
    n = 4
    comms = nv.Comm.init_all(n)
    assert [c.rank for c in comms] == list(range(n)) and all(c.nranks == n for c in comms)

    def body(r):
        c = comms[r]
        x = np.full(1000, r + 1.0, np.float32)
        y = np.zeros(1000, np.float32)
        vp = C.c_void_p
        nv.check(L.ncclAllReduce(vp(x.ctypes.data), vp(y.ctypes.data), 1000, nv.FLOAT32, nv.SUM, c.handle, None))
        assert np.all(y == 10)
        nv.check(L.ncclAllReduce(vp(x.ctypes.data), vp(x.ctypes.data), 1000, nv.FLOAT32, nv.AVG, c.handle, None))
        assert np.allclose(x, 2.5)
        g = np.zeros(4 * 10, np.int32)
        mine = np.full(10, r, np.int32)
        nv.check(L.ncclAllGather(vp(mine.ctypes.data), vp(g.ctypes.data), 10, nv.INT32, c.handle, None))
        assert np.all(g.reshape(4, 10) == np.arange(4)[:, None])
        rs = np.zeros(10, np.int32)
        nv.check(L.ncclReduceScatter(vp(g.ctypes.data), vp(rs.ctypes.data), 10, nv.INT32, nv.SUM, c.handle, None))
        assert np.all(rs == 4 * r)
        b = np.full(33, r, np.int64)
        nv.check(L.ncclBcast(vp(b.ctypes.data), 33, nv.INT64, 2, c.handle, None))
        assert np.all(b == 2)
        red = np.zeros(7, np.float64)
        src = np.full(7, float(r), np.float64)
        nv.check(L.ncclReduce(vp(src.ctypes.data), vp(red.ctypes.data), 7, nv.FLOAT64, nv.MAX, 1, c.handle, None))
        if r == 1:
            assert np.all(red == 3)
        # user-defined pre-multiplied sum
        op = C.c_int()
        scalar = C.c_float(0.5)
        nv.check(L.ncclRedOpCreatePreMulSum(C.byref(op), C.byref(scalar), nv.FLOAT32, 1, c.handle))
        ones = np.ones(16, np.float32)
        nv.check(L.ncclAllReduce(vp(ones.ctypes.data), vp(ones.ctypes.data), 16, nv.FLOAT32, op.value, c.handle, None))
        assert np.allclose(ones, 2.0)
        nv.check(L.ncclRedOpDestroy(op.value, c.handle))
        assert L.ncclRedOpDestroy(op.value, c.handle) == nv.INVALID_ARGUMENT
        assert c.async_error() == nv.SUCCESS

    run_ranks(n, body)
    for c in comms:
        c.destroy()


def test_send_recv_and_groups(host_backend):
    nv = host_backend
    L = nv.lib()
    n = 4
    comms = nv.Comm.init_all(n)

    def body(r):
        c = comms[r]
        vp = C.c_void_p
        nxt, prv = (r + 1) % n, (r - 1) % n
        out = np.full(5000, r, np.int32)
        inp = np.zeros(5000, np.int32)
        # ring exchange: everybody sends and receives in one group
        nv.check(L.ncclGroupStart())
        nv.check(L.ncclSend(vp(out.ctypes.data), 5000, nv.INT32, nxt, c.handle, None))
        nv.check(L.ncclRecv(vp(inp.ctypes.data), 5000, nv.INT32, prv, c.handle, None))
        nv.check(L.ncclGroupEnd())
        assert np.all(inp == prv)
        # all-to-all built from grouped send / recv, receiving into heap memory
        heap = c.alloc(4 * 8 * n)
        hv = host_array(heap, 8 * n, np.int32)
        src = np.repeat(np.arange(n, dtype=np.int32) + 10 * r, 8)
        nv.check(L.ncclGroupStart())
        for p in range(n):
            if p == r:
                hv[8 * p:8 * p + 8] = src[8 * p:8 * p + 8]
                continue
            nv.check(L.ncclSend(vp(src.ctypes.data + 32 * p), 8, nv.INT32, p, c.handle, None))
            nv.check(L.ncclRecv(vp(heap + 32 * p), 8, nv.INT32, p, c.handle, None))
        nv.check(L.ncclGroupEnd())
        assert np.all(hv.reshape(n, 8) == (r + 10 * np.arange(n))[:, None])
        # plain blocking pair outside a group
        if r == 0:
            nv.check(L.ncclSend(vp(out.ctypes.data), 10, nv.INT32, 1, c.handle, None))
        elif r == 1:
            nv.check(L.ncclRecv(vp(inp.ctypes.data), 10, nv.INT32, 0, c.handle, None))
            assert np.all(inp[:10] == 0)
        assert L.ncclSend(vp(out.ctypes.data), 1, nv.INT32, 99, c.handle, None) == nv.INVALID_ARGUMENT

    run_ranks(n, body)
    for c in comms:
        c.destroy()
    assert nv.lib().ncclGroupEnd() == nv.INVALID_USAGE


def test_comm_split_builds_tp_and_dp_groups(host_backend):
    """2 x 2 layout: colour by row gives tensor-parallel pairs, by column data-parallel pairs;
    collectives registered on the sub-communicators run through the same daemon."""
    nv = host_backend
    comms = nv.Comm.init_loopback(4)

    def body(r):
        world = comms[r]
        tp = world.split(r // 2, r)
        dp = world.split(r % 2, r)
        assert tp.nranks == 2 and dp.nranks == 2 and tp.rank == r % 2 and dp.rank == r // 2
        ctx = nv.RankCtx(r)
        ctx.prepare(0, world, nv.ALLREDUCE, 100, nv.FLOAT32)
        ctx.prepare(10 + r // 2, tp, nv.ALLREDUCE, 100, nv.FLOAT32)
        ctx.prepare(20 + r % 2, dp, nv.ALLGATHER, 50, nv.FLOAT32)
        ctx.finalize()
        a, b, d = world.alloc(400), world.alloc(400), world.alloc(400)
        for p in (a, b):
            host_array(p, 100, np.float32)[:] = r + 1
        ids = [0, 10 + r // 2, 20 + r % 2]
        order = ids if r % 2 == 0 else ids[::-1]
        for i in order:
            ctx.run(i, {0: a, 10 + r // 2: b, 20 + r % 2: a}[i], {0: a, 10 + r // 2: b, 20 + r % 2: d}[i]) if i != 0 else ctx.run(0, a, a)
            if i == 0:
                assert ctx.wait(0, 20000) == nv.SUCCESS   # world sum must land before a is gathered or vice versa
        assert ctx.wait_all(20000) == nv.SUCCESS
        assert np.all(host_array(b, 100, np.float32) == (3 if r < 2 else 7))
        ctx.destroy()
        tp.destroy()
        dp.destroy()

    run_ranks(4, body)
    for c in comms:
        c.destroy()


def test_stream_ordered_submissions_may_run_ahead(host_backend):
    """A stream-ordered caller re-submits an id without waiting for the previous completion
    (the device timeline orders them): nothing is dropped, nothing is reordered."""
    nv = host_backend
    comms = nv.Comm.init_loopback(2)

    def body(r):
        ctx = nv.RankCtx(r)
        ctx.prepare(0, comms[r], nv.ALLREDUCE, 512, nv.FLOAT32)
        ctx.prepare(1, comms[r], nv.ALLREDUCE, 512, nv.FLOAT32)
        ctx.finalize()
        p, q = comms[r].alloc(2048), comms[r].alloc(2048)
        host_array(p, 512, np.float32)[:] = 1.0
        host_array(q, 512, np.float32)[:] = 1.0
        for it in range(40):
            for cid, buf in ((0, p), (1, q)) if (it + r) % 2 else ((1, q), (0, p)):
                ctx.run_on_stream(cid, buf, buf, 0)          # in place: every round doubles the values
        assert ctx.wait_all(60000) == nv.SUCCESS
        assert ctx.stats()["cqesDelivered"] == 80
        ctx.destroy()

    run_ranks(2, body)
    for c in comms:
        c.destroy()


def test_staged_buffers_with_several_blocks(host_backend):
    """Unregistered buffers and more than one block per collective: the staging copies must use
    the same partition as the data movement (block b's flags order only block b's bytes)."""
    nv = host_backend
    import test_host_collectives as T
    with _env(DFCCL_DAEMON_BLOCKS=3, DFCCL_MIN_BYTES_PER_BLOCK=1024):
        for kind in T.KINDS:
            T._run_case(nv, kind, 4, 30011, nv.FLOAT32, heap=False, root=1, iters=2)


def test_functional_collectives_on_torch_tensors(host_backend):
    """The torch-tensor layer over the stream-ordered entry points (host backend: CPU tensors)."""
    import torch
    from helpers import run_ranks
    from dfccl_b200.ops import collectives as coll
    nv = host_backend
    world = 3
    comms = nv.Comm.init_loopback(world)
    res = {}

    def body(r):
        c = comms[r]
        x = torch.full((6, 4), float(r + 1))
        out = {"ar": coll.all_reduce(c, x.clone()), "avg": coll.all_reduce(c, x.clone(), op="avg"),
               "ag": coll.all_gather(c, x[:2].contiguous()), "rs": coll.reduce_scatter(c, x.clone()),
               "bc": coll.broadcast(c, x.clone(), root=2), "rd": coll.reduce(c, x.clone(), root=1, op="max")}
        res[r] = out

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    for r in range(world):
        assert torch.all(res[r]["ar"] == 6) and torch.all(res[r]["avg"] == 2) and torch.all(res[r]["bc"] == 3)
        assert res[r]["ag"].shape == (6, 4) and torch.equal(res[r]["ag"][:, 0], torch.tensor([1., 1, 2, 2, 3, 3]))
        assert res[r]["rs"].shape == (2, 4) and torch.all(res[r]["rs"] == 6)
    assert torch.all(res[1]["rd"] == 3) and res[0]["rd"] is None
