"""Scheduler features of the daemon on the host backend: the sliced, resumable data phase, the adaptive wait
budget, deferred submissions released by a separate (capturable) trigger, grouped send / recv with both ends in
one thread.  No GPU is needed or touched."""
import ctypes as C
import os
import random

import numpy as np
import pytest

from helpers import host_array, run_ranks
from test_host_runtime import _env


@pytest.mark.parametrize("nranks", [2, 3])
def test_sliced_data_phase_resumes_at_its_cursor(host_backend, nranks):
    """Tiny slices force every collective through many yield / resume cycles while other collectives are queued:
    every kind, odd element counts, per-rank shuffled orders.  Results must be exact and yields must have happened."""
    nv = host_backend
    kinds = [nv.ALLREDUCE, nv.ALLGATHER, nv.REDUCESCATTER, nv.BROADCAST, nv.REDUCE]
    rng = random.Random(3)
    counts = [rng.choice([4097, 30011, 12345, 65536 + 7]) for _ in kinds] * 2
    kinds = kinds * 2
    comms = nv.Comm.init_loopback(nranks)
    stats = {}

    def body(r):
        c = comms[r]
        ctx = nv.RankCtx(r)
        bufs = []
        for i, (k, n) in enumerate(zip(kinds, counts)):
            ctx.prepare(i, c, k, n, nv.FLOAT32, root=i % nranks)
            sn = n * (nranks if k == nv.REDUCESCATTER else 1)
            rn = n * (nranks if k == nv.ALLGATHER else 1)
            sp, rp = c.alloc(sn * 4), c.alloc(rn * 4)
            bufs.append((sp, rp, host_array(sp, sn, np.float32), host_array(rp, rn, np.float32)))
        ctx.finalize()
        order_rng = random.Random(50 + r)
        for it in range(3):
            order = list(range(len(kinds)))
            order_rng.shuffle(order)
            for i in order:
                # position-dependent data: a slice that lands at the wrong offset cannot go unnoticed
                sn = bufs[i][2].size
                bufs[i][2][:] = (np.arange(sn, dtype=np.float32) % 251) + (r + 1) * 1000 + it
                ctx.run(i, bufs[i][0], bufs[i][1])
            assert ctx.wait_all(120000) == nv.SUCCESS
            for i, (k, n) in enumerate(zip(kinds, counts)):
                out = bufs[i][3]

                def src(q, m):
                    return (np.arange(m, dtype=np.float32) % 251) + (q + 1) * 1000 + it
                if k == nv.ALLREDUCE:
                    np.testing.assert_array_equal(out, sum(src(q, n) for q in range(nranks)))
                elif k == nv.REDUCESCATTER:
                    np.testing.assert_array_equal(out, sum(src(q, n * nranks)[r * n:(r + 1) * n] for q in range(nranks)))
                elif k == nv.ALLGATHER:
                    np.testing.assert_array_equal(out, np.concatenate([src(q, n) for q in range(nranks)]))
                elif k == nv.BROADCAST:
                    np.testing.assert_array_equal(out, src(i % nranks, n))
                elif k == nv.REDUCE and r == i % nranks:
                    np.testing.assert_array_equal(out, sum(src(q, n) for q in range(nranks)))
        import time
        time.sleep(0.05)
        stats[r] = ctx.stats()
        ctx.destroy()

    with _env(DFCCL_SLICE_BYTES=4096, DFCCL_DAEMON_BLOCKS=2, DFCCL_MIN_BYTES_PER_BLOCK=16384, DFCCL_IDLE_QUIT_US=2000):
        run_ranks(nranks, body, timeout=300)
    for c in comms:
        c.destroy()
    assert all(s["dataYields"] > 0 for s in stats.values()), stats


def test_unsliced_data_phase_never_yields(host_backend):
    nv = host_backend
    comms = nv.Comm.init_loopback(2)
    stats = {}

    def body(r):
        ctx = nv.RankCtx(r)
        for i in range(4):
            ctx.prepare(i, comms[r], nv.ALLREDUCE, 50000, nv.FLOAT32)
        ctx.finalize()
        p = comms[r].alloc(200000)
        host_array(p, 50000, np.float32)[:] = 1
        for i in range(4):
            ctx.run(i, p, comms[r].alloc(200000))
        assert ctx.wait_all(60000) == nv.SUCCESS
        import time
        time.sleep(0.05)
        stats[r] = ctx.stats()
        ctx.destroy()

    with _env(DFCCL_SLICE_BYTES=0):
        run_ranks(2, body)
    for c in comms:
        c.destroy()
    assert all(s["dataYields"] == 0 for s in stats.values())


@pytest.mark.parametrize("trigger_first", [False, True])
def test_deferred_submission_runs_when_released(host_backend, trigger_first):
    """dfcclRunDeferred publishes, dfcclTriggerOnStream releases; either order; one release per submission."""
    nv = host_backend
    comms = nv.Comm.init_loopback(2)

    def body(r):
        ctx = nv.RankCtx(r)
        ctx.prepare(0, comms[r], nv.ALLREDUCE, 1000, nv.FLOAT32)
        ctx.prepare(1, comms[r], nv.ALLREDUCE, 1000, nv.FLOAT32)
        ctx.finalize()
        p, q = comms[r].alloc(4000), comms[r].alloc(4000)
        a, b = host_array(p, 1000, np.float32), host_array(q, 1000, np.float32)
        for it in range(5):
            a[:] = r + 1 + it
            b[:] = 10 * (r + 1) + it
            ids = (0, 1) if (r + it) % 2 else (1, 0)               # ranks publish in different orders
            if trigger_first:
                for i in ids:
                    ctx.trigger_on_stream(i, 0)
            for i in ids:
                ctx.run_deferred(i, p if i == 0 else q, p if i == 0 else q)
            if not trigger_first:
                import time
                time.sleep(0.002)
                assert ctx.host_stats()["cqesDelivered"] == 2 * it          # nothing runs before its release
                for i in reversed(ids):
                    ctx.trigger_on_stream(i, 0)
            assert ctx.wait_all(60000) == nv.SUCCESS
            assert np.all(a == 3 + 2 * it) and np.all(b == 30 + 2 * it)
        ctx.destroy()

    run_ranks(2, body)
    for c in comms:
        c.destroy()


def test_patience_grows_after_successful_waits(host_backend):
    """With a tiny base budget and a large success factor, collectives still complete under disordered issue, and
    fewer context switches are needed than with the factor switched off."""
    nv = host_backend
    switches = {}
    for factor in (0, 50):
        comms = nv.Comm.init_loopback(2)
        st = {}

        def body(r):
            ctx = nv.RankCtx(r)
            for i in range(8):
                ctx.prepare(i, comms[r], nv.ALLREDUCE, 20000, nv.FLOAT32, algo=nv.ALGO_TWOSHOT)
            ctx.finalize()
            p = [comms[r].alloc(80000) for _ in range(8)]
            rng = random.Random(r)
            for it in range(10):
                order = list(range(8))
                rng.shuffle(order)
                for i in order:
                    host_array(p[i], 20000, np.float32)[:] = 1
                    ctx.run(i, p[i], p[i])
                assert ctx.wait_all(60000) == nv.SUCCESS
                for i in range(8):
                    assert np.all(host_array(p[i], 20000, np.float32) == 2)
            import time
            time.sleep(0.05)
            st[r] = ctx.stats()
            ctx.destroy()

        with _env(DFCCL_BASE_CTX_SWITCH_THRESHOLD=2, DFCCL_NUM_TRY_TASKQ_HEAD=1, DFCCL_RECV_SUCCESS_FACTOR=factor):
            run_ranks(2, body, timeout=240)
        for c in comms:
            c.destroy()
        switches[factor] = sum(s["ctxSwitches"] for s in st.values())
    assert switches[0] > 0            # the tiny budget did force preemptions; the run with patience completed as well


def test_grouped_send_recv_with_both_ends_in_one_thread(host_backend):
    """ncclCommInitAll, then one thread issues a group with a send and a receive on every communicator: every
    kernel of the flush is started before any is waited for, staging pieces are released without blocking."""
    nv = host_backend
    L = nv.lib()
    n = 3
    comms = nv.Comm.init_all(n)
    vp = C.c_void_p
    out = [np.full(3000, 7 + r, np.int32) for r in range(n)]
    inp = [np.zeros(3000, np.int32) for r in range(n)]           # plain host arrays: receives are staged
    for rep in range(3):
        nv.check(L.ncclGroupStart())
        for r in range(n):
            nv.check(L.ncclSend(vp(out[r].ctypes.data), 3000, nv.INT32, (r + 1) % n, comms[r].handle, None))
            nv.check(L.ncclRecv(vp(inp[r].ctypes.data), 3000, nv.INT32, (r - 1) % n, comms[r].handle, None))
        nv.check(L.ncclGroupEnd())
        for r in range(n):
            assert np.all(inp[r] == 7 + (r - 1) % n)
            inp[r][:] = 0
    for c in comms:
        c.destroy()


def test_registered_fused_operators_among_shuffled_data_parallel_buckets(host_backend):
    """tp2 x dp2 on four ranks: every rank registers two fused tensor-parallel operators (all-gather -> GEMM and
    GEMM -> reduce-scatter, on its tensor-parallel communicator) and four gradient all-reduces (on its data-parallel
    communicator) with ONE rank context, then issues the operators in model order and the all-reduces in its own
    shuffled order in between.  Everything completes, results match numpy, launches are counted."""
    from helpers import bf16_bits_to_f32, f32_to_bf16_bits
    nv = host_backend
    comms = nv.Comm.init_loopback(4)
    rows, k, n = 128, 64, 256
    rng0 = np.random.default_rng(5)
    xs = [f32_to_bf16_bits(rng0.standard_normal((rows, k)).astype(np.float32) * 0.5) for _ in range(4)]          # AG input rows per rank
    ws = [f32_to_bf16_bits(rng0.standard_normal((n, k)).astype(np.float32) * 0.5) for _ in range(4)]             # per-rank weights
    x2 = [f32_to_bf16_bits(rng0.standard_normal((2 * rows, k)).astype(np.float32) * 0.5) for _ in range(4)]     # RS input per rank
    counts = [1000, 40000, 257, 9000]
    stats = {}

    def body(r):
        c = comms[r]
        tp_comm = c.split(r // 2, r)              # ranks {0,1}, {2,3}
        dp_comm = c.split(r % 2, r)               # ranks {0,2}, {1,3}
        ctx = nv.RankCtx(r)
        ctx.prepare_fused(0, tp_comm, nv.FUSED_ALLGATHER_GEMM, rows, k, n)
        ctx.prepare_fused(1, tp_comm, nv.FUSED_GEMM_REDUCESCATTER, rows, k, n)
        bufs = []
        for i, cnt in enumerate(counts):
            ctx.prepare(2 + i, dp_comm, nv.ALLREDUCE, cnt, nv.FLOAT32)
            p = dp_comm.alloc(cnt * 4)
            bufs.append((p, host_array(p, cnt, np.float32)))
        ctx.finalize()
        with pytest.raises(nv.DfcclError):                       # the ids of fused operators are not submittable collectives
            ctx.run(0, bufs[0][0], bufs[0][0])
        order_rng = random.Random(900 + r)
        out_ag = np.zeros((2 * rows, n), np.uint16)
        out_rs = np.zeros((rows, n), np.uint16)
        for it in range(3):
            plan = [("f", 0), ("f", 1)] + [("d", i) for i in range(len(counts))]
            dp_part = [p for p in plan if p[0] == "d"]
            order_rng.shuffle(dp_part)
            cut = sorted(order_rng.sample(range(len(dp_part) + 1), 2))          # where the two operators sit among the buckets
            seq = dp_part[:cut[0]] + [("f", 0)] + dp_part[cut[0]:cut[1]] + [("f", 1)] + dp_part[cut[1]:]
            for kind, i in seq:
                if kind == "d":
                    bufs[i][1][:] = (r + 1) * (i + 1) + it
                    ctx.run(2 + i, bufs[i][0], bufs[i][0])
                elif i == 0:
                    ctx.run_fused(0, xs[r].ctypes.data, ws[r].ctypes.data, out_ag.ctypes.data, 0)
                else:
                    ctx.run_fused(1, x2[r].ctypes.data, ws[r].ctypes.data, out_rs.ctypes.data, 0)
            assert ctx.wait_all(60000) == nv.SUCCESS
            peer = r ^ 1
            lo, hi = min(r, peer), max(r, peer)
            gathered = np.concatenate([bf16_bits_to_f32(xs[lo]), bf16_bits_to_f32(xs[hi])])
            np.testing.assert_allclose(bf16_bits_to_f32(out_ag), gathered @ bf16_bits_to_f32(ws[r]).T, rtol=2e-2, atol=2e-2)
            full = sum(bf16_bits_to_f32(x2[q]) @ bf16_bits_to_f32(ws[q]).T for q in (lo, hi))
            mine = full[(r % 2) * rows:(r % 2 + 1) * rows]
            np.testing.assert_allclose(bf16_bits_to_f32(out_rs), mine, rtol=3e-2, atol=3e-2)
            for i, cnt in enumerate(counts):
                other = r ^ 2
                assert np.all(bufs[i][1] == (r + 1) * (i + 1) + it + (other + 1) * (i + 1) + it)
        stats[r] = ctx.stats()
        assert ctx.async_error() == nv.SUCCESS
        ctx.destroy()
        tp_comm.destroy()
        dp_comm.destroy()

    run_ranks(4, body, timeout=240)
    for c in comms:
        c.destroy()
    assert all(s["fusedLaunches"] == 6 and s["cqesDelivered"] == 12 for s in stats.values()), stats


def test_comm_abort_ends_a_stuck_stream_collective_quickly(host_backend):
    """One rank never joins the all-reduce.  ncclCommAbort from another thread raises the abort word first, so the
    waiting kernel leaves at its next look at it - long before its 30 s wait limit - and the abort call returns."""
    import threading
    import time
    nv = host_backend
    L = nv.lib()
    comms = nv.Comm.init_loopback(2)
    buf = comms[0].alloc(4096)
    result = {}

    def stuck():
        t0 = time.time()
        result["rc"] = L.ncclAllReduce(C.c_void_p(buf), C.c_void_p(buf), 1024, nv.FLOAT32, nv.SUM, comms[0].handle, None)
        result["s"] = time.time() - t0

    with _env(DFCCL_WAIT_TIMEOUT_MS=30000):
        t = threading.Thread(target=stuck, daemon=True)
        t.start()
        time.sleep(0.3)
        t0 = time.time()
        assert L.ncclCommAbort(comms[0].handle) == nv.SUCCESS
        abort_s = time.time() - t0
        t.join(10)
    assert not t.is_alive() and result["s"] < 5 and abort_s < 5, (result, abort_s)
    assert result["rc"] in (nv.ABORTED, nv.TIMEOUT)
    comms[1].destroy()


def test_group_defers_collectives_and_communicator_creation(host_backend):
    """One thread owns every rank: communicators created with ncclCommInitRank inside a group (each creation waits for
    the others, so they must run concurrently at ncclGroupEnd), then collectives of all ranks issued inside a group
    (on the host backend a collective is a blocking call: the group runs each communicator's calls on its own thread)."""
    nv = host_backend
    L = nv.lib()
    n = 3
    uid = nv.UniqueId()
    C.memmove(C.addressof(uid), nv.get_unique_id(), 128)
    handles = [C.c_void_p() for _ in range(n)]
    nv.check(L.ncclGroupStart())
    for r in range(n):
        nv.check(L.ncclCommInitRank(C.byref(handles[r]), n, uid, r))
        assert not handles[r].value                      # nothing is created before the group ends
    nv.check(L.ncclGroupEnd())
    assert all(h.value for h in handles)
    ins = [np.full(5000, r + 1, np.float32) for r in range(n)]
    outs = [np.zeros(5000, np.float32) for r in range(n)]
    gath = [np.zeros(3 * 100, np.int32) for r in range(n)]
    parts = [np.full(100, 10 * (r + 1), np.int32) for r in range(n)]
    for rep in range(2):
        nv.check(L.ncclGroupStart())
        for r in range(n):
            nv.check(L.ncclAllReduce(C.c_void_p(ins[r].ctypes.data), C.c_void_p(outs[r].ctypes.data), 5000, nv.FLOAT32, nv.SUM, handles[r], None))
            nv.check(L.ncclAllGather(C.c_void_p(parts[r].ctypes.data), C.c_void_p(gath[r].ctypes.data), 100, nv.INT32, handles[r], None))
        assert np.all(outs[0] == 0) or rep > 0               # recorded, not run
        nv.check(L.ncclGroupEnd())
        for r in range(n):
            assert np.all(outs[r] == 6)
            assert np.all(gath[r].reshape(3, 100) == np.array([10, 20, 30], np.int32)[:, None])
    for h in handles:
        nv.check(L.ncclCommDestroy(h))


def test_collectives_that_need_few_blocks_start_at_different_blocks(host_backend):
    """Five daemon blocks and collectives that need one to five of them: each starts at a block of its own (chosen per
    rank from the id) and wraps around the daemon's blocks; ranks meet by the relative block index only.  Every kind,
    position-dependent data, per-rank shuffled orders, several rounds."""
    nv = host_backend
    nranks = 3
    kinds = [nv.ALLREDUCE, nv.ALLGATHER, nv.REDUCESCATTER, nv.BROADCAST, nv.REDUCE] * 4
    counts = [(1 + (7 * i) % 5) * 1024 + 3 * i for i in range(len(kinds))]          # 1 .. 5 blocks at 4 KB per block
    comms = nv.Comm.init_loopback(nranks)

    def body(r):
        c = comms[r]
        ctx = nv.RankCtx(r)
        bufs = []
        for i, (k, n) in enumerate(zip(kinds, counts)):
            ctx.prepare(i + 40, c, k, n, nv.FLOAT32, root=i % nranks, algo=nv.ALGO_TWOSHOT if k == nv.ALLREDUCE else 0)
            sn = n * (nranks if k == nv.REDUCESCATTER else 1)
            rn = n * (nranks if k == nv.ALLGATHER else 1)
            sp, rp = c.alloc(sn * 4), c.alloc(rn * 4)
            bufs.append((sp, rp, host_array(sp, sn, np.float32), host_array(rp, rn, np.float32)))
        ctx.finalize()
        order_rng = random.Random(9 + r)
        for it in range(3):
            order = list(range(len(kinds)))
            order_rng.shuffle(order)
            for i in order:
                sn = bufs[i][2].size
                bufs[i][2][:] = (np.arange(sn, dtype=np.float32) % 127) + (r + 1) * 100 + it
                ctx.run(i + 40, bufs[i][0], bufs[i][1])
            assert ctx.wait_all(120000) == nv.SUCCESS
            for i, (k, n) in enumerate(zip(kinds, counts)):
                out = bufs[i][3]

                def src(q, m):
                    return (np.arange(m, dtype=np.float32) % 127) + (q + 1) * 100 + it
                if k == nv.ALLREDUCE:
                    np.testing.assert_array_equal(out, sum(src(q, n) for q in range(nranks)))
                elif k == nv.REDUCESCATTER:
                    np.testing.assert_array_equal(out, sum(src(q, n * nranks)[r * n:(r + 1) * n] for q in range(nranks)))
                elif k == nv.ALLGATHER:
                    np.testing.assert_array_equal(out, np.concatenate([src(q, n) for q in range(nranks)]))
                elif k == nv.BROADCAST:
                    np.testing.assert_array_equal(out, src(i % nranks, n))
                elif k == nv.REDUCE and r == i % nranks:
                    np.testing.assert_array_equal(out, sum(src(q, n) for q in range(nranks)))
        ctx.destroy()

    with _env(DFCCL_DAEMON_BLOCKS=5, DFCCL_MIN_BYTES_PER_BLOCK=4096, DFCCL_PUSH=0, DFCCL_IDLE_QUIT_US=2000):
        run_ranks(nranks, body, timeout=300)
    for c in comms:
        c.destroy()
