"""The NVLS all-reduce schedule on the host backend: the switch's multicast view is emulated by a loop
over the members' arena blocks, everything around it (slots, staging, rendezvous, in-place buffers,
fused scale and cast, fall-back when the arena is full) is the code that runs on GPUs."""
import ctypes as C

import numpy as np
import pytest

from helpers import bf16_bits_to_f32, f32_to_bf16_bits, host_array, np_dtype, run_ranks


def _inputs(nv, dt, n, nranks, seed):
    out = []
    for r in range(nranks):
        x = np.random.default_rng(seed + r).uniform(-1, 1, n).astype(np.float32)
        out.append(f32_to_bf16_bits(x) if dt == nv.BFLOAT16 else x.astype(np_dtype(nv, dt)))
    return out


def _f32(nv, dt, a):
    return bf16_bits_to_f32(a) if dt == nv.BFLOAT16 else a.astype(np.float32)


@pytest.mark.parametrize("dt_name,out_name", [("FLOAT32", "FLOAT32"), ("BFLOAT16", "BFLOAT16"), ("BFLOAT16", "FLOAT32"),
                                              ("FLOAT16", "FLOAT16"), ("FLOAT16", "FLOAT32")])
@pytest.mark.parametrize("where", ["arena", "heap", "user"])
def test_daemon_allreduce_nvls(host_backend, dt_name, out_name, where):
    nv = host_backend
    dt, odt = getattr(nv, dt_name), getattr(nv, out_name)
    nranks, count, scale = 4, 40 * 1024, 0.25
    comms = nv.Comm.init_loopback(nranks)
    ins = _inputs(nv, dt, count, nranks, 7)
    exp = sum(_f32(nv, dt, a).astype(np.float64) for a in ins) * scale
    got = {}

    def body(r):
        c = comms[r]
        assert c.nvls_init(8 << 20)
        ctx = nv.RankCtx(r)
        ctx.prepare(3, c, nv.ALLREDUCE, count, dt, out_dtype=odt, op=nv.SUM, scale=scale, algo=nv.ALGO_NVLS)
        ctx.finalize()
        es, eo = nv.DTYPE_SIZE[dt], nv.DTYPE_SIZE[odt]
        keep = []
        if where == "arena":
            sp, rp = c.nvls_alloc(count * es), c.nvls_alloc(count * eo)
        elif where == "heap":
            sp, rp = c.alloc(count * es), c.alloc(count * eo)
        else:
            a, b = np.zeros(count, np_dtype(nv, dt)), np.zeros(count, np_dtype(nv, odt))
            keep += [a, b]
            sp, rp = a.ctypes.data, b.ctypes.data
        sv, rv = host_array(sp, count, np_dtype(nv, dt)), host_array(rp, count, np_dtype(nv, odt))
        for it in range(3):
            sv[:] = ins[r]
            rv[:] = 0
            ctx.run(3, sp, rp)
            assert ctx.wait(3, 30000) == nv.SUCCESS
        got[r] = rv.copy()
        st = ctx.stats()
        ctx.destroy()
        assert st["waitTimeouts"] == 0

    run_ranks(nranks, body)
    for c in comms:
        c.destroy()
    tol = 2e-2 if odt != nv.FLOAT32 or dt != nv.FLOAT32 else 1e-5
    for r in range(nranks):
        np.testing.assert_allclose(_f32(nv, odt, got[r]), exp, rtol=tol, atol=tol)


def test_stream_allreduce_nvls_chunked_and_in_place(host_backend, monkeypatch):
    """ncclAllReduce picks the schedule by size; a message larger than the staging slots goes in pieces;
    a buffer from the arena is reduced in place."""
    nv = host_backend
    monkeypatch.setenv("DFCCL_NVLS_STREAM_BYTES", str(1 << 20))
    monkeypatch.setenv("DFCCL_NVLS_MIN_BYTES", "4096")
    monkeypatch.setenv("DFCCL_ALGO", "nvls")
    nranks, count = 2, 600 * 1024 + 64          # 2.4 MB of fp32: 5 pieces of 512 KB
    comms = nv.Comm.init_loopback(nranks)
    ins = _inputs(nv, nv.FLOAT32, count, nranks, 3)
    exp = ins[0].astype(np.float64) + ins[1]
    got = {}

    def body(r):
        c = comms[r]
        assert c.nvls_init(16 << 20)
        a, b = ins[r].copy(), np.zeros(count, np.float32)
        nv.check(nv.lib().ncclAllReduce(a.ctypes.data, b.ctypes.data, count, nv.FLOAT32, nv.SUM, c.handle, None))
        p = c.nvls_alloc(count * 4)
        v = host_array(p, count, np.float32)
        v[:] = ins[r]
        nv.check(nv.lib().ncclAllReduce(p, p, count, nv.FLOAT32, nv.SUM, c.handle, None))
        got[r] = (b, v.copy())

    run_ranks(nranks, body)
    for c in comms:
        c.destroy()
    for r in range(nranks):
        np.testing.assert_allclose(got[r][0], exp, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(got[r][1], exp, rtol=1e-5, atol=1e-5)


def test_arena_full_falls_back(host_backend):
    nv = host_backend
    nranks, count = 2, 1 << 20
    comms = nv.Comm.init_loopback(nranks)
    ins = _inputs(nv, nv.FLOAT32, count, nranks, 5)
    exp = ins[0] + ins[1]

    def body(r):
        c = comms[r]
        assert c.nvls_init(2 << 20)                # too small for 4 MB in + 4 MB out
        ctx = nv.RankCtx(r)
        ctx.prepare(0, c, nv.ALLREDUCE, count, nv.FLOAT32, algo=nv.ALGO_NVLS)
        ctx.finalize()
        a, b = ins[r].copy(), np.zeros(count, np.float32)
        ctx.run(0, a.ctypes.data, b.ctypes.data)
        assert ctx.wait(0, 30000) == nv.SUCCESS
        ctx.destroy()
        np.testing.assert_allclose(b, exp, rtol=1e-5, atol=1e-5)

    run_ranks(nranks, body)
    for c in comms:
        c.destroy()


@pytest.mark.parametrize("kind", ["reducescatter", "allgather"])
@pytest.mark.parametrize("where", ["arena", "heap", "user"])
def test_daemon_reducescatter_allgather_nvls(host_backend, kind, where):
    """The multimem forms of reduce-scatter (switch reduces, result stays local) and all-gather (one multicast store
    per piece), pinned at registration; the member-side buffer (reduce-scatter output, all-gather input) is used
    where it is, the shared side lives in the arena or is staged through the collective's slot."""
    nv = host_backend
    nranks, count, scale = 4, 12 * 1024, 0.5
    rs = kind == "reducescatter"
    dt, odt = (nv.BFLOAT16, nv.FLOAT32) if rs else (nv.FLOAT32, nv.FLOAT32)
    comms = nv.Comm.init_loopback(nranks)
    send_n = count * nranks if rs else count
    recv_n = count if rs else count * nranks
    ins = _inputs(nv, dt, send_n, nranks, 21)
    got = {}

    def body(r):
        c = comms[r]
        assert c.nvls_init(8 << 20)
        ctx = nv.RankCtx(r)
        ctx.prepare(5, c, nv.REDUCESCATTER if rs else nv.ALLGATHER, count, dt, out_dtype=odt, op=nv.SUM,
                    scale=scale if rs else 1.0, algo=nv.ALGO_NVLS)
        ctx.finalize()
        es, eo = nv.DTYPE_SIZE[dt], nv.DTYPE_SIZE[odt]
        keep = []

        def buf(n, e, npdt, shared):
            if where == "arena" and shared:
                return c.nvls_alloc(n * e)
            if where in ("arena", "heap"):
                return c.alloc(n * e)
            a = np.zeros(n, npdt)
            keep.append(a)
            return a.ctypes.data
        sp = buf(send_n, es, np_dtype(nv, dt), shared=rs)          # the reduce-scatter input is what the switch reads
        rp = buf(recv_n, eo, np_dtype(nv, odt), shared=not rs)     # the all-gather output is what the switch writes
        sv, rv = host_array(sp, send_n, np_dtype(nv, dt)), host_array(rp, recv_n, np_dtype(nv, odt))
        for it in range(3):
            sv[:] = ins[r]
            rv[:] = 0
            ctx.run(5, sp, rp)
            assert ctx.wait(5, 30000) == nv.SUCCESS
        got[r] = rv.copy()
        st = ctx.stats()
        ctx.destroy()
        assert st["waitTimeouts"] == 0

    run_ranks(nranks, body)
    for c in comms:
        c.destroy()
    if rs:
        tot = sum(_f32(nv, dt, a).astype(np.float64) for a in ins) * scale
        for r in range(nranks):
            np.testing.assert_allclose(got[r], tot[r * count:(r + 1) * count], rtol=2e-2, atol=2e-2)
    else:
        exp = np.concatenate(ins)
        for r in range(nranks):
            np.testing.assert_array_equal(got[r], exp)


@pytest.mark.parametrize("where", ["arena", "heap", "user"])
@pytest.mark.parametrize("root", [0, 2])
def test_daemon_broadcast_nvls(host_backend, where, root):
    """Broadcast on the multimem schedule, pinned at registration: the root's multicast stores put its buffer into
    every member's output (in the arena, or this collective's arena slot when the caller's buffer lives elsewhere);
    the others move nothing and wait for the root's done flag.  The root's input is used where it is."""
    nv = host_backend
    nranks, count = 4, 20 * 1024 + 4
    comms = nv.Comm.init_loopback(nranks)
    got = {}

    def body(r):
        c = comms[r]
        assert c.nvls_init(8 << 20)
        ctx = nv.RankCtx(r)
        ctx.prepare(7, c, nv.BROADCAST, count, nv.FLOAT32, root=root, algo=nv.ALGO_NVLS)
        ctx.finalize()
        keep = []
        if where == "arena":
            rp = c.nvls_alloc(count * 4)
        elif where == "heap":
            rp = c.alloc(count * 4)
        else:
            keep.append(np.zeros(count, np.float32))
            rp = keep[-1].ctypes.data
        rv = host_array(rp, count, np.float32)
        sv = np.zeros(count, np.float32)
        res = []
        for it in range(3):
            sv[:] = np.arange(count, dtype=np.float32) + 1000 * (r + 1) + it
            rv[:] = -1
            ctx.run(7, sv.ctypes.data if r == root else 0, rp)
            assert ctx.wait(7, 30000) == nv.SUCCESS
            res.append(rv.copy())
        got[r] = res
        st = ctx.stats()
        ctx.destroy()
        assert st["waitTimeouts"] == 0

    run_ranks(nranks, body)
    for c in comms:
        c.destroy()
    for r in range(nranks):
        for it in range(3):
            np.testing.assert_array_equal(got[r][it], np.arange(count, dtype=np.float32) + 1000 * (root + 1) + it)
