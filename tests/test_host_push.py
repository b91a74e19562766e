"""Push schedule of small all-reduces on the host backend: inputs are written into slots at the peers together
with the arrival flag, every rank reduces locally - one hop, the user's buffers used where they are (heap or
not), no done handshake, slots alternating with the call's parity."""
import numpy as np
import pytest

from helpers import bf16_bits_to_f32, f32_to_bf16_bits, host_array, np_dtype, run_ranks


@pytest.mark.parametrize("world", [2, 3, 4])
@pytest.mark.parametrize("where", ["heap", "user"])
def test_daemon_push_allreduce(host_backend, world, where):
    nv = host_backend
    comms = nv.Comm.init_loopback(world)
    counts = [1, 37, 4096, 20000]
    iters = 5                                     # several calls per id: both parities of the slots, reuse
    got = {}

    def body(r):
        c = comms[r]
        ctx = nv.RankCtx(r)
        for i, n in enumerate(counts):
            ctx.prepare(i, c, nv.ALLREDUCE, n, nv.BFLOAT16, out_dtype=nv.FLOAT32, op=nv.SUM, scale=0.5, algo=nv.ALGO_PUSH)
        ctx.finalize()
        outs = []
        for i, n in enumerate(counts):
            if where == "heap":
                sp, rp = c.alloc(2 * n + 64), c.alloc(4 * n + 64)
                sv, rv = host_array(sp, n, np.uint16), host_array(rp, n, np.float32)
            else:
                sv, rv = np.zeros(n, np.uint16), np.zeros(n, np.float32)
                sp, rp = sv.ctypes.data, rv.ctypes.data
            res = []
            for it in range(iters):
                sv[:] = f32_to_bf16_bits(np.full(n, float(r + 1 + it), np.float32))
                ctx.run(i, sp, rp)
                assert ctx.wait(i, 30000) == nv.SUCCESS
                res.append(rv.copy())
            outs.append((sv, rv, res))
        got[r] = outs
        st = ctx.stats()
        ctx.destroy()
        assert st["waitTimeouts"] == 0

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    for r in range(world):
        for i, n in enumerate(counts):
            for it in range(iters):
                exp = 0.5 * sum(j + 1 + it for j in range(world))
                assert np.all(got[r][i][2][it] == exp), (r, i, it, got[r][i][2][it][:4], exp)


@pytest.mark.parametrize("world", [2, 3, 4])
@pytest.mark.parametrize("where", ["heap", "user", "inplace"])
@pytest.mark.parametrize("kind", ["allgather", "reducescatter"])
def test_daemon_push_allgather_reducescatter(host_backend, world, where, kind):
    """Small all-gathers and reduce-scatters take the same one-hop schedule: every member puts what each peer needs of
    its input into its slot there (its piece; chunk j for member j) together with the arrival flag, and finishes
    locally.  Odd counts put the chunks off the 16-byte grid; several calls per id use both slot parities."""
    nv = host_backend
    comms = nv.Comm.init_loopback(world)
    counts = [1, 37, 4099, 20000]
    iters = 4
    kid = nv.ALLGATHER if kind == "allgather" else nv.REDUCESCATTER
    got = {}

    def val(r, it, q):                    # element value: depends on the rank, the call and (reduce-scatter) the chunk
        return float(r + 1 + it + 3 * q)

    def body(r):
        c = comms[r]
        ctx = nv.RankCtx(r)
        for i, n in enumerate(counts):
            ctx.prepare(i, c, kid, n, nv.FLOAT32, op=nv.SUM)          # schedule left to the library: push by size
        ctx.finalize()
        res = {}
        for i, n in enumerate(counts):
            sn, rn = (n, n * world) if kind == "allgather" else (n * world, n)
            if where == "heap":
                sv, rv = host_array(c.alloc(4 * sn + 64), sn, np.float32), host_array(c.alloc(4 * rn + 64), rn, np.float32)
            elif where == "user":
                sv, rv = np.zeros(sn, np.float32), np.zeros(rn, np.float32)
            else:                                                     # in place, NCCL conventions
                big = host_array(c.alloc(4 * n * world + 64), n * world, np.float32)
                sv, rv = (big[r * n:(r + 1) * n], big) if kind == "allgather" else (big, big[r * n:(r + 1) * n])
            res[i] = []
            for it in range(iters):
                if kind == "allgather":
                    sv[:] = val(r, it, 0)
                else:
                    for q in range(world):
                        sv[q * n:(q + 1) * n] = val(r, it, q)
                ctx.run(i, sv.ctypes.data, rv.ctypes.data)
                assert ctx.wait(i, 30000) == nv.SUCCESS
                res[i].append(rv.copy())
        got[r] = res
        st = ctx.stats()
        ctx.destroy()
        assert st["waitTimeouts"] == 0

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    for r in range(world):
        for i, n in enumerate(counts):
            for it in range(iters):
                out = got[r][i][it]
                if kind == "allgather":
                    for q in range(world):
                        assert np.all(out[q * n:(q + 1) * n] == val(q, it, 0)), (r, i, it, q)
                else:
                    assert np.all(out == sum(val(q, it, r) for q in range(world))), (r, i, it, out[:4])


def test_stream_push_allreduce_mixed_with_other_schedules(host_backend, monkeypatch):
    """Small calls take the push schedule (DFCCL_PUSH=1), larger ones the handshaking schedules, on one communicator."""
    nv = host_backend
    monkeypatch.setenv("DFCCL_PUSH", "1")
    world = 3
    comms = nv.Comm.init_loopback(world)
    sizes = [8, 300000, 1000, 70000, 64, 500000, 5]          # 256 KB is the switch-over
    got = {}

    def body(r):
        c, L = comms[r], nv.lib()
        res = []
        for rep in range(3):
            for n in sizes:
                a = np.full(n, float(r + 1 + rep), np.float32)
                nv.check(L.ncclAllReduce(a.ctypes.data, a.ctypes.data, n, nv.FLOAT32, nv.SUM, c.handle, None))
                res.append((n, rep, float(a.min()), float(a.max())))
        got[r] = res

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    for r in range(world):
        for n, rep, lo, hi in got[r]:
            exp = float(sum(j + 1 + rep for j in range(world)))
            assert lo == exp and hi == exp, (r, n, rep, lo, hi, exp)
