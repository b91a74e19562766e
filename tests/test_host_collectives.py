"""Every collective, dtype and operator through the daemon on the host backend
(CPU threads play the thread blocks, shared memory plays peer memory) against a
numpy reference of the same operation."""
import numpy as np
import pytest

from helpers import bf16_bits_to_f32, f32_to_bf16_bits, host_array, np_dtype, run_ranks

KINDS = ["allreduce", "allgather", "reducescatter", "broadcast", "reduce"]


def _make_input(nv, dt, n, rank, rng):
    npdt = np_dtype(nv, dt)
    if dt == nv.BFLOAT16:
        return f32_to_bf16_bits(rng.uniform(-1, 1, n).astype(np.float32))
    if np.issubdtype(npdt, np.floating):
        return rng.uniform(-1, 1, n).astype(npdt)
    if np.issubdtype(npdt, np.signedinteger):
        return rng.integers(-5, 6, n).astype(npdt)
    return rng.integers(0, 7, n).astype(npdt)


def _to_math(nv, dt, a):
    if dt == nv.BFLOAT16:
        return bf16_bits_to_f32(a).astype(np.float64)
    return a.astype(np.float64) if np.issubdtype(a.dtype, np.floating) else a.astype(np.int64)


def _reference(nv, op, stacked, nranks, is_float):
    if op == nv.SUM:
        return stacked.sum(0)
    if op == nv.PROD:
        return stacked.prod(0)
    if op == nv.MAX:
        return stacked.max(0)
    if op == nv.MIN:
        return stacked.min(0)
    s = stacked.sum(0)
    return s / nranks if is_float else np.trunc(s / nranks).astype(np.int64)


def _run_case(nv, kind, nranks, count, dt, op=None, root=0, in_place=False, heap=True, algo=0, out_dt=None, scale=1.0, iters=2):
    op = nv.SUM if op is None else op
    out_dt = dt if out_dt is None else out_dt
    comms = nv.Comm.init_loopback(nranks)
    kid = getattr(nv, kind.upper())
    es, eo = nv.DTYPE_SIZE[dt], nv.DTYPE_SIZE[out_dt]
    send_n = count * nranks if kind == "reducescatter" else count
    recv_n = count * nranks if kind == "allgather" else count
    inputs = [[_make_input(nv, dt, send_n, r, np.random.default_rng(1000 * it + r)) for r in range(nranks)] for it in range(iters)]
    results = {}

    def body(r):
        c = comms[r]
        ctx = nv.RankCtx(r)
        ctx.prepare(7, c, kid, count, dt, out_dtype=out_dt, op=op, root=root, scale=scale, algo=algo)
        ctx.finalize()
        keep = []
        if heap:
            sp = c.alloc(max(send_n * es, recv_n * eo) + 64)
            if in_place:
                rp = sp + (r * count * es if kind == "allgather" else 0)
                if kind == "allgather":
                    sp, rp = rp, sp                       # send is my slot inside the gathered buffer
                elif kind == "reducescatter":
                    rp = sp + r * count * es
                else:
                    rp = sp
            else:
                rp = c.alloc(recv_n * eo + 64)
            sv = host_array(sp, send_n, np_dtype(nv, dt))
            rv = host_array(rp, recv_n, np_dtype(nv, out_dt))
        else:
            sv = np.zeros(send_n, np_dtype(nv, dt))
            rv = np.zeros(recv_n, np_dtype(nv, out_dt))
            sp, rp = sv.ctypes.data, rv.ctypes.data
            keep += [sv, rv]
        outs = []
        for it in range(iters):
            sv[:] = inputs[it][r]
            ctx.run(7, sp, rp)
            assert ctx.wait(7, 30000) == nv.SUCCESS
            outs.append(rv.copy())
        results[r] = outs
        assert ctx.wait_all(1000) == nv.SUCCESS
        ctx.destroy()

    run_ranks(nranks, body)
    for c in comms:
        c.destroy()

    is_float = dt in (nv.FLOAT16, nv.FLOAT32, nv.FLOAT64, nv.BFLOAT16)
    tol = {nv.FLOAT16: 2e-2, nv.BFLOAT16: 6e-2, nv.FLOAT32: 1e-5, nv.FLOAT64: 1e-12}.get(out_dt if is_float else dt, 0)
    for it in range(iters):
        stacked = np.stack([_to_math(nv, dt, inputs[it][r]) for r in range(nranks)])
        for r in range(nranks):
            got = _to_math(nv, out_dt, results[r][it])
            if kind == "allreduce":
                exp = _reference(nv, op, stacked, nranks, is_float) * (scale if is_float else 1)
            elif kind == "reduce":
                if r != root:
                    continue
                exp = _reference(nv, op, stacked, nranks, is_float)
            elif kind == "reducescatter":
                exp = _reference(nv, op, stacked, nranks, is_float)[r * count:(r + 1) * count]
            elif kind == "allgather":
                exp = stacked.reshape(-1)
            else:
                exp = stacked[root]
            if not is_float and dt in (nv.INT8, nv.UINT8, nv.INT32, nv.UINT32):
                exp = exp.astype(np_dtype(nv, dt)).astype(np.int64)   # wrap-around like the device
            if tol:
                np.testing.assert_allclose(got, exp, rtol=tol, atol=tol * max(1.0, np.abs(exp).max()), err_msg=f"{kind} rank {r} it {it}")
            else:
                np.testing.assert_array_equal(got, exp, err_msg=f"{kind} rank {r} it {it}")


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("nranks", [1, 2, 4])
def test_kinds_fp32(host_backend, kind, nranks):
    _run_case(host_backend, kind, nranks, 10007, host_backend.FLOAT32, root=nranks - 1)


@pytest.mark.parametrize("dt_name", ["INT8", "UINT8", "INT32", "UINT32", "INT64", "UINT64", "FLOAT16", "FLOAT32", "FLOAT64", "BFLOAT16"])
@pytest.mark.parametrize("op_name", ["SUM", "PROD", "MAX", "MIN", "AVG"])
def test_allreduce_every_dtype_and_op(host_backend, dt_name, op_name):
    nv = host_backend
    _run_case(nv, "allreduce", 3, 2051, getattr(nv, dt_name), op=getattr(nv, op_name), iters=1)


@pytest.mark.parametrize("kind", ["reducescatter", "reduce"])
@pytest.mark.parametrize("dt_name", ["INT32", "BFLOAT16", "FLOAT64"])
def test_reducing_kinds_other_dtypes(host_backend, kind, dt_name):
    nv = host_backend
    _run_case(nv, kind, 4, 777, getattr(nv, dt_name), op=nv.SUM, root=2, iters=1)


@pytest.mark.parametrize("kind", KINDS)
def test_in_place(host_backend, kind):
    _run_case(host_backend, kind, 4, 4096, host_backend.FLOAT32, in_place=True, root=1)


@pytest.mark.parametrize("kind", KINDS)
def test_buffers_outside_the_heap_are_staged(host_backend, kind):
    _run_case(host_backend, kind, 3, 5000, host_backend.FLOAT32, heap=False, root=0)


@pytest.mark.parametrize("algo_name", ["ALGO_ONESHOT", "ALGO_TWOSHOT"])
@pytest.mark.parametrize("count", [1, 15, 16, 17, 1000, 70001])
def test_allreduce_schedules_and_odd_sizes(host_backend, algo_name, count):
    nv = host_backend
    _run_case(nv, "allreduce", 4, count, nv.FLOAT32, algo=getattr(nv, algo_name), iters=1)


def test_oneshot_in_place_takes_the_private_copy_path(host_backend):
    nv = host_backend
    _run_case(nv, "allreduce", 4, 3000, nv.FLOAT32, algo=nv.ALGO_ONESHOT, in_place=True)


def test_eight_ranks(host_backend):
    _run_case(host_backend, "allreduce", 8, 4099, host_backend.FLOAT32, iters=1)


@pytest.mark.parametrize("kind", ["allreduce", "allgather", "reducescatter", "broadcast"])
def test_twenty_ranks(host_backend, kind, monkeypatch):
    """More ranks than one node has GPUs (an NVLink domain may span a rack): the engine serves up to 64 members per
    communicator; 20 thread-ranks run every schedule family (push for the small kinds, two-shot for the large one)."""
    monkeypatch.setenv("DFCCL_HEAP_BYTES", str(16 << 20))
    nv = host_backend
    _run_case(nv, kind, 20, 611, nv.FLOAT32, root=17, iters=2)
    if kind == "allreduce":
        _run_case(nv, kind, 20, 100003, nv.FLOAT32, iters=1)


@pytest.mark.parametrize("in_name,out_name", [("BFLOAT16", "FLOAT32"), ("FLOAT16", "FLOAT32"), ("FLOAT32", "BFLOAT16"), ("FLOAT32", "FLOAT16")])
def test_fused_scale_and_cast(host_backend, in_name, out_name):
    """Gradient path: out = cast(scale * sum(in)), applied in registers before the only store."""
    nv = host_backend
    _run_case(nv, "allreduce", 4, 6001, getattr(nv, in_name), out_dt=getattr(nv, out_name), scale=0.25)
