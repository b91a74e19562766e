"""The daemon kernel on a real GPU.  Several ranks share ONE device: their daemons are
one cooperative launch (blocks of all ranks co-resident), so every multi-rank code path
- flags in peer heaps, preemption, quit / relaunch - runs on a single B200.
References are plain PyTorch fp32 computations of the same operation."""
import os
import random
import threading
import time

import pytest
import torch

from helpers import run_ranks

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nv():
    from dfccl_b200 import native
    native.lib()
    native.set_backend("cuda")
    import ctypes
    loaded = open("/proc/self/maps").read()
    assert "libdfccl.so" in loaded, "native library is not loaded"
    return native


def _t(ptr, n, dtype):
    from dfccl_b200.utils import tensor_from_ptr
    return tensor_from_ptr(ptr, (n,), dtype, "cuda:0")


TORCH_OF = {"FLOAT32": torch.float32, "BFLOAT16": torch.bfloat16, "FLOAT16": torch.float16, "INT32": torch.int32,
            "FLOAT64": torch.float64, "INT64": torch.int64, "UINT8": torch.uint8, "INT8": torch.int8}


def _loopback_case(nv, kind, nranks, count, dt_name, *, op="SUM", root=0, out_name=None, scale=1.0, algo=0, heap=True,
                   in_place=False, iters=2, blocks=None, skew=(0, 0), transport="peer"):
    torch.cuda.set_device(0)
    dt, out_dt = TORCH_OF[dt_name], TORCH_OF[out_name or dt_name]
    kid = getattr(nv, kind.upper())
    send_n = count * nranks if kind == "reducescatter" else count
    recv_n = count * nranks if kind == "allgather" else count
    g = torch.Generator(device="cpu").manual_seed(1234)
    def mk():
        if dt.is_floating_point:
            return (torch.rand(send_n, generator=g) * 2 - 1).to(dt)
        return torch.randint(-5 if dt != torch.uint8 else 0, 6, (send_n,), generator=g).to(dt)
    inputs = [[mk() for _ in range(nranks)] for _ in range(iters)]
    env = {"DFCCL_DAEMON_BLOCKS": str(blocks or max(1, min(8, 96 // nranks)))}
    old = {k: os.environ.get(k) for k in env}
    os.environ.update(env)
    comms = nv.Comm.init_loopback(nranks, 0)
    assert all(c.transport() == (transport if nranks > 1 else "peer") for c in comms), [c.transport() for c in comms]
    results = {}

    def body(r):
        torch.cuda.set_device(0)
        c = comms[r]
        ctx = nv.RankCtx(r, 0)
        ctx.prepare(3, c, kid, count, getattr(nv, dt_name), out_dtype=getattr(nv, out_name or dt_name), op=getattr(nv, op),
                    root=root, scale=scale, algo=algo)
        ctx.finalize()
        es, eo = inputs[0][0].element_size(), torch.empty((), dtype=out_dt).element_size()
        if heap:
            sp = c.alloc(max(send_n * es, recv_n * eo) + 256)
            if in_place:
                rp = sp
                if kind == "allgather":
                    sp = rp + r * count * es
                elif kind == "reducescatter":
                    rp = sp + r * count * es
            else:
                rp = c.alloc(recv_n * eo + 256)
                sp, rp = sp + skew[0] * es, rp + skew[1] * eo       # buffers that start off the 16-byte grid
            sv, rv = _t(sp, send_n, dt), _t(rp, recv_n, out_dt)
        else:
            sv = torch.empty(send_n, dtype=dt, device="cuda:0")
            rv = torch.zeros(recv_n, dtype=out_dt, device="cuda:0")
            sp, rp = sv.data_ptr(), rv.data_ptr()
        outs = []
        for it in range(iters):
            sv.copy_(inputs[it][r])
            torch.cuda.current_stream().synchronize()
            ctx.run(3, sp, rp)
            assert ctx.wait(3, 60000) == nv.SUCCESS
            outs.append(rv.clone().cpu())
        results[r] = (outs, ctx.stats())
        ctx.destroy()

    try:
        run_ranks(nranks, body, timeout=180)
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    for c in comms:
        c.destroy()

    for it in range(iters):
        st = torch.stack([x.double() if dt.is_floating_point else x.long() for x in inputs[it]])
        red = {"SUM": st.sum(0), "PROD": st.prod(0), "MAX": st.max(0).values, "MIN": st.min(0).values,
               "AVG": st.sum(0) / nranks}[op] * (scale if dt.is_floating_point else 1)
        for r in range(nranks):
            got = results[r][0][it].double() if out_dt.is_floating_point else results[r][0][it].long()
            if kind == "allreduce":
                exp = red
            elif kind == "reduce":
                if r != root:
                    continue
                exp = red
            elif kind == "reducescatter":
                exp = red[r * count:(r + 1) * count]
            elif kind == "allgather":
                exp = st.reshape(-1)
            else:
                exp = st[root]
            if out_dt.is_floating_point:
                tol = {torch.float32: 1e-5, torch.float64: 1e-12, torch.float16: 2e-2, torch.bfloat16: 6e-2}[out_dt]
                torch.testing.assert_close(got, exp.double(), rtol=tol, atol=tol * max(1.0, float(exp.abs().max())))
            else:
                if dt in (torch.int8, torch.uint8, torch.int32):
                    exp = exp.to(dt).long()
                assert torch.equal(got, exp)
    return results


@pytest.mark.parametrize("kind", ["allreduce", "allgather", "reducescatter", "broadcast", "reduce"])
@pytest.mark.parametrize("nranks", [1, 2, 4])
def test_loopback_kinds_fp32(nv, kind, nranks):
    _loopback_case(nv, kind, nranks, 100003, "FLOAT32", root=nranks - 1)


@pytest.mark.parametrize("kind", ["allreduce", "allgather", "reducescatter"])
@pytest.mark.parametrize("nranks,count,heap,in_place", [(2, 1, True, False), (4, 4099, True, False), (8, 1001, False, False),
                                                        (4, 30001, True, True), (3, 65536, False, False)])
def test_loopback_small_messages_take_one_hop(nv, kind, nranks, count, heap, in_place):
    """Pieces up to 256 KB: every member stores what each peer needs of its input into its slot there together with the
    arrival flag and finishes locally (push schedule) - all-reduce, all-gather and reduce-scatter, odd counts (chunks
    off the 16-byte grid), buffers in and outside the heap, in place, three calls per id (both slot parities)."""
    _loopback_case(nv, kind, nranks, count, "FLOAT32", iters=3, heap=heap, in_place=in_place, blocks=4)


@pytest.mark.parametrize("dt", ["BFLOAT16", "FLOAT16", "INT32", "FLOAT64", "INT64", "UINT8", "INT8"])
def test_loopback_allreduce_dtypes(nv, dt):
    _loopback_case(nv, "allreduce", 4, 65537, dt, iters=1)


@pytest.mark.parametrize("op", ["PROD", "MAX", "MIN", "AVG"])
def test_loopback_allreduce_ops(nv, op):
    _loopback_case(nv, "allreduce", 4, 4099, "FLOAT32", op=op, iters=1)


@pytest.mark.parametrize("algo", ["ALGO_ONESHOT", "ALGO_TWOSHOT"])
@pytest.mark.parametrize("count", [1, 17, 4096, 1 << 20])
def test_loopback_allreduce_schedules(nv, algo, count):
    _loopback_case(nv, "allreduce", 4, count, "BFLOAT16", algo=getattr(nv, algo), iters=1)


@pytest.mark.parametrize("kind", ["allreduce", "allgather", "reducescatter", "broadcast", "reduce"])
@pytest.mark.parametrize("dt,count,skew", [("BFLOAT16", 150001, (0, 0)), ("BFLOAT16", 150001, (3, 5)), ("UINT8", 70003, (1, 6)),
                                           ("FLOAT32", 99999, (1, 3))])
def test_loopback_buffers_off_the_16_byte_grid(nv, kind, dt, count, skew):
    """Odd element counts put the per-rank pieces of all-gather / reduce-scatter at odd byte offsets, skewed pointers
    do the same to every kind: the data path then reads its sources as shifted packs (two aligned loads and a
    funnel shift, the upper pack by warp shuffle) and must give exactly the aligned result."""
    _loopback_case(nv, kind, 4, count, dt, root=1, iters=1, skew=skew, blocks=4)


@pytest.mark.parametrize("kind", ["allreduce", "allgather", "reducescatter", "broadcast"])
@pytest.mark.parametrize("heap", [True, False])
def test_loopback_on_the_shared_memory_heap(nv, kind, heap, monkeypatch):
    """GPUs of one host that may not map one another's memory (here: NCCL_P2P_DISABLE=1, the reference's knob) select
    the second transport together: a symmetric heap in registered host shared memory.  The same daemon kernel and
    schedules then run with every flag and every peer access going through host memory; buffers outside the heap are
    staged into it as on the first transport."""
    monkeypatch.setenv("NCCL_P2P_DISABLE", "1")
    _loopback_case(nv, kind, 3, 70001, "FLOAT32", root=2, iters=2, blocks=2, heap=heap, transport="shm")


def test_shared_memory_heap_can_be_refused(nv, monkeypatch):
    """NCCL_SHM_DISABLE=1 on top leaves the third transport: host-staged collectives over the network transport."""
    monkeypatch.setenv("NCCL_P2P_DISABLE", "1")
    monkeypatch.setenv("NCCL_SHM_DISABLE", "1")
    comms = nv.Comm.init_loopback(2, 0)
    assert [c.transport() for c in comms] == ["net", "net"]
    for c in comms:
        c.destroy()


def test_loopback_eight_ranks_large(nv):
    _loopback_case(nv, "allreduce", 8, (8 << 20) + 24, "BFLOAT16", iters=1, blocks=8)


def test_fused_scale_cast_gradient_path(nv):
    _loopback_case(nv, "allreduce", 4, 1 << 20, "BFLOAT16", out_name="FLOAT32", scale=0.25)
    _loopback_case(nv, "allreduce", 4, 1 << 20, "FLOAT32", out_name="BFLOAT16", scale=0.25)


@pytest.mark.parametrize("kind", ["allreduce", "allgather", "reducescatter", "broadcast", "reduce"])
def test_in_place_and_unregistered_buffers(nv, kind):
    _loopback_case(nv, kind, 4, 30011, "FLOAT32", in_place=True, root=2, iters=1)
    _loopback_case(nv, kind, 4, 30011, "FLOAT32", heap=False, root=1, iters=1)


def test_disordered_issue_on_device(nv):
    """Four ranks, 24 collectives, every rank its own order, five rounds: all complete and
    the device really did park and resume collectives."""
    torch.cuda.set_device(0)
    nranks, ncolls, iters = 4, 24, 5
    rng = random.Random(3)
    kinds = [rng.choice([nv.ALLREDUCE, nv.ALLGATHER, nv.REDUCESCATTER, nv.BROADCAST]) for _ in range(ncolls)]
    counts = [int(2 ** rng.uniform(10, 20)) for _ in range(ncolls)]
    os.environ["DFCCL_DAEMON_BLOCKS"] = "8"
    comms = nv.Comm.init_loopback(nranks, 0)
    stats = {}

    def body(r):
        torch.cuda.set_device(0)
        c = comms[r]
        ctx = nv.RankCtx(r, 0)
        bufs = []
        for i in range(ncolls):
            ctx.prepare(i, c, kinds[i], counts[i], nv.BFLOAT16, root=i % nranks)
            sn = counts[i] * (nranks if kinds[i] == nv.REDUCESCATTER else 1)
            rn = counts[i] * (nranks if kinds[i] == nv.ALLGATHER else 1)
            sp, rp = c.alloc(sn * 2), c.alloc(rn * 2)
            bufs.append((sp, rp, _t(sp, sn, torch.bfloat16), _t(rp, rn, torch.bfloat16)))
        ctx.finalize()
        orng = random.Random(50 + r)
        for it in range(iters):
            for i in range(ncolls):
                bufs[i][2].fill_(float((r + 1) * ((i % 5) + 1)))
            torch.cuda.current_stream().synchronize()
            order = list(range(ncolls))
            orng.shuffle(order)
            for i in order:
                ctx.run(i, bufs[i][0], bufs[i][1])
            assert ctx.wait_all(120000) == nv.SUCCESS
            for i in range(ncolls):
                vals = [float((q + 1) * ((i % 5) + 1)) for q in range(nranks)]
                out = bufs[i][3].float()
                if kinds[i] in (nv.ALLREDUCE, nv.REDUCESCATTER):
                    assert bool((out == sum(vals)).all()), (i, out[:4], sum(vals))
                elif kinds[i] == nv.ALLGATHER:
                    assert bool((out.view(nranks, -1) == torch.tensor(vals, device="cuda:0")[:, None]).all())
                else:
                    assert bool((out == vals[i % nranks]).all())
        time.sleep(0.05)                           # device counters are folded in when the daemon parks
        stats[r] = ctx.stats()
        ctx.destroy()

    try:
        run_ranks(nranks, body, timeout=300)
    finally:
        os.environ.pop("DFCCL_DAEMON_BLOCKS", None)
    for c in comms:
        c.destroy()
    tot = {k: sum(s[k] for s in stats.values()) for k in stats[0]}
    assert tot["cqesDelivered"] == nranks * ncolls * iters
    assert tot["ctxSwitches"] > 0
    print("disordered stats", tot)


def test_device_wait_runs_out_with_a_status_not_a_hang(nv):
    """A flag nobody sets: rank 1 never submits.  The device wait gives up after the
    limit, the collective reports a timeout and the context (and the GPU) stay usable."""
    torch.cuda.set_device(0)
    os.environ["DFCCL_WAIT_TIMEOUT_MS"] = "500"
    os.environ["DFCCL_DAEMON_BLOCKS"] = "2"
    comms = nv.Comm.init_loopback(2, 0)
    out = {}
    gate = threading.Event()

    def body(r):
        torch.cuda.set_device(0)
        ctx = nv.RankCtx(r, 0)
        ctx.prepare(0, comms[r], nv.ALLREDUCE, 1024, nv.FLOAT32)
        ctx.finalize()
        p = comms[r].alloc(4096)
        if r == 0:
            t0 = time.time()
            ctx.run(0, p, p)
            out["rc"] = ctx.wait(0, 30000)
            out["dt"] = time.time() - t0
            gate.set()
        else:
            gate.wait(60)
        ctx.destroy()

    try:
        run_ranks(2, body, timeout=120)
    finally:
        os.environ.pop("DFCCL_WAIT_TIMEOUT_MS", None)
        os.environ.pop("DFCCL_DAEMON_BLOCKS", None)
    for c in comms:
        c.destroy()
    assert out["rc"] == nv.TIMEOUT and out["dt"] < 20
    x = torch.ones(1024, device="cuda:0")
    assert float(x.sum()) == 1024.0          # the context still works


def test_stream_ordered_submit_and_wait(nv):
    """No host thread between producer kernel, collective and consumer kernel: the submit is
    released by a stream memory operation and the consumer stream waits on the device flag."""
    torch.cuda.set_device(0)
    (c,) = nv.Comm.init_loopback(1, 0)
    ctx = nv.RankCtx(0, 0)
    n = 1 << 20
    ctx.prepare(0, c, nv.ALLREDUCE, n, nv.FLOAT32, scale=3.0)
    ctx.finalize()
    p = c.alloc(4 * n)
    q = c.alloc(4 * n)
    a, b = _t(p, n, torch.float32), _t(q, n, torch.float32)
    s = torch.cuda.Stream()
    for it in range(5):
        with torch.cuda.stream(s):
            a.fill_(float(it + 1))                      # producer kernel
            ctx.run_on_stream(0, p, q, s.cuda_stream)   # starts only after the fill
            ctx.stream_wait(0, s.cuda_stream)           # consumer below starts only after completion
            total = b.sum()
        s.synchronize()
        assert float(total) == 3.0 * (it + 1) * n
        assert ctx.wait(0, 10000) == nv.SUCCESS
    st = ctx.stats()
    assert st["sqesSubmitted"] == 5
    ctx.destroy()
    c.destroy()


@pytest.mark.parametrize("ptype", ["BFLOAT16", "FLOAT32"])
@pytest.mark.parametrize("n", [4096, 1000003])
def test_fused_optimizer_kernels_match_pytorch(nv, ptype, n):
    """dfcclFusedSgdStep and dfcclFusedAdamWStep against the same updates written in PyTorch fp32."""
    import ctypes as C
    torch.cuda.set_device(0)
    L = nv.lib()
    pt = TORCH_OF[ptype]
    g = torch.Generator(device="cuda").manual_seed(3)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def ptr(t):
        return C.c_void_p(t.data_ptr())

    # SGD with momentum and weight decay, two steps (the first one initialises the momentum)
    w = torch.randn(n, device="cuda", generator=g)
    m = torch.empty(n, device="cuda")
    p = torch.empty(n, device="cuda", dtype=pt)
    rw, rm = w.clone(), torch.zeros(n, device="cuda")
    for step in range(2):
        grad = torch.randn(n, device="cuda", generator=g)
        nv.check(L.dfcclFusedSgdStep(ptr(w), ptr(grad), ptr(m), ptr(p), n, getattr(nv, ptype), 0.1, 0.9, 1e-2, 1 if step == 0 else 0, st))
        gg = grad + 1e-2 * rw
        rm = gg if step == 0 else 0.9 * rm + gg
        rw = rw - 0.1 * rm
        torch.cuda.synchronize()
        torch.testing.assert_close(w, rw, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(p.float(), w.to(pt).float(), rtol=0, atol=0)
    # AdamW, three steps
    w = torch.randn(n, device="cuda", generator=g)
    m1, m2 = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    rw, r1, r2 = w.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    for t in range(1, 4):
        grad = torch.randn(n, device="cuda", generator=g)
        nv.check(L.dfcclFusedAdamWStep(ptr(w), ptr(grad), ptr(m1), ptr(m2), ptr(p), n, getattr(nv, ptype), lr, b1, b2, eps, wd, t, st))
        r1 = b1 * r1 + (1 - b1) * grad
        r2 = b2 * r2 + (1 - b2) * grad * grad
        rw = rw * (1 - lr * wd) - (lr / (1 - b1 ** t)) * r1 / (r2.sqrt() / (1 - b2 ** t) ** 0.5 + eps)
        torch.cuda.synchronize()
        torch.testing.assert_close(w, rw, rtol=2e-5, atol=1e-6)
        torch.testing.assert_close(p.float(), w.to(pt).float(), rtol=0, atol=0)
