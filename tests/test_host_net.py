"""Network path: communicators forced through the host-staged ring algorithms over the built-in TCP
transport (DFCCL_FORCE_NET=1 makes same-host ranks behave as if they sat on different hosts), the
register-then-submit interface on top of it with per-rank disordered submission, and the plugin loader."""
import os
import random
import subprocess
import sys
import threading

import numpy as np
import pytest

from helpers import bf16_bits_to_f32, f32_to_bf16_bits, np_dtype, run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture
def net_backend(host_backend, monkeypatch):
    monkeypatch.setenv("DFCCL_FORCE_NET", "1")
    return host_backend


def _data(nv, dt, n, r, seed=0):
    x = np.random.default_rng(seed * 100 + r).integers(-4, 5, n).astype(np.float32)
    if dt == nv.BFLOAT16:
        return f32_to_bf16_bits(x)
    return x.astype(np_dtype(nv, dt))


def _f(nv, dt, a):
    return bf16_bits_to_f32(a).astype(np.float64) if dt == nv.BFLOAT16 else a.astype(np.float64)


@pytest.mark.parametrize("world", [2, 3, 4])
def test_stream_interface_over_the_network_path(net_backend, world):
    nv = net_backend
    comms = nv.Comm.init_loopback(world)
    n = 1000 * world + 7 * world                      # not a multiple of anything convenient per chunk
    ins = [_data(nv, nv.FLOAT32, n, r) for r in range(world)]
    total = sum(a.astype(np.float64) for a in ins)
    out = {}

    def body(r):
        c, L = comms[r], nv.lib()
        res = {}
        a, b = ins[r].copy(), np.zeros(n, np.float32)
        nv.check(L.ncclAllReduce(a.ctypes.data, b.ctypes.data, n, nv.FLOAT32, nv.SUM, c.handle, None))
        res["ar"] = b.copy()
        nv.check(L.ncclAllReduce(a.ctypes.data, a.ctypes.data, n, nv.FLOAT32, nv.AVG, c.handle, None))   # in place, averaged
        res["avg"] = a.copy()
        per = n // world
        g = np.zeros(per * world, np.float32)
        part = ins[r][:per].copy()
        nv.check(L.ncclAllGather(part.ctypes.data, g.ctypes.data, per, nv.FLOAT32, c.handle, None))
        res["ag"] = g
        s = np.zeros(per, np.float32)
        blocks = ins[r][:per * world].copy()
        nv.check(L.ncclReduceScatter(blocks.ctypes.data, s.ctypes.data, per, nv.FLOAT32, nv.SUM, c.handle, None))
        res["rs"] = s
        bc = ins[r].copy()
        nv.check(L.ncclBroadcast(bc.ctypes.data, bc.ctypes.data, n, nv.FLOAT32, 1 % world, c.handle, None))
        res["bc"] = bc
        rd = np.zeros(n, np.float32)
        mine = ins[r].copy()
        nv.check(L.ncclReduce(mine.ctypes.data, rd.ctypes.data, n, nv.FLOAT32, nv.MAX, world - 1, c.handle, None))
        res["rd"] = rd
        out[r] = res

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    per = n // world
    for r in range(world):
        np.testing.assert_allclose(out[r]["ar"], total, rtol=1e-6)
        np.testing.assert_allclose(out[r]["avg"], total / world, rtol=1e-6)
        np.testing.assert_array_equal(out[r]["ag"], np.concatenate([ins[j][:per] for j in range(world)]))
        np.testing.assert_allclose(out[r]["rs"], total[r * per:(r + 1) * per], rtol=1e-6)
        np.testing.assert_array_equal(out[r]["bc"], ins[1 % world])
    np.testing.assert_array_equal(out[world - 1]["rd"], np.max(np.stack(ins), 0))


def test_daemon_interface_over_the_network_path_disordered(net_backend):
    """Eight registered collectives with fused scale and cast, submitted by every rank in its own order."""
    nv = net_backend
    world, ncoll, iters = 3, 8, 3
    comms = nv.Comm.init_loopback(world)
    counts = [257 * (i + 1) for i in range(ncoll)]
    ins = [[_data(nv, nv.BFLOAT16, counts[i], r, seed=i) for i in range(ncoll)] for r in range(world)]
    got = {}

    def body(r):
        c = comms[r]
        ctx = nv.RankCtx(r)
        for i in range(ncoll):
            ctx.prepare(i, c, nv.ALLREDUCE, counts[i], nv.BFLOAT16, out_dtype=nv.FLOAT32, op=nv.SUM, scale=0.5)
        ctx.finalize()
        outs = [np.zeros(counts[i], np.float32) for i in range(ncoll)]
        fired = []
        rng = random.Random(17 + r)
        for _ in range(iters):
            order = list(range(ncoll))
            rng.shuffle(order)
            for i in order:
                ctx.run(i, ins[r][i].ctypes.data, outs[i].ctypes.data, callback=lambda cid: fired.append(cid))
            assert ctx.wait_all(60000) == nv.SUCCESS
        st = ctx.stats()
        ctx.destroy()
        assert st["cqesDelivered"] == ncoll * iters and len(fired) == ncoll * iters
        got[r] = outs

    run_ranks(world, body, timeout=180)
    for c in comms:
        c.destroy()
    for i in range(ncoll):
        exp = 0.5 * sum(_f(nv, nv.BFLOAT16, ins[r][i]) for r in range(world))
        for r in range(world):
            np.testing.assert_allclose(got[r][i], exp, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("world", [2, 3])
def test_send_recv_over_the_network_path(net_backend, world):
    """Members that cannot map one another's memory exchange send / recv as messages over the communicator's
    out-of-band connections.  Every rank sends to every other rank before it receives (a pattern that deadlocks an
    implementation whose sends wait for the matching receive), two messages per pair to check their order."""
    nv = net_backend
    comms = nv.Comm.init_loopback(world)
    got = {}

    def body(r):
        c, L = comms[r], nv.lib()
        outs = {p: [np.full(5000 + p, 100.0 * r + p, np.float32), np.full(3, -1.0 * r, np.float32)] for p in range(world) if p != r}
        ins = {p: [np.zeros(5000 + r, np.float32), np.zeros(3, np.float32)] for p in range(world) if p != r}
        nv.check(L.ncclGroupStart())
        for p, (a, b) in outs.items():
            nv.check(L.ncclSend(a.ctypes.data, a.size, nv.FLOAT32, p, c.handle, None))
            nv.check(L.ncclSend(b.ctypes.data, b.size, nv.FLOAT32, p, c.handle, None))
        for p, (a, b) in ins.items():
            nv.check(L.ncclRecv(a.ctypes.data, a.size, nv.FLOAT32, p, c.handle, None))
            nv.check(L.ncclRecv(b.ctypes.data, b.size, nv.FLOAT32, p, c.handle, None))
        nv.check(L.ncclGroupEnd())
        got[r] = ins

    run_ranks(world, body, timeout=120)
    for c in comms:
        c.destroy()
    for r in range(world):
        for p, (a, b) in got[r].items():
            assert np.all(a == 100.0 * p + r) and np.all(b == -1.0 * p), (r, p)


def test_dummy_plugin_falls_back_to_sockets(tmp_path):
    """A plugin that loads but offers no device must leave the built-in transport in charge."""
    so = tmp_path / "libdfccl-net.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-I", os.path.join(ROOT, "dfccl_b200", "csrc", "include"),
                           os.path.join(ROOT, "dfccl_b200", "csrc", "ext-net", "dummy", "plugin.c"), "-o", str(so)])
    code = f"""
import sys, threading
sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {os.path.join(ROOT, 'tests')!r})
import numpy as np
from dfccl_b200 import native as nv
nv.set_backend("host")
comms = nv.Comm.init_loopback(2)
res = {{}}
def body(r):
    a = np.full(100, r + 1.0, np.float32)
    nv.check(nv.lib().ncclAllReduce(a.ctypes.data, a.ctypes.data, 100, nv.FLOAT32, nv.SUM, comms[r].handle, None))
    res[r] = float(a[0])
ts = [threading.Thread(target=body, args=(r,)) for r in range(2)]
[t.start() for t in ts]; [t.join() for t in ts]
assert res == {{0: 3.0, 1: 3.0}}, res
print("OK")
"""
    env = dict(os.environ, DFCCL_FORCE_NET="1", DFCCL_NET_PLUGIN=str(so), DFCCL_DEBUG="INFO", DFCCL_DEBUG_SUBSYS="NET,INIT")
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "OK" in p.stdout, p.stdout + p.stderr
    assert "offers no device" in (p.stdout + p.stderr)


def test_transport_selection_falls_back_when_peer_memory_is_off(host_backend, monkeypatch):
    """No FORCE_NET: the members merely cannot (are told not to) map one another's memory - NCCL_P2P_DISABLE=1, the
    reference's knob.  The communicator is still created, picks the host-staged path by itself (every member reaches
    the same verdict) and computes the right result."""
    monkeypatch.delenv("DFCCL_FORCE_NET", raising=False)
    monkeypatch.setenv("NCCL_P2P_DISABLE", "1")
    nv = host_backend
    world, n = 3, 5003
    comms = nv.Comm.init_loopback(world)
    ins = [_data(nv, nv.FLOAT32, n, r, seed=3) for r in range(world)]
    total = sum(a.astype(np.float64) for a in ins)

    def body(r):
        a, b = ins[r].copy(), np.zeros(n, np.float32)
        nv.check(nv.lib().ncclAllReduce(a.ctypes.data, b.ctypes.data, n, nv.FLOAT32, nv.SUM, comms[r].handle, None))
        np.testing.assert_allclose(b.astype(np.float64), total)
        assert not comms[r].peer_base((r + 1) % world)          # no member maps another member's heap in this mode

    run_ranks(world, body, timeout=120)
    for c in comms:
        c.destroy()
