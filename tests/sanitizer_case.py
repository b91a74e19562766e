"""Scenario run under a sanitizer build of the library (see test_sanitizers.py): three ranks on the host
backend, several registered collectives submitted in different orders per rank, the stream-ordered
entry points, and the network path - the host twin of the device code, the runtime threads (poller,
observer, network workers) and the queues all take part."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import numpy as np  # noqa: E402

from dfccl_b200 import native as nv  # noqa: E402
from helpers import run_ranks  # noqa: E402


def daemon_case(world):
    comms = nv.Comm.init_loopback(world)

    def body(r):
        ctx = nv.RankCtx(r)
        kinds = [nv.ALLREDUCE, nv.ALLGATHER, nv.REDUCESCATTER, nv.BROADCAST]
        n = 4096
        for i, k in enumerate(kinds):
            ctx.prepare(i, comms[r], k, n, nv.FLOAT32, root=1)
        ctx.finalize()
        a = [np.full(n * (world if k == nv.REDUCESCATTER else 1), r + 1.0, np.float32) for k in kinds]
        b = [np.zeros(n * (world if k == nv.ALLGATHER else 1), np.float32) for k in kinds]
        for it in range(3):
            order = list(range(len(kinds)))
            if r % 2:
                order.reverse()
            for i in order:
                ctx.run(i, a[i].ctypes.data, b[i].ctypes.data)
            assert ctx.wait_all(120000) == nv.SUCCESS
        tot = world * (world + 1) / 2
        assert float(b[0][0]) == tot and float(b[2][-1]) == tot and float(b[3][5]) == 2.0
        assert [float(b[1][j * n]) for j in range(world)] == [j + 1.0 for j in range(world)]
        x = np.full(1000, r + 1.0, np.float32)
        nv.check(nv.lib().ncclAllReduce(x.ctypes.data, x.ctypes.data, 1000, nv.FLOAT32, nv.SUM, comms[r].handle, None))
        assert float(x[7]) == tot
        ctx.destroy()

    run_ranks(world, body, timeout=600)
    for c in comms:
        c.destroy()


if __name__ == "__main__":
    nv.set_backend("host")
    daemon_case(3)
    os.environ["DFCCL_FORCE_NET"] = "1"
    daemon_case(2)
    print("CASE OK")
