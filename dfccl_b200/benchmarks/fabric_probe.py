"""Fabric probe: peer read / write bandwidth of this library's own copy kernels for every load
flavour, unroll and grid size, and the flag round-trip time between two GPUs.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m dfccl_b200.benchmarks.fabric_probe --out probe.json
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from dfccl_b200 import native as nv
from dfccl_b200.parallel import init_distributed

LOADS = {0: "ld.relaxed.sys", 1: "ld.volatile", 2: "ld.global.cg", 3: "plain ld", 4: "ld.global.nc"}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbytes", type=int, default=256)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    d = init_distributed()
    L = nv.lib()
    peer = (d.rank + 1) % d.world
    rows = []
    us = C.c_double()
    for direction in (0, 1):
        for kind in LOADS:
            for unroll in (1, 4, 8, 16):
                for blocks in (16, 32, 64, 148):
                    if direction == 1 and kind not in (0, 3):
                        continue
                    d.barrier()
                    nv.check(L.dfcclProbePeerCopy(d.comm.handle, peer, a.mbytes << 20, direction, kind, unroll, blocks, a.iters,
                                                  C.byref(us)), "dfcclProbePeerCopy")
                    row = {"dir": "read peer" if direction == 0 else "write peer", "load": LOADS[kind], "unroll": unroll,
                           "blocks": blocks, "us": us.value, "gbs": (a.mbytes << 20) / us.value / 1e3}
                    rows.append(row)
                    if d.rank == 0:
                        print(json.dumps(row), flush=True)
    rtt = None
    if d.world > 1:
        nv.check(L.dfcclProbeFlagRoundTrip(d.comm.handle, peer if d.world == 2 else (d.rank ^ 1), 1000, C.byref(us)))
        rtt = us.value
        if d.rank == 0:
            print(json.dumps({"flag_round_trip_us": rtt}), flush=True)
    if d.rank == 0 and a.out:
        json.dump({"world": d.world, "rows": rows, "flag_round_trip_us": rtt}, open(a.out, "w"), indent=1)
    d.destroy()


if __name__ == "__main__":
    main()
