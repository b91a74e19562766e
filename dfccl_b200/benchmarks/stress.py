"""Disordered-issue stress: every rank registers the same set of collectives (mixed kinds, sizes
log-uniform between --min-bytes and --max-bytes, bf16) and submits all of them each iteration in
its OWN seeded random order.  A stream-ordered library deadlocks on such a workload; here every
iteration must complete.  Results are verified against closed-form expectations.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m dfccl_b200.benchmarks.stress \\
        --colls 64 --iters 1000 --out stress.json
"""
from __future__ import annotations

import argparse
import json
import math
import os
import random
import time

import torch

from dfccl_b200 import native as nv
from dfccl_b200.parallel import init_distributed
from dfccl_b200.utils import tensor_from_ptr


def inorder_verdict(colls: int, iters: int, world: int, seed: int) -> dict:
    """What a library that executes each rank's collectives strictly in launch order would do with the very
    orders this run uses (they are functions of the seed and the rank): per iteration, build the wait-for
    graph of the in-order model and look for a cycle.  Pure host arithmetic, nothing is launched."""
    from dfccl_b200.simulator.waitgraph import build_fifo_wait_for_graph, find_cycle
    rngs = [random.Random(seed * 31 + r) for r in range(world)]
    dead, first = 0, None
    for it in range(iters):
        orders = {}
        for r in range(world):
            o = list(range(colls))
            rngs[r].shuffle(o)
            orders[r] = o
        cyc = find_cycle(build_fifo_wait_for_graph(orders))
        if cyc is not None:
            dead += 1
            if first is None:
                first = {"iteration": it, "cycle_length": len(cyc)}
    return {"iterations_with_incompatible_orders": dead, "of": iters, "first": first}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--colls", type=int, default=64)
    ap.add_argument("--iters", type=int, default=1000)
    ap.add_argument("--min-bytes", dest="min_bytes", type=int, default=4 << 10)
    ap.add_argument("--max-bytes", dest="max_bytes", type=int, default=64 << 20)
    ap.add_argument("--verify-every", type=int, default=50)
    ap.add_argument("--seed", type=int, default=2024)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--out", default="")
    ap.add_argument("--trace", default="", help="write the device trace (Chrome trace JSON) here, one file per rank")
    a = ap.parse_args(argv)
    if a.trace:
        os.environ["DFCCL_TRACE"] = "1"
        os.environ.setdefault("DFCCL_TRACE_EVENTS", str(1 << 18))

    rng = random.Random(a.seed)                       # the SAME set of collectives on every rank
    kinds = [rng.choice([nv.ALLREDUCE, nv.ALLGATHER, nv.REDUCESCATTER, nv.BROADCAST]) for _ in range(a.colls)]
    sizes = [int(math.exp(rng.uniform(math.log(a.min_bytes), math.log(a.max_bytes)))) for _ in range(a.colls)]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    counts, total = [], 0
    for k, sz in zip(kinds, sizes):
        n = max(8, sz // 2)                           # bf16 elements of the "message"
        per = max(8, n // world) if k in (nv.ALLGATHER, nv.REDUCESCATTER) else n
        counts.append(per)
        total += 2 * (per * world if k in (nv.ALLGATHER, nv.REDUCESCATTER) else per) * 2 + 4096
    os.environ.setdefault("DFCCL_HEAP_BYTES", str(total + (768 << 20)))      # buffers + flag words, push slots (up to 4 MB per small collective), staging
    os.environ.setdefault("DFCCL_WAIT_TIMEOUT_MS", "60000")
    d = init_distributed()
    rank, dev = d.rank, d.device
    ctx = nv.RankCtx(rank, d.local_rank)
    if a.blocks:
        ctx.set_daemon_geometry(a.blocks, 0)
    bufs = []
    for i in range(a.colls):
        ctx.prepare(i, d.comm, kinds[i], counts[i], nv.BFLOAT16, root=i % world)
        sn = counts[i] * (world if kinds[i] == nv.REDUCESCATTER else 1)
        rn = counts[i] * (world if kinds[i] == nv.ALLGATHER else 1)
        sp, rp = d.comm.alloc(sn * 2), d.comm.alloc(rn * 2)
        bufs.append((sp, rp, tensor_from_ptr(sp, (sn,), torch.bfloat16, dev), tensor_from_ptr(rp, (rn,), torch.bfloat16, dev)))
    ctx.finalize()
    order_rng = random.Random(a.seed * 31 + rank)     # a DIFFERENT order on every rank
    stream = torch.cuda.current_stream()
    for i in range(a.colls):
        bufs[i][2].fill_(float((rank % 4) + 1))       # small integers: sums are exact in bf16
    torch.cuda.synchronize()
    d.barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    done_iters, bad = 0, 0
    for it in range(a.iters):
        order = list(range(a.colls))
        order_rng.shuffle(order)
        for i in order:
            ctx.run_on_stream(i, bufs[i][0], bufs[i][1], stream.cuda_stream)
        for i in order:
            ctx.stream_wait(i, stream.cuda_stream)
        if (it + 1) % a.verify_every == 0 or it == a.iters - 1:
            torch.cuda.synchronize()
            vals = [float((q % 4) + 1) for q in range(world)]
            for i in range(a.colls):
                out = bufs[i][3].float()
                if kinds[i] in (nv.ALLREDUCE, nv.REDUCESCATTER):
                    ok = bool((out == sum(vals)).all())
                elif kinds[i] == nv.ALLGATHER:
                    ok = bool((out.view(world, -1) == torch.tensor(vals, device=dev)[:, None]).all())
                else:
                    ok = bool((out == vals[i % world]).all())
                bad += 0 if ok else 1
        done_iters += 1
    e1.record()
    torch.cuda.synchronize()
    rc = ctx.wait_all(120000)
    wall = time.perf_counter() - t0
    time.sleep(0.05)
    st = ctx.stats()
    res = torch.tensor([done_iters, bad, rc, st["ctxSwitches"], st["waitTimeouts"], st["dataYields"]], device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        allres = [torch.zeros_like(res) for _ in range(world)]
        dist.all_gather(allres, res)
    else:
        allres = [res]
    if a.trace:
        ctx.trace_dump(a.trace + (f".rank{rank}" if rank else ""))
    ctx.destroy()
    if rank == 0:
        out = {"world": world, "colls": a.colls, "iters_requested": a.iters,
               "iters_completed_min": int(min(float(r[0]) for r in allres)),
               "wrong_results": int(sum(float(r[1]) for r in allres)),
               "nonzero_status_ranks": int(sum(1 for r in allres if float(r[2]) != 0)),
               "ctx_switches_total": int(sum(float(r[3]) for r in allres)),
               "ctx_switches_per_iter_per_rank": sum(float(r[3]) for r in allres) / world / max(done_iters, 1),
               "data_yields_per_iter_per_rank": sum(float(r[5]) for r in allres) / world / max(done_iters, 1),
               "daemon_blocks": a.blocks or int(os.environ.get("DFCCL_DAEMON_BLOCKS", "32")),
               "wait_timeouts_total": int(sum(float(r[4]) for r in allres)),
               "bytes_min": a.min_bytes, "bytes_max": a.max_bytes, "dtype": "bf16",
               "device_ms_per_iter": e0.elapsed_time(e1) / max(done_iters, 1), "wall_s": wall,
               "collective_bytes_per_iter_per_rank": int(sum(sizes)),
               "hangs": 0 if min(float(r[0]) for r in allres) == a.iters else 1,
               # rank 0's daemon, summed over its blocks: scheduler passes and where their time went
               "rank0_scheduler": {k: st[k] for k in ("schedulerPasses", "nsTriggers", "nsWalk", "nsQueues", "daemonLaunches",
                                                       "ctxSaves", "ctxLoads", "waitPolls", "maxSwitchNs", "totalSwitchNs")},
               "inorder_library_model": inorder_verdict(a.colls, a.iters, world, a.seed)}
        print(json.dumps(out), flush=True)
        if a.out:
            json.dump(out, open(a.out, "w"), indent=1)
    d.destroy()


if __name__ == "__main__":
    main()
