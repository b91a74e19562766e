"""Collective sweep: latency and bus bandwidth of the daemon engine (and of the
stream-ordered kernels) against NCCL as shipped with PyTorch, same buffers, same sizes.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m dfccl_b200.benchmarks.coll_sweep \\
        --kinds allreduce,allgather,reducescatter --dtypes bf16,fp32 --min-bytes 1024 --max-bytes 1073741824 --out sweep.json

Every number is device time (CUDA events on the launching stream, warm-up first, max over
ranks).  Inputs are uniform(-1, 1) from a seed.  busBW follows the usual convention:
all-reduce algBW x 2(n-1)/n, all-gather / reduce-scatter algBW x (n-1)/n with algBW over the
full (n x per-rank) buffer.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from dfccl_b200 import native as nv
from dfccl_b200.parallel import init_distributed
from dfccl_b200.utils import tensor_from_ptr

KIND = {"allreduce": nv.ALLREDUCE, "allgather": nv.ALLGATHER, "reducescatter": nv.REDUCESCATTER,
        "broadcast": nv.BROADCAST, "reduce": nv.REDUCE}
DT = {"bf16": (torch.bfloat16, nv.BFLOAT16), "fp32": (torch.float32, nv.FLOAT32)}


def bus_factor(kind: str, n: int) -> float:
    if n == 1:
        return 1.0
    if kind == "allreduce":
        return 2.0 * (n - 1) / n
    if kind in ("allgather", "reducescatter"):
        return (n - 1) / n
    return 1.0


def time_loop(fn, iters: int, warm: int, world: int) -> float:
    """Mean device microseconds per call of fn, max over ranks."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    import time
    e0.record()
    h0 = time.perf_counter()
    for _ in range(iters):
        fn()
    time_loop.host_us = (time.perf_counter() - h0) * 1e6 / iters     # host time to enqueue one call
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    if world > 1:
        t = torch.tensor([us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t)
    return us


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kinds", default="allreduce,allgather,reducescatter")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--min-bytes", dest="min", type=int, default=1024)
    ap.add_argument("--max-bytes", dest="max", type=int, default=1 << 30)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--algo", default="auto", choices=["auto", "oneshot", "twoshot", "nvls"])
    ap.add_argument("--nvls-from", dest="nvls_from", type=int, default=-1,
                    help="with --algo auto: message sizes from this many bytes up take the multimem schedule, operands in the "
                         "multicast arena (-1 = 512 KiB, the first size past the push schedule, on 4 or more ranks, off below; 0 = off)")
    ap.add_argument("--blocks", type=int, default=0, help="daemon blocks per rank (0 = default)")
    ap.add_argument("--ids", type=int, default=4, help="registrations per case, used round-robin so that the host can enqueue ahead")
    ap.add_argument("--skip-nccl", action="store_true")
    ap.add_argument("--skip-stream-api", action="store_true")
    ap.add_argument("--trace", default="", help="write the device trace of rank 0 (Chrome trace JSON) here")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)

    os.environ.setdefault("DFCCL_WAIT_TIMEOUT_MS", "30000")
    if a.trace:
        os.environ["DFCCL_TRACE"] = "1"
    d = init_distributed()
    world, rank, dev = d.world, d.rank, d.device
    L = nv.lib()
    algo = {"auto": nv.ALGO_AUTO, "oneshot": nv.ALGO_ONESHOT, "twoshot": nv.ALGO_TWOSHOT, "nvls": nv.ALGO_NVLS}[a.algo]
    sizes = []
    s = a.min
    while s <= a.max:
        sizes.append(s)
        s *= a.factor
    cases = [(k, dt, sz) for k in a.kinds.split(",") for dt in a.dtypes.split(",") for sz in sizes]

    # one registration per case, one context for all of them
    ctx = nv.RankCtx(rank, d.local_rank)
    if a.blocks:
        ctx.set_daemon_geometry(a.blocks, 0)
    bufs = {}
    max_bytes = max(sizes)
    nvls = False
    nvls_from = a.nvls_from if a.nvls_from >= 0 else ((512 << 10) if world >= 4 else 0)
    if a.algo == "nvls":
        nvls_from = 1
    if nvls_from and world > 1:
        # operands live in the switch-multicast arena, so the schedule works on them in place
        os.environ.setdefault("DFCCL_NVLS_MIN_BYTES", "4096" if a.algo == "nvls" else str(nvls_from))
        nvls = d.comm.nvls_init(2 * max_bytes + (96 << 20))
        if rank == 0:
            print(json.dumps({"nvls_available": bool(nvls), "nvls_from_bytes": nvls_from}), flush=True)
    if nvls:
        send_p, recv_p = d.comm.nvls_alloc(max_bytes + 256), d.comm.nvls_alloc(max_bytes + 256)
    else:
        send_p, recv_p = d.comm.alloc(max_bytes + 256), d.comm.alloc(max_bytes + 256)
    for cid, (k, dt, sz) in enumerate(cases):
        tdt, ndt = DT[dt]
        es = torch.empty((), dtype=tdt).element_size()
        total = sz // es                              # elements of the "message" as NCCL tests count it
        count = total // world if k in ("allgather", "reducescatter") else total
        if count == 0:
            continue
        big = nvls and sz >= nvls_from and (count * es) % 16 == 0 and k in ("allreduce", "allgather", "reducescatter")
        for j in range(a.ids):
            ctx.prepare(cid * a.ids + j, d.comm, KIND[k], count, ndt,
                        algo=nv.ALGO_NVLS if big else (algo if k == "allreduce" and a.algo != "nvls" else nv.ALGO_AUTO), arena_buffers=big)
        bufs[cid] = (count, total, big)
    ctx.finalize()
    stream = torch.cuda.current_stream()
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    rows = []
    for cid, (k, dt, sz) in enumerate(cases):
        if cid not in bufs:
            continue
        tdt, ndt = DT[dt]
        count, total, big = bufs[cid]
        sn = count * world if k == "reducescatter" else count
        rn = count * world if k == "allgather" else count
        sv = tensor_from_ptr(send_p, (sn,), tdt, dev)
        rv = tensor_from_ptr(recv_p, (rn,), tdt, dev)
        sv.copy_((torch.rand(min(sn, 1 << 22), generator=g) * 2 - 1).to(tdt).repeat((sn + (1 << 22) - 1) // (1 << 22))[:sn])
        torch.cuda.synchronize()
        iters = a.iters if sz <= (64 << 20) else max(3, a.iters // 4)

        turn = [0]

        def daemon_op():
            i = cid * a.ids + turn[0] % a.ids
            turn[0] += 1
            ctx.run_on_stream(i, send_p, recv_p, stream.cuda_stream)
            ctx.stream_wait(i, stream.cuda_stream)

        def daemon_window():
            # the way a trainer uses the daemon: several registered collectives released back to back, waited for
            # together - the daemon works on all of them at once instead of one round trip at a time
            base = cid * a.ids
            for j in range(a.ids):
                ctx.run_on_stream(base + j, send_p, recv_p, stream.cuda_stream)
            for j in range(a.ids):
                ctx.stream_wait(base + j, stream.cuda_stream)

        row = {"kind": k, "dtype": dt, "bytes": sz, "n": world, "daemon_schedule": "multimem" if big else "peer"}
        us = time_loop(daemon_op, iters, a.warmup, world)
        assert ctx.wait_all(60000) == nv.SUCCESS
        row["daemon_us"] = us
        row["daemon_host_enqueue_us"] = time_loop.host_us
        if a.ids > 1 and sz <= (16 << 20):
            usw = time_loop(daemon_window, max(3, iters // a.ids), max(2, a.warmup // 2), world)
            assert ctx.wait_all(60000) == nv.SUCCESS
            row["daemon_window_us_per_op"] = usw / a.ids
        row["daemon_busbw_gbs"] = sz / us / 1e3 * bus_factor(k, world)
        # correctness spot check against torch on the same data
        if k == "allreduce" and world > 1:
            ref = sv.float().clone()
            dist.all_reduce(ref)
            err = float((rv.float() - ref).abs().max() / (ref.abs().max() + 1e-6))
            row["max_rel_err"] = err
        elif k == "allgather" and world > 1:                  # a copy: must be exact
            ref = torch.empty(rn, dtype=tdt, device=dev)
            dist.all_gather_into_tensor(ref, sv.clone())
            row["max_rel_err"] = float((rv.float() - ref.float()).abs().max())
            del ref
        elif k == "reducescatter" and world > 1:              # fp32 reference of the same sum
            ref = torch.empty(rn, dtype=torch.float32, device=dev)
            dist.reduce_scatter_tensor(ref, sv.float())
            row["max_rel_err"] = float((rv.float() - ref).abs().max() / (ref.abs().max() + 1e-6))
            del ref
        if not a.skip_stream_api and k in ("allreduce", "allgather", "reducescatter"):
            fn = {"allreduce": lambda: nv.check(L.ncclAllReduce(send_p, recv_p, count, ndt, nv.SUM, d.comm.handle, stream.cuda_stream)),
                  "allgather": lambda: nv.check(L.ncclAllGather(send_p, recv_p, count, ndt, d.comm.handle, stream.cuda_stream)),
                  "reducescatter": lambda: nv.check(L.ncclReduceScatter(send_p, recv_p, count, ndt, nv.SUM, d.comm.handle, stream.cuda_stream))}[k]
            us2 = time_loop(fn, iters, a.warmup, world)
            row["stream_us"] = us2
            row["stream_busbw_gbs"] = sz / us2 / 1e3 * bus_factor(k, world)
        if not a.skip_nccl and world > 1:
            tin = sv.clone()
            tout = torch.empty_like(rv)
            fn = {"allreduce": lambda: dist.all_reduce(tin),
                  "allgather": lambda: dist.all_gather_into_tensor(tout, tin),
                  "reducescatter": lambda: dist.reduce_scatter_tensor(tout, tin),
                  "broadcast": lambda: dist.broadcast(tin, 0),
                  "reduce": lambda: dist.reduce(tin, 0)}[k]
            us3 = time_loop(fn, iters, a.warmup, world)
            row["nccl_us"] = us3
            row["nccl_busbw_gbs"] = sz / us3 / 1e3 * bus_factor(k, world)
            del tin, tout
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    st = ctx.stats()
    if a.trace:
        import time
        time.sleep(0.05)
        ctx.trace_dump(a.trace + (f".rank{rank}" if rank else ""))
    ctx.destroy()
    if rank == 0 and a.out:
        with open(a.out, "w") as fh:
            json.dump({"world": world, "rows": rows, "daemon_stats": st, "algo": a.algo, "blocks": a.blocks}, fh, indent=1)
    d.destroy()


if __name__ == "__main__":
    main()
