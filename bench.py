#!/usr/bin/env python
"""Headline benchmark: ResNet-50 data-parallel training, bf16, batch 128 per GPU, synthetic
N(0,1) images and random labels, gradients all-reduced in 25 MB buckets through the daemon
(fused 1/N scale and bf16->fp32 cast, per-rank randomized bucket order), fused SGD.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the reference's own library

For N > 1 launch one rank per GPU with torchrun (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*
come from the environment).  Rank 0 prints one JSON line.  ``value`` is the device-timed
(CUDA events, max over ranks) throughput of K steps with inputs resident on the GPU;
``e2e`` repeats the K steps through the public API with a pinned-host -> device copy of
every step's batch and a device -> host read of every step's loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH_PER_GPU = 128
IMG = (3, 224, 224)
CLASSES = 1000
BUCKET_MB = 25.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="dfccl", choices=["dfccl", "reference"])
    ap.add_argument("--graph", type=int, default=1, help="capture forward+backward in a CUDA graph (this library's arm only)")
    ap.add_argument("--overlap", type=int, default=1, help="graphed step: release every gradient bucket from inside the captured backward pass")
    ap.add_argument("--daemon-blocks", type=int, default=int(os.environ.get("BENCH_DAEMON_BLOCKS", "8")),
                    help="thread blocks of the daemon kernel (SMs it holds while gradient buckets are in flight)")
    ap.add_argument("--sweep", type=int, default=1, help="after the training runs, time a few all-reduce sizes through the daemon (N > 1)")
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help=argparse.SUPPRESS)
    ap.add_argument("--model", default="resnet50", help=argparse.SUPPRESS)
    return ap.parse_args()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda" if dist.get_backend() == "nccl" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class Trainer:
    """One training step of the flagship workload on top of a gradient backend."""

    def __init__(self, args, dist_info, backend):
        self.dev = dist_info.device
        torch.manual_seed(1234)                       # same random-init weights on every rank
        if args.impl == "reference":                  # vanilla torchvision model: nothing of this repository on that arm
            from baseline.reference_backend import make_model
            self.net = make_model(self.dev, CLASSES, tiny=args.model != "resnet50")
        else:
            from dfccl_b200.models import resnet50, resnet_tiny, to_bf16_channels_last
            net = resnet50(CLASSES) if args.model == "resnet50" else resnet_tiny(CLASSES)
            self.net = to_bf16_channels_last(net.to(self.dev))
        self.crit = nn.CrossEntropyLoss()
        self.backend = backend
        backend.attach(self.net)
        self.batch = args.batch
        self.graphed = None
        self.use_graph = bool(args.graph) and args.impl == "dfccl"
        self.overlap = bool(args.overlap)

    def loss_fn(self, out, y):
        return self.crit(out.float(), y)

    def step(self, x, y):
        if self.use_graph:
            if self.graphed is None:
                from dfccl_b200.parallel import GraphedStep
                self.graphed = GraphedStep(self.net, self.loss_fn, self.backend.ddp, x, y, overlap=self.overlap)
            loss = self.graphed(x, y)
        else:
            loss = self.loss_fn(self.net(x), y)
            loss.backward()
        self.backend.finish_backward()
        self.backend.step()
        return loss


class DaemonBackend:
    name = "dfccl"

    def __init__(self, dist_info, daemon_blocks=4):
        self.d = dist_info
        self.ddp = None
        self.daemon_blocks = daemon_blocks

    def attach(self, net):
        from dfccl_b200.parallel import DaemonDDP
        self.ddp = DaemonDDP(net, self.d, bucket_mb=BUCKET_MB, lr=0.1, momentum=0.9, weight_decay=1e-4,
                             randomize_order=True, window=2, seed=17, daemon_blocks=self.daemon_blocks)

    def finish_backward(self):
        self.ddp.finish_backward()

    def step(self):
        self.ddp.step()

    def launches(self):
        st = self.ddp.stats()
        return st["daemonLaunches"] + self.ddp.launches

    def info(self):
        return {"buckets": len(self.ddp.buckets), "bucket_mb": BUCKET_MB, "daemon_blocks": self.daemon_blocks,
                "schedule": self.ddp.gradient_path(), "stats": self.ddp.stats()}

    def close(self):
        self.ddp.close()


def allreduce_sweep(d):
    """The other half of the headline metric: all-reduce latency and bus bandwidth through the daemon (register, then
    stream-ordered submit and wait, one call in flight), bf16, next to this library's stream-ordered kernel and to the
    NCCL that ships with PyTorch on the same buffers.  Device time (CUDA events), max over ranks."""
    import torch.distributed as dist
    from dfccl_b200 import native as nv
    from dfccl_b200.utils import tensor_from_ptr
    world, L = d.world, nv.lib()
    sizes = [1 << 10, 64 << 10, 1 << 20, 16 << 20, 256 << 20]
    ctx = nv.RankCtx(d.rank, d.local_rank)
    ctx.set_daemon_geometry(64, 0)
    nvls = bool(d.comm.nvls_init(0))
    if nvls:                                   # room left in the arena for both buffers?  (every rank sees the same numbers)
        _uc, _mc, total, used = d.comm.nvls_info()
        nvls = total - used >= 2 * max(sizes) + 4096
    send_p = d.comm.nvls_alloc(max(sizes)) if nvls else d.comm.alloc(max(sizes))
    recv_p = d.comm.nvls_alloc(max(sizes)) if nvls else d.comm.alloc(max(sizes))
    ids = 4
    for k, sz in enumerate(sizes):
        for j in range(ids):
            big = nvls and world >= 4 and sz >= (1 << 20)
            ctx.prepare(k * ids + j, d.comm, nv.ALLREDUCE, sz // 2, nv.BFLOAT16, algo=nv.ALGO_NVLS if big else nv.ALGO_AUTO, arena_buffers=big)
    ctx.finalize()
    stream = torch.cuda.current_stream()
    x = tensor_from_ptr(send_p, (max(sizes) // 2,), torch.bfloat16, d.device)
    x.uniform_(-1, 1)
    nccl_buf = x.clone()

    def timed(fn, iters, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) * 1e3 / iters, world)

    rows = []
    f = 2.0 * (world - 1) / world
    for k, sz in enumerate(sizes):
        turn = [0]

        def daemon_op():
            i = k * ids + turn[0] % ids
            turn[0] += 1
            ctx.run_on_stream(i, send_p, recv_p, stream.cuda_stream)
            ctx.stream_wait(i, stream.cuda_stream)
        iters = 20 if sz <= (16 << 20) else 5
        us_d = timed(daemon_op, iters)
        assert ctx.wait_all(60000) == nv.SUCCESS
        us_s = timed(lambda: nv.check(L.ncclAllReduce(send_p, recv_p, sz // 2, nv.BFLOAT16, nv.SUM, d.comm.handle, stream.cuda_stream)), iters)
        view = nccl_buf[:sz // 2]
        us_n = timed(lambda: dist.all_reduce(view), iters)
        rows.append({"bytes": sz, "daemon_us": round(us_d, 1), "daemon_busbw_gbs": round(sz / us_d / 1e3 * f, 1),
                     "stream_kernel_us": round(us_s, 1), "stream_kernel_busbw_gbs": round(sz / us_s / 1e3 * f, 1),
                     "nccl_2_28_us": round(us_n, 1), "nccl_2_28_busbw_gbs": round(sz / us_n / 1e3 * f, 1)})
    ctx.destroy()
    return {"dtype": "bf16", "n_gpus": world, "multimem_schedule_from_1MB": bool(nvls and world >= 4), "rows": rows}


def run(args):
    import faulthandler
    # a stalled run prints every thread's stack and exits instead of sitting on the GPU
    faulthandler.dump_traceback_later(int(os.environ.get("BENCH_WATCHDOG_S", "900")), exit=True)
    os.environ.setdefault("DFCCL_WAIT_TIMEOUT_MS", "60000")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch one rank per GPU with torchrun")
    torch.backends.cudnn.benchmark = True
    if args.impl == "reference":
        from baseline.reference_backend import ReferenceBackend, reference_unavailable
        why = reference_unavailable()
        if why:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": why}))
            return
        from baseline.reference_backend import RefDist
        d = RefDist()
        backend = ReferenceBackend(d)
    else:
        from dfccl_b200.parallel import init_distributed
        if args.graph and args.overlap:
            # The buckets of a captured backward pass are released milliseconds apart.  A daemon that stayed for all of
            # them would hold its SMs through most of the step; it leaves soon after each bucket instead and the
            # poller thread launches it again when the next release shows up (a few tens of microseconds).
            os.environ.setdefault("DFCCL_IDLE_QUIT_US", "100")
        d = init_distributed()
        if d.world > 1 and os.environ.get("DFCCL_DDP_NVLS", "1") != "0":
            # one multicast arena for the gradient buckets (about 160 MB) and the buffers of the all-reduce sweep
            d.comm.nvls_init(900 << 20)
        backend = DaemonBackend(d, args.daemon_blocks)
    from dfccl_b200.utils.clocks import ClockSampler        # reads nvidia-smi only
    tr = Trainer(args, d, backend)
    dev, B = d.device, args.batch
    g = torch.Generator(device="cpu").manual_seed(100 + d.rank)
    # synthetic data: N(0,1) images in bf16 and uniform random labels, pinned on the host
    n_host = 4
    host_x = [torch.randn(B, *IMG, generator=g).to(torch.bfloat16).pin_memory() for _ in range(n_host)]
    host_y = [torch.randint(0, CLASSES, (B,), generator=g).pin_memory() for _ in range(n_host)]
    dev_x = host_x[0].to(dev, non_blocking=True).contiguous(memory_format=torch.channels_last)
    dev_y = host_y[0].to(dev, non_blocking=True)
    torch.cuda.synchronize()

    def sync():
        d.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (cuDNN autotune, daemon start, allocator)
    for _ in range(max(args.warmup, 3)):
        tr.step(dev_x, dev_y)
    sync()

    # ---- timed region 1: device-resident inputs, CUDA events
    launches0 = backend.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(d.local_rank) as clk:
        sync()
        e0.record()
        for _ in range(args.steps):
            loss = tr.step(dev_x, dev_y)
        e1.record()
        sync()
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    launches = backend.launches() - launches0
    final_loss = float(loss.detach())
    clocks = clk.summary()

    # ---- timed region 2: end to end through the public API: H2D of each batch, D2H of each loss
    copy_stream = torch.cuda.Stream()
    loss_host = torch.zeros(args.steps, dtype=torch.float32).pin_memory()
    bufs = [(torch.empty_like(dev_x), torch.empty_like(dev_y)) for _ in range(2)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]

    def prefetch(i):
        k = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[k])
            # the copy itself converts the NCHW host batch to the channels-last device buffer
            bufs[k][0].copy_(host_x[i % n_host], non_blocking=True)
            bufs[k][1].copy_(host_y[i % n_host], non_blocking=True)
            ready[k].record(copy_stream)

    for k in range(2):
        consumed[k].record()
    sync()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    prefetch(0)
    for i in range(args.steps):
        if i + 1 < args.steps:
            prefetch(i + 1)
        k = i % 2
        torch.cuda.current_stream().wait_event(ready[k])
        loss = tr.step(bufs[k][0], bufs[k][1])
        consumed[k].record()
        loss_host[i:i + 1].copy_(loss.detach().reshape(1), non_blocking=True)
    e3.record()
    sync()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(e2.elapsed_time(e3), 0.0), world)
    assert torch.isfinite(loss_host).all(), "non-finite loss in the end-to-end run"

    info = backend.info()
    backend.close()
    sweep = allreduce_sweep(d) if (args.impl == "dfccl" and args.sweep and world > 1) else None
    if d.rank == 0:
        gb = B * world
        h2d = host_x[0].numel() * host_x[0].element_size() + host_y[0].numel() * host_y[0].element_size()
        out = {
            "metric": "resnet50_train_samples_per_s", "value": gb * args.steps / (ms / 1e3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic N(0,1) images 3x224x224 + uniform random labels; random-init weights",
            "impl": args.impl,
            "config": {"model": "ResNet-50 v1.5" if args.model == "resnet50" else args.model, "global_batch": gb,
                       "batch_per_gpu": B, "seq_len": None, "parallelism": f"dp{world}",
                       "grad_buckets_mb": BUCKET_MB,
                       "optimizer": ("fused SGD kernel, momentum 0.9 wd 1e-4, fp32 master weights" if args.impl == "dfccl"
                                     else "torch.optim.SGD momentum 0.9 wd 1e-4 on the bf16 parameters (no master copy)"),
                       "cuda_graph": bool(tr.use_graph), "overlap": bool(tr.use_graph and tr.overlap),
                       "gradient_path": (f"daemon all-reduce ({info.get('schedule', '')}), fused 1/N scale + bf16->fp32 cast, per-rank randomized "
                                         f"bucket order, {'released from inside the captured backward pass' if tr.use_graph and tr.overlap else 'submitted after the backward pass' if tr.use_graph else 'submitted from gradient hooks'}"
                                         if args.impl == "dfccl" else "reference library ncclAllReduce per bucket"),
                       "l2": "activations and gradients per step far exceed the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": gb * args.steps / (e2e_ms / 1e3), "unit": "samples/s", "ms_per_step": e2e_ms / args.steps,
                    "wall_ms_per_step": wall_ms / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "final_loss": final_loss,
            "backend_info": info,
        }
        if sweep is not None:
            out["allreduce_through_daemon"] = sweep
        print(json.dumps(out))
    d.destroy()


if __name__ == "__main__":
    run(parse())
