"""GPT-2 hybrid-parallel training throughput (tensor x pipeline x data parallel on one node).

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m dfccl_b200.benchmarks.gpt2_hybrid \\
        --tp 2 --pp 2 --dp 2 --steps 10 --warmup 3 --out gpt2.json
    ... --impl nccl      # comparison arm: same model and schedule, torch.distributed (NCCL) collectives + cuBLAS

GPT-2 medium (24 layers, d 1024, 16 heads, sequence 1024, vocabulary 50257), random-init bf16 weights,
uniform random token ids.  Per step every replica runs ``n_micro`` micro-batches of ``micro_batch``
sequences.  On this library's arm the tensor-parallel linears are the fused all-gather -> GEMM and
GEMM -> reduce-scatter kernels, gradients are all-reduced through the daemon (sharded weights over
the data-parallel group, replicated parameters over the stage group, per-rank shuffled order) and
the optimizer is the fused SGD kernel; pipeline transfers use NCCL point-to-point on both arms.
Times are CUDA events, max over ranks; the end-to-end figure includes the pinned-host -> device
copy of each step's tokens and the device -> host read of its loss.
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import threading
import time

import torch
import torch.distributed as dist

from dfccl_b200.models.gpt2 import GPT2Config, GPT2Stage
from dfccl_b200.parallel import init_distributed
from dfccl_b200.parallel import hybrid as hyb
from dfccl_b200.parallel.hybrid import HybridTrainer, build_mesh
from dfccl_b200.utils.clocks import ClockSampler


class TorchGradSync:
    """Comparison arm: flat gradient all-reduce per parameter group with torch.distributed, foreach SGD."""

    def __init__(self, groups, lr, momentum):
        self.groups, self.lr, self.mu = groups, lr, momentum
        self.hooks_enabled = False
        self.buckets = []
        self.launches = 0
        self.bufs = {}

    def finish_backward(self):
        for params, pg, scale in self.groups:
            grads = [p.grad for p in params if p.grad is not None]
            if not grads:
                continue
            flat = torch._utils._flatten_dense_tensors(grads)
            if pg is not None:
                dist.all_reduce(flat, group=pg)
            flat.mul_(scale)
            for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
                g.copy_(f)

    @torch.no_grad()
    def step(self):
        for params, _, _ in self.groups:
            ps = [p for p in params if p.grad is not None]
            gs = [p.grad for p in ps]
            ms = [self.bufs.setdefault(p, torch.zeros_like(p)) for p in ps]
            torch._foreach_mul_(ms, self.mu)
            torch._foreach_add_(ms, gs)
            torch._foreach_add_(ps, ms, alpha=-self.lr)
            torch._foreach_zero_(gs)                      # kept allocated: a captured backward pass accumulates in place

    def submit_all(self):
        pass

    def zero_grads(self):
        for params, _, _ in self.groups:
            gs = [p.grad for p in params if p.grad is not None]
            if gs:
                torch._foreach_zero_(gs)

    def stats(self):
        return {}

    def close(self):
        pass


def torch_groups(d, mesh):
    """torch.distributed groups matching the mesh's data-parallel and stage communicators."""
    tp, pp, dp = mesh.tp, mesh.pp, mesh.dp
    dp_pg = stage_pg = None
    for c in range(tp * pp):
        h = dist.new_group([c + k * tp * pp for k in range(dp)])
        if c == d.rank % (tp * pp):
            dp_pg = h
    for s in range(pp):
        h = dist.new_group([r for r in range(d.world) if (r // tp) % pp == s])
        if s == mesh.pp_rank:
            stage_pg = h
    return dp_pg, stage_pg


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=0)
    ap.add_argument("--pp", type=int, default=0)
    ap.add_argument("--dp", type=int, default=0)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--n-micro", type=int, default=4)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="medium", choices=["medium", "tiny"])
    ap.add_argument("--impl", default="dfccl", choices=["dfccl", "nccl"])
    ap.add_argument("--optimizer", default="sgd", choices=["sgd", "adamw"], help="fused optimizer of this library's arm")
    ap.add_argument("--graph", type=int, default=0, help="capture forward + backward of the whole step in one CUDA graph")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    faulthandler.dump_traceback_later(int(os.environ.get("BENCH_WATCHDOG_S", "600")), exit=True)
    os.environ.setdefault("DFCCL_WAIT_TIMEOUT_MS", "60000")
    d = init_distributed()
    w = d.world
    if not a.tp:
        a.tp, a.pp, a.dp = {1: (1, 1, 1), 2: (2, 1, 1), 4: (2, 2, 1), 8: (2, 2, 2)}[w]
    cfg = GPT2Config.medium() if a.model == "medium" else GPT2Config.tiny()
    mesh = build_mesh(d, a.tp, a.pp, a.dp)
    mesh.tp_group.library = "dfccl" if a.impl == "dfccl" else "torch"
    stage = GPT2Stage(cfg, mesh.tp_group, mesh.pp_rank, a.pp, a.micro_batch)
    tr = HybridTrainer(d, mesh, stage, n_micro=a.n_micro, lr=0.01 if a.optimizer == "sgd" else 3e-4, seed=5, use_graph=bool(a.graph), optimizer=a.optimizer)
    if a.impl == "nccl":
        tr.ddp.close()
        params = [p for p in stage.parameters()]
        dp_pg, stage_pg = torch_groups(d, mesh) if w > 1 else (None, None)
        for p in params:                                  # undo the flat-bucket views of the daemon arm
            p.data = p.data.clone()
            p.grad = None
        tr.ddp = TorchGradSync([([p for p in params if not getattr(p, "tp_replicated", False)], dp_pg, 1.0 / a.dp),
                                ([p for p in params if getattr(p, "tp_replicated", False)], stage_pg, 1.0 / a.dp)], 0.01, 0.9)
    dev = d.device
    g = torch.Generator().manual_seed(100 + mesh.dp_rank)
    shape = (a.n_micro, a.micro_batch, cfg.seq_len + 1)
    host = [torch.randint(0, cfg.vocab, shape, generator=g).pin_memory() for _ in range(4)]
    dtok = host[0][..., :-1].to(dev)
    dtgt = host[0][..., 1:].to(dev)

    def sync():
        d.barrier()
        torch.cuda.synchronize()

    progress = {"step": 0, "t": time.time()}

    def monitor():                                          # a stalled run says where the daemon stands, then leaves
        limit = float(os.environ.get("BENCH_STALL_S", "60"))
        while True:
            time.sleep(2.0)
            if progress["step"] < 0:
                return
            if time.time() - progress["t"] > limit:
                hs = tr.ddp.ctx.host_stats() if hasattr(tr.ddp, "ctx") else {}
                print(f"[rank {d.rank}] no step finished for {limit:.0f} s at step {progress['step']}; daemon (host view): {hs}", flush=True)
                faulthandler.dump_traceback()
                os._exit(3)

    threading.Thread(target=monitor, daemon=True).start()

    def one_step(tok, tgt):
        out = tr.step(tok, tgt)
        progress["step"] += 1
        progress["t"] = time.time()
        return out

    for _ in range(max(a.warmup, 3)):
        one_step(dtok, dtgt)
        torch.cuda.synchronize()
    sync()
    l0 = tr.ddp.stats().get("daemonLaunches", 0) + tr.ddp.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(d.local_rank) as clk:
        sync()
        e0.record()
        for _ in range(a.steps):
            loss = one_step(dtok, dtgt)
        e1.record()
        sync()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if w > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t) / a.steps
    launches = tr.ddp.stats().get("daemonLaunches", 0) + tr.ddp.launches - l0
    final_loss = float(loss)
    # end to end: tokens from pinned host memory every step, loss read back every step
    loss_host = torch.zeros(a.steps, dtype=torch.float32).pin_memory()
    sync()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(a.steps):
        hb = host[i % len(host)]
        db = hb.to(dev, non_blocking=True)
        loss = one_step(db[..., :-1], db[..., 1:])
        loss_host[i:i + 1].copy_(loss, non_blocking=True)
    e3.record()
    sync()
    t = torch.tensor([e2.elapsed_time(e3)], device=dev, dtype=torch.float64)
    if w > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t) / a.steps
    tokens = a.dp * a.n_micro * a.micro_batch * cfg.seq_len
    flops = 6.0 * cfg.n_params() * tokens + 12.0 * cfg.n_layer * cfg.d_model * cfg.seq_len * tokens
    stats = tr.ddp.stats()
    progress["step"] = -1
    tr.close()
    if d.rank == 0:
        out = {"metric": "gpt2_medium_train_tokens_per_s" if a.model == "medium" else "gpt2_tiny_train_tokens_per_s",
               "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": w, "steps": a.steps, "warmup": max(a.warmup, 3),
               "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "impl": a.impl,
               "data": "uniform random token ids; random-init weights",
               "model_tflops_per_gpu": flops / (ms / 1e3) / 1e12 / w,
               "config": {"model": f"GPT-2 {a.model}", "parallelism": f"tp{a.tp} x pp{a.pp} x dp{a.dp}", "micro_batch": a.micro_batch,
                          "n_micro": a.n_micro, "global_batch": a.dp * a.n_micro * a.micro_batch, "seq_len": cfg.seq_len, "cuda_graph": bool(a.graph),
                          "schedule": "1F1B, receives posted one micro-batch ahead" if tr.schedule == "1f1b" else "GPipe",
                          "pipeline_link_ctas": hyb.PP_CTAS, "optimizer": "SGD momentum 0.9, fp32 master weights" if a.impl == "dfccl" else "SGD momentum 0.9 (bf16)"},
               "clocks": clk.summary(),
               "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": host[0].numel() * 8, "d2h_bytes_per_step": 4},
               "gpu_launches": launches, "final_loss": final_loss, "pp_bytes_per_step": tr.pp_bytes // (max(a.warmup, 3) + 2 * a.steps),
               "daemon_stats": stats}
        print(json.dumps(out))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(out, f, indent=1)
    d.destroy()


if __name__ == "__main__":
    main()
