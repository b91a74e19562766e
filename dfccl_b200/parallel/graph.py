"""Whole-step CUDA graph: forward, loss and backward of a fixed-shape training step captured
once and replayed, so that the several hundred short kernels of a step cost one launch.

Works together with :class:`~dfccl_b200.parallel.ddp.DaemonDDP`: gradients are accumulated
into the static bucket views (fixed addresses, so they can be captured).  With ``overlap``
(the default) the gradient hooks run during capture and record, at the point of the backward
pass where a bucket becomes complete, a one-thread kernel that releases that bucket's
all-reduce (``dfcclTriggerOnStream``); before every replay the buckets' submissions are
published to the daemon in this rank's shuffled order (``dfcclRunDeferred``).  The daemon then
reduces a bucket while the rest of the captured backward pass is still running, and only the
last, small bucket is left when the replay ends.  Without ``overlap`` all buckets are submitted
after the replay.
"""
from __future__ import annotations

from typing import Callable

import torch


class GraphedStep:
    def __init__(self, net: torch.nn.Module, loss_fn: Callable, ddp, x: torch.Tensor, y: torch.Tensor, warmup: int = 3,
                 overlap: bool = True):
        self.ddp = ddp
        self.overlap = overlap
        # a replayed step is enqueued with a handful of calls: the daemon is woken by the poller when the first
        # bucket is released instead of being held on its SMs from the moment the waits are enqueued
        ddp.ctx.set_hold_on_wait(False)
        self.x = x.clone()
        self.y = y.clone()
        dev = x.device
        ddp.hooks_enabled = False
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):                   # cuDNN autotuning and allocator warm-up outside the capture
                loss_fn(net(self.x), self.y).backward()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        ddp.zero_grads()
        self.graph = torch.cuda.CUDAGraph()
        if overlap:
            ddp.begin_capture()
        with torch.cuda.graph(self.graph):
            self.loss = loss_fn(net(self.x), self.y)
            self.loss.backward()
        if overlap:
            ddp.end_capture()
        torch.cuda.synchronize(dev)
        ddp.zero_grads()

    def __call__(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        self.x.copy_(x, non_blocking=True)
        self.y.copy_(y, non_blocking=True)
        if self.overlap:
            self.ddp.publish_deferred()
            self.graph.replay()
            self.ddp.release_uncaptured()
        else:
            self.graph.replay()
            self.ddp.submit_all()
        return self.loss
