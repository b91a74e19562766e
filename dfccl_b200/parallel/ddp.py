"""Data parallelism over the daemon.

Parameters are regrouped into flat buckets (default 25 MB of gradient each).  Every
bucket owns
  * a flat parameter array (the module's parameters become views into it),
  * a flat gradient array in the symmetric heap (``param.grad`` are views into it, so the
    backward pass writes gradients where the peers can read them - nothing is copied),
  * an fp32 array the all-reduce writes the averaged gradient to: the 1/world scale and the
    cast to fp32 happen inside the collective,
  * fp32 master weights and momentum for the fused optimizer step.
One all-reduce per bucket is registered with the daemon.  When the last gradient of a
bucket has been accumulated the bucket is submitted *stream-ordered*: a stream memory
operation releases it after the backward kernels already enqueued, no host thread waits.
Submission order can be shuffled per rank (``randomize_order``) - ranks then issue the
same collectives in different orders, which is exactly what the daemon makes safe.

The reference has no training integration in its tree; its authors drove data-parallel
training from an external framework through the register-then-submit calls
(reference: src/nccl.h.in:318-333, debug constants for a 161-collective ResNet job in
src/include/collectives_ofccl.h:63,78-100).
"""
from __future__ import annotations

import ctypes as C
import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from .. import native as nv
from ..utils.tensors import HeapTensorPool, nccl_dtype
from .groups import Dist


@dataclass(eq=False)
class Bucket:
    index: int
    dtype: torch.dtype
    params: List[nn.Parameter] = field(default_factory=list)
    offsets: List[int] = field(default_factory=list)
    numel: int = 0
    flat_param: Optional[torch.Tensor] = None
    grad: Optional[torch.Tensor] = None        # heap, param dtype
    grad32: Optional[torch.Tensor] = None      # heap, fp32: all-reduce output
    master: Optional[torch.Tensor] = None
    momentum: Optional[torch.Tensor] = None    # SGD momentum, or AdamW first moment
    moment2: Optional[torch.Tensor] = None     # AdamW second moment
    pending: int = 0
    coll_id: int = 0
    comm: Optional[nv.Comm] = None             # the group this bucket is reduced over
    scale: float = 1.0
    nvls: bool = False                         # arrays live in the switch-multicast arena, reduced by multimem
    deferred: bool = False                     # published ahead of a captured step; its release is part of the graph


def _esize(dt: torch.dtype) -> int:
    return torch.empty((), dtype=dt).element_size()


def _pad512(n: int) -> int:
    return (n + 511) // 512 * 512


def _view_like(flat: torch.Tensor, off: int, p: torch.Tensor) -> torch.Tensor:
    """View of flat[off : off + p.numel()] with p's shape and memory format."""
    seg = flat[off:off + p.numel()]
    if p.dim() == 4 and p.is_contiguous(memory_format=torch.channels_last) and not p.is_contiguous():
        n, c, h, w = p.shape
        return seg.view(n, h, w, c).permute(0, 3, 1, 2)
    return seg.view(p.shape)


class DaemonDDP:
    """Wraps ``module`` for data-parallel training through the daemon.

    Typical step::

        loss = criterion(ddp.module(x), y)
        loss.backward()          # buckets are submitted from gradient hooks
        ddp.finish_backward()    # the compute stream waits (on the device) for all buckets
        ddp.step()               # fused SGD over the flat buckets, gradients zeroed
    """

    def __init__(self, module: nn.Module, dist: Dist, *, bucket_mb: float = 25.0, lr: float = 0.1, momentum: float = 0.9,
                 weight_decay: float = 1e-4, randomize_order: bool = True, window: int = 2, seed: int = 0,
                 coll_id_base: int = 0, comm: Optional[nv.Comm] = None, n_blocks: int = 0,
                 daemon_blocks: int = 8, daemon_threads: int = 0, param_groups: Optional[Sequence[dict]] = None,
                 optimizer: str = "sgd", betas=(0.9, 0.999), eps: float = 1e-8, nvls: Optional[bool] = None,
                 ctx: Optional[nv.RankCtx] = None):
        """``param_groups`` (hybrid parallelism): a list of ``{"params": [...], "comm": Comm, "scale": float}``;
        every group gets its own buckets, reduced over its own communicator (sum times ``scale``).  All
        groups share this rank's one daemon, so ranks may submit them in any order.

        ``nvls``: keep the gradient buckets in the communicator's switch-multicast arena and reduce them with the
        multimem schedule (the NVLink switch adds the members' copies; every GPU moves one message size instead of
        two).  ``None`` = when the fabric offers it and the communicator has at least four ranks
        (``DFCCL_DDP_NVLS=0`` switches it off); memory bound to a
        multicast object ties the ranks' fates together, so tests of failure paths pass ``False``.

        ``ctx``: a rank context that already holds registrations (the fused tensor-parallel operators of a hybrid
        job, under ids below ``coll_id_base``) and is not finalized yet; the buckets are added to it and this
        wrapper finalizes and, in ``close``, destroys it."""
        self.module = module
        self.dist = dist
        self.comm = comm or dist.comm
        self.world = self.comm.nranks
        self.device = dist.device
        self.lr, self.mu, self.wd = lr, momentum, weight_decay
        if optimizer not in ("sgd", "adamw"):
            raise ValueError("optimizer must be 'sgd' or 'adamw'")
        self.optimizer, self.betas, self.eps = optimizer, (float(betas[0]), float(betas[1])), float(eps)
        self._t = 0                              # optimizer steps taken (AdamW bias correction)
        self.randomize = randomize_order
        self.window = max(1, window)
        self._rng = random.Random(seed * 7919 + dist.rank)
        self._lib = nv.lib()
        self._pool = HeapTensorPool(self.comm, self.device)
        self._ready: List[Bucket] = []
        self._submitted: List[Bucket] = []
        self._first_step = True
        self._capturing = False                 # gradient hooks record bucket releases into a stream capture (see graph.GraphedStep)
        self._captured: List[Bucket] = []
        self.hooks_enabled = True               # switched off while a captured step runs (see graph.GraphedStep)
        self.launches = 0                       # kernels of this library launched by step()
        self.buckets: List[Bucket] = []
        self._nvls_request = nvls
        self.nvls_comms: List[nv.Comm] = []       # communicators whose buckets live in the multicast arena
        if param_groups is None:
            param_groups = [{"params": [p for p in module.parameters() if p.requires_grad], "comm": self.comm,
                             "scale": 1.0 / self.world}]
        for g in param_groups:
            self._build_buckets(int(bucket_mb * (1 << 20)), g["params"], g.get("comm") or self.comm, float(g["scale"]))
        self._place_gradients()
        self.ctx = ctx if ctx is not None else nv.RankCtx(dist.rank, dist.local_rank if self.device.type == "cuda" else -1)
        # gradient buckets need a fraction of the fabric: a small grid leaves the SMs to the training kernels
        if self.device.type == "cuda":
            self.ctx.set_daemon_geometry(daemon_blocks, daemon_threads)
        for b in self.buckets:
            b.coll_id = coll_id_base + b.index
            self.ctx.prepare(b.coll_id, b.comm, nv.ALLREDUCE, b.numel, nccl_dtype(b.dtype), out_dtype=nv.FLOAT32,
                             op=nv.SUM, scale=b.scale, n_blocks=n_blocks,
                             algo=nv.ALGO_NVLS if b.nvls else nv.ALGO_AUTO, arena_buffers=b.nvls)
        self.ctx.finalize()
        if self.device.type == "cuda":
            nv.check(self._lib.dfcclOpsWarm(), "dfcclOpsWarm")   # load the optimizer kernels before any stream can block
        self._hooks = []
        for b in self.buckets:
            for p in b.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(b)))

    # ------------------------------------------------------------------ construction
    def _build_buckets(self, bucket_bytes: int, params, comm, scale: float) -> None:
        first = len(self.buckets)
        params = [p for p in params if p.requires_grad]
        by_dtype: Dict[torch.dtype, List[nn.Parameter]] = {}
        for p in reversed(params):              # gradients arrive roughly in reverse registration order
            by_dtype.setdefault(p.dtype, []).append(p)
        for dt, plist in by_dtype.items():
            cur: Optional[Bucket] = None
            esize = torch.empty((), dtype=dt).element_size()
            for p in plist:
                if cur is None or (cur.numel + p.numel()) * esize > bucket_bytes and cur.numel > 0:
                    cur = Bucket(len(self.buckets), dt)
                    self.buckets.append(cur)
                cur.offsets.append(cur.numel)
                cur.params.append(p)
                cur.numel += (p.numel() + 7) // 8 * 8      # keep every parameter 16-byte aligned
        for b in self.buckets[first:]:
            b.comm, b.scale = comm, scale
            b.flat_param = torch.empty(b.numel, dtype=b.dtype, device=self.device)
            b.flat_param.zero_()
            with torch.no_grad():
                for p, off in zip(b.params, b.offsets):
                    v = _view_like(b.flat_param, off, p)
                    v.copy_(p.data)
                    p.data = v
            b.master = b.flat_param.float().clone()
            b.momentum = torch.zeros_like(b.master)
            b.moment2 = torch.zeros_like(b.master) if self.optimizer == "adamw" else None
            b.pending = len(b.params)

    def _place_gradients(self) -> None:
        """Gradient arrays (input of the all-reduce, in the parameters' dtype) and fp32 results: in the multicast
        arena of the bucket's communicator where the fabric has one, in the symmetric heap otherwise."""
        import os
        want = self._nvls_request
        if want is None:
            want = os.environ.get("DFCCL_DDP_NVLS", "1") != "0"
        by_comm: Dict[int, List[Bucket]] = {}
        for b in self.buckets:
            by_comm.setdefault(id(b.comm), []).append(b)
        for bl in by_comm.values():
            comm = bl[0].comm
            need = sum(_pad512(b.numel * _esize(b.dtype)) + _pad512(b.numel * 4) for b in bl)
            # the switch halves the bytes a GPU moves only from four ranks on (on two ranks every schedule moves one
            # message size per direction, and plain peer loads / stores do that faster)
            min_ranks = int(os.environ.get("DFCCL_DDP_NVLS_MIN_RANKS", "4")) if self._nvls_request is None else 2
            # (on the host backend only when asked for by name: the arena is emulated there, for tests)
            use = bool(want) and (self.device.type == "cuda" or self._nvls_request is True) and comm.nranks >= min_ranks and \
                all(b.dtype in (torch.bfloat16, torch.float16, torch.float32) for b in bl)
            # collective call: every member asks, and all of them get the same answer
            if use and not comm.nvls_init(need + ((80 << 20) if self.device.type == "cuda" else (1 << 20))):
                use = False
            if use:
                _uc, _mc, total, used = comm.nvls_info()
                use = total - used >= need              # an arena made earlier (by someone else) may be too small
            if use:
                self.nvls_comms.append(comm)
            for b in bl:
                b.nvls = use
                if use:
                    from ..utils.tensors import tensor_from_ptr
                    b.grad = tensor_from_ptr(comm.nvls_alloc(b.numel * _esize(b.dtype)), (b.numel,), b.dtype, self.device).zero_()
                    b.grad32 = tensor_from_ptr(comm.nvls_alloc(b.numel * 4), (b.numel,), torch.float32, self.device).zero_()
                else:
                    b.grad = self._pool.zeros((b.numel,), b.dtype)
                    b.grad32 = self._pool.zeros((b.numel,), torch.float32)
                with torch.no_grad():
                    for p, off in zip(b.params, b.offsets):
                        p.grad = _view_like(b.grad, off, p)

    def gradient_path(self) -> str:
        """Which schedule the buckets take, for benchmark records."""
        kinds = sorted({"multimem (NVLS)" if b.nvls else "peer loads/stores" for b in self.buckets})
        return " + ".join(kinds)

    def _make_hook(self, b: Bucket):
        def hook(_param):
            if self._capturing:
                b.pending -= 1
                if b.pending == 0:
                    self.ctx.trigger_on_stream(b.coll_id, self._stream())
                    self._captured.append(b)
                return
            if not self.hooks_enabled:
                return
            b.pending -= 1
            if b.pending == 0:
                self._bucket_ready(b)
        return hook

    # ------------------------------------------------------------------ per step
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream if self.device.type == "cuda" else 0

    def _bucket_ready(self, b: Bucket) -> None:
        self._ready.append(b)
        if len(self._ready) >= self.window:
            self._flush()

    def _flush(self) -> None:
        batch, self._ready = self._ready, []
        if self.randomize:
            self._rng.shuffle(batch)
        s = self._stream()
        for b in batch:
            self.ctx.run_on_stream(b.coll_id, b.grad.data_ptr(), b.grad32.data_ptr(), s)
            self._submitted.append(b)

    def submit_all(self) -> None:
        """Submit every bucket now (after a captured backward pass), in this rank's shuffled order."""
        self._ready = [b for b in self.buckets if b not in self._submitted]
        self._flush()

    # ---- captured steps: the release of a bucket is a kernel inside the graph, the submission is published before
    # ---- the replay, so the bucket is reduced while the rest of the captured backward pass still runs
    def begin_capture(self) -> None:
        """Gradient hooks now record the buckets' releases into the stream that is being captured."""
        self._capturing = True
        self._captured: List[Bucket] = []
        for b in self.buckets:
            b.pending = len(b.params)

    def end_capture(self) -> None:
        self._capturing = False
        for b in self.buckets:
            b.pending = len(b.params)

    def publish_deferred(self) -> None:
        """Before a replay: publish every bucket's submission, in this rank's shuffled order."""
        batch = [b for b in self.buckets if b not in self._submitted]
        if self.randomize:
            self._rng.shuffle(batch)
        for b in batch:
            self.ctx.run_deferred(b.coll_id, b.grad.data_ptr(), b.grad32.data_ptr())
            self._submitted.append(b)

    def release_uncaptured(self) -> None:
        """After a replay: buckets whose release is not part of the graph (not every parameter received a gradient
        during capture) are released now."""
        s = self._stream()
        for b in self.buckets:
            if b not in self._captured:
                self.ctx.trigger_on_stream(b.coll_id, s)

    def zero_grads(self) -> None:
        for b in self.buckets:
            b.grad.zero_()

    def finish_backward(self) -> None:
        """Submit what is still queued and make the current stream wait for every bucket."""
        for b in self.buckets:                   # buckets whose parameters did not all receive a gradient
            if b not in self._submitted and b not in self._ready:
                self._ready.append(b)
        self._flush()
        s = self._stream()
        for b in self._submitted:
            self.ctx.stream_wait(b.coll_id, s)
        self._submitted = []
        for b in self.buckets:
            b.pending = len(b.params)

    def step(self, lr: Optional[float] = None) -> None:
        """One fused optimizer kernel per flat bucket (SGD with momentum, or AdamW), then clear the gradients."""
        lr = self.lr if lr is None else lr
        s = self._stream()
        self._t += 1
        b1, b2 = self.betas
        for b in self.buckets:
            if self.device.type == "cuda":
                if self.optimizer == "adamw":
                    nv.check(self._lib.dfcclFusedAdamWStep(
                        C.c_void_p(b.master.data_ptr()), C.c_void_p(b.grad32.data_ptr()), C.c_void_p(b.momentum.data_ptr()),
                        C.c_void_p(b.moment2.data_ptr()), C.c_void_p(b.flat_param.data_ptr()), b.numel, nccl_dtype(b.dtype),
                        lr, b1, b2, self.eps, self.wd, self._t, C.c_void_p(s)), "dfcclFusedAdamWStep")
                else:
                    nv.check(self._lib.dfcclFusedSgdStep(
                        C.c_void_p(b.master.data_ptr()), C.c_void_p(b.grad32.data_ptr()), C.c_void_p(b.momentum.data_ptr()),
                        C.c_void_p(b.flat_param.data_ptr()), b.numel, nccl_dtype(b.dtype), lr, self.mu, self.wd,
                        1 if self._first_step else 0, C.c_void_p(s)), "dfcclFusedSgdStep")
                self.launches += 1
            elif self.optimizer == "adamw":        # host backend (tests): the same arithmetic in PyTorch
                g = b.grad32
                b.momentum.mul_(b1).add_(g, alpha=1 - b1)
                b.moment2.mul_(b2).addcmul_(g, g, value=1 - b2)
                step_size = lr / (1 - b1 ** self._t)
                denom = b.moment2.sqrt() / (1 - b2 ** self._t) ** 0.5 + self.eps
                b.master.mul_(1 - lr * self.wd).addcdiv_(b.momentum, denom, value=-step_size)
                b.flat_param.copy_(b.master)
            else:
                g = b.grad32 + self.wd * b.master
                b.momentum.mul_(0.0 if self._first_step else self.mu).add_(g)
                b.master.sub_(lr * b.momentum)
                b.flat_param.copy_(b.master)
            b.grad.zero_()
        self._first_step = False

    def stats(self) -> Dict[str, int]:
        return self.ctx.stats()

    # ------------------------------------------------------------------ checkpoint / resume
    def state_dict(self) -> Dict[str, object]:
        """Optimizer state of this rank (fp32 master weights and momentum per bucket), for ``torch.save``.  The
        bucket layout is a function of the module and the bucket size, so a wrapper built the same way loads it."""
        return {"first_step": self._first_step, "lr": self.lr, "momentum": self.mu, "weight_decay": self.wd,
                "optimizer": self.optimizer, "t": self._t,
                "buckets": [{"numel": b.numel, "dtype": str(b.dtype), "master": b.master.detach().cpu().clone(),
                             "momentum": b.momentum.detach().cpu().clone(),
                             "moment2": None if b.moment2 is None else b.moment2.detach().cpu().clone()} for b in self.buckets]}

    def load_state_dict(self, state: Dict[str, object]) -> None:
        bs = state["buckets"]
        if state.get("optimizer", "sgd") != self.optimizer:
            raise ValueError("checkpoint was written by another optimizer")
        if len(bs) != len(self.buckets) or any(x["numel"] != b.numel or x["dtype"] != str(b.dtype) for x, b in zip(bs, self.buckets)):
            raise ValueError("checkpoint was written with another bucket layout (module or bucket size differ)")
        with torch.no_grad():
            for x, b in zip(bs, self.buckets):
                b.master.copy_(x["master"])
                b.momentum.copy_(x["momentum"])
                if b.moment2 is not None:
                    b.moment2.copy_(x["moment2"])
                b.flat_param.copy_(b.master)          # the module's parameters are views of the flat array
                b.grad.zero_()
        self._first_step = bool(state["first_step"])
        self._t = int(state.get("t", 0))
        self.lr, self.mu, self.wd = float(state["lr"]), float(state["momentum"]), float(state["weight_decay"])

    def close(self) -> None:
        for h in self._hooks:
            h.remove()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.ctx.destroy()
        self._pool.release()
