"""Hybrid tensor x pipeline x data parallel training on one daemon per rank.

Rank layout (tensor-parallel ranks adjacent, then pipeline stages, then replicas):

    rank = dp_rank * (pp * tp) + pp_rank * tp + tp_rank

Communicators of this library are split from the world communicator: the tensor-parallel group (fused
GEMM + collective kernels and the backward collectives), the data-parallel group (gradients of the
sharded weights) and the "stage" group = every rank holding the same stage (gradients of the
replicated parameters: layer norms, row-parallel biases, embeddings - summed over the tensor-parallel
ranks, averaged over the replicas).  All gradient all-reduces of a rank, whatever their group, are
registered with the rank's one daemon and submitted stream-ordered in a per-rank shuffled order:
collectives of overlapping groups issued in different orders by different ranks is the situation the
reference's simulator shows deadlocking in-order libraries (reference: simulator/simulator.py:434-493)
and the daemon makes safe.  Activations and their gradients move between stages with
``torch.distributed`` point-to-point (NCCL on GPUs, gloo in the CPU tests).

Schedule: one-forward-one-backward (1F1B) by default - stage ``s`` of ``pp`` runs ``pp - 1 - s``
forward passes ahead, then alternates forward and backward, so it holds at most ``pp - s`` micro-batches
of activations instead of all of them; ``schedule="gpipe"`` runs all forwards, then all backwards.
Receives are posted ahead: the input of the next forward pass and the gradient of the next backward
pass are already being received while the current micro-batch computes.  Every neighbour and direction
has a two-member process group of its own (activations to the successor, gradients back), so a stage's
posted receive from its successor can never sit in front of its own send to that successor in one
communicator's queue (that order, on one in-order queue per pair, is a deadlock), and every link is
opened once while the mesh is built, both ends in the same order: the first transfer of a link blocks
on the host until the other end joins, which receives posted ahead would turn into a cycle.
Gradients are accumulated in the flat buckets; the buckets are
released to the daemon from the gradient hooks of the last micro-batch's backward pass.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import native as nv
from ..ops.fused_linear import TpGroup
from ..utils.tensors import nccl_dtype
from .ddp import DaemonDDP
from .groups import Dist


@dataclass
class Mesh:
    tp: int
    pp: int
    dp: int
    tp_rank: int
    pp_rank: int
    dp_rank: int
    tp_group: TpGroup
    dp_comm: nv.Comm
    stage_comm: nv.Comm
    # pipeline traffic: one two-member process group per neighbour and direction, so that every transfer has a
    # communicator (and a stream) of its own; None where there is no such neighbour
    fwd_prev: object = None      # activations arriving from the previous stage
    fwd_next: object = None      # activations leaving for the next stage
    bwd_next: object = None      # activation gradients arriving from the next stage
    bwd_prev: object = None      # activation gradients leaving for the previous stage
    ctx: object = None           # this rank's context: fused tensor-parallel operators and gradient buckets share it

    def close(self) -> None:
        for c in (self.tp_group.comm, self.dp_comm, self.stage_comm):
            c.destroy()


PP_CTAS = int(os.environ.get("DFCCL_PP_CTAS", "2"))


def _pp_group_options(d: Dist):
    """A receive that is posted ahead is a kernel that holds its SMs until the matching send runs - possibly for a whole
    pipeline stage's compute.  The fused tensor-parallel kernels need all their CTAs resident together, so the SMs such
    receives may hold are bounded here (``PP_CTAS`` CTAs per transfer) and kept out of the fused grids
    (``HybridTrainer``: daemon blocks + one posted receive per direction)."""
    if d.device.type != "cuda":
        return None
    try:
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.min_ctas = 1
        opts.config.max_ctas = PP_CTAS
        return opts
    except Exception:                                        # a build of the bindings without communicator configuration
        return None


def build_mesh(d: Dist, tp: int, pp: int, dp: int) -> Mesh:
    assert tp * pp * dp == d.world, f"tp {tp} x pp {pp} x dp {dp} != world {d.world}"
    r = d.rank
    tp_rank, pp_rank, dp_rank = r % tp, (r // tp) % pp, r // (tp * pp)
    tp_comm = d.comm.split(r // tp, r)
    dp_comm = d.comm.split(r % (tp * pp), r)
    stage_comm = d.comm.split(pp_rank, r)
    pg = None
    if d.world > 1 and tp > 1:
        for g in range(d.world // tp):                      # every rank creates every group, in the same order
            ranks = list(range(g * tp, (g + 1) * tp))
            h = dist.new_group(ranks)
            if g == r // tp:
                pg = h
    links = {}
    if d.world > 1 and pp > 1:
        # every rank creates every group, in the same order: (lower rank a, its neighbour a + tp of the next stage),
        # one group for the activations and one for their gradients
        opts = _pp_group_options(d)
        for a in range(d.world):
            if (a // tp) % pp == pp - 1:
                continue
            f, b = dist.new_group([a, a + tp], pg_options=opts), dist.new_group([a, a + tp], pg_options=opts)
            if r in (a, a + tp):
                links[a] = (f, b)
    fwd_prev, bwd_prev = links.get(r - tp, (None, None)) if pp_rank > 0 else (None, None)
    fwd_next, bwd_next = links.get(r, (None, None)) if pp_rank < pp - 1 else (None, None)
    if links:
        # The first transfer between two ranks sets their connection up on the host and blocks until the other side
        # calls its half.  Receives that are posted ahead would meet in a cycle there (stage 0 posts its gradient
        # receive before it has sent anything, stage 1 its activation receive), so every link is opened here once,
        # boundary by boundary, both sides in the same order.
        tiny = torch.zeros(8, device=d.device)
        for k in range(pp - 1):
            if pp_rank == k:
                dist.send(tiny, r + tp, group=fwd_next)
                dist.recv(tiny, r + tp, group=bwd_next)
            elif pp_rank == k + 1:
                dist.recv(tiny, r - tp, group=fwd_prev)
                dist.send(tiny, r - tp, group=bwd_prev)
        if d.device.type == "cuda":
            torch.cuda.synchronize(d.device)
    # one rank context for everything this rank registers: on GPUs the fused tensor-parallel operators take the first
    # ids (as the model is built), the gradient buckets follow (HybridTrainer)
    ctx = nv.RankCtx(d.rank, d.local_rank) if d.device.type == "cuda" else None
    return Mesh(tp, pp, dp, tp_rank, pp_rank, dp_rank, TpGroup(tp_comm, pg, d.device, ctx=ctx), dp_comm, stage_comm, fwd_prev, fwd_next, bwd_next,
                bwd_prev, ctx)


class HybridTrainer:
    """One optimizer step = ``n_micro`` micro-batches of ``micro_batch`` sequences per replica."""

    def __init__(self, d: Dist, mesh: Mesh, stage: torch.nn.Module, *, n_micro: int, bucket_mb: float = 25.0, lr: float = 0.01,
                 momentum: float = 0.9, weight_decay: float = 0.0, seed: int = 0, daemon_blocks: int = 8, use_graph: bool = False,
                 optimizer: str = "sgd", schedule: str = "1f1b"):
        if schedule not in ("1f1b", "gpipe"):
            raise ValueError("schedule must be '1f1b' or 'gpipe'")
        self.d, self.mesh, self.stage, self.n_micro, self.schedule = d, mesh, stage, n_micro, schedule
        params = [p for p in stage.parameters() if p.requires_grad]
        sharded = [p for p in params if not getattr(p, "tp_replicated", False)]
        replicated = [p for p in params if getattr(p, "tp_replicated", False)]
        groups = [{"params": sharded, "comm": mesh.dp_comm, "scale": 1.0 / mesh.dp},
                  {"params": replicated, "comm": mesh.stage_comm, "scale": 1.0 / mesh.dp}]
        # the context already holds the fused operators the stage registered while it was built; finalizing it (inside
        # DaemonDDP) also keeps the daemon's SMs out of the fused kernels' grids
        self.ddp = DaemonDDP(stage, d, bucket_mb=bucket_mb, lr=lr, momentum=momentum, weight_decay=weight_decay,
                             randomize_order=True, seed=seed, param_groups=groups, daemon_blocks=daemon_blocks, optimizer=optimizer,
                             ctx=mesh.ctx, coll_id_base=mesh.tp_group.next_id if mesh.ctx is not None else 0)
        self.ddp.hooks_enabled = False
        if d.device.type == "cuda" and mesh.pp > 1 and mesh.tp > 1:
            # SMs that may be taken while a fused kernel starts: the daemon's blocks and one posted receive per direction
            nv.check(nv.lib().dfcclGemmReserveSms(daemon_blocks + 2 * PP_CTAS), "dfcclGemmReserveSms")
        # DFCCL_PP_POST_AHEAD=0: post every pipeline receive right before it is waited for (no kernel of the transfer
        # library is then resident while this rank computes)
        self.post_ahead = os.environ.get("DFCCL_PP_POST_AHEAD", "1") != "0"
        # The first step of a process loads kernels and grows allocator pools, and some of that waits for the device to
        # go idle - which it never does while a receive that was posted ahead spins for a peer that is stuck in its own
        # first launches.  So the first step posts every receive right before its wait; posting ahead starts with the
        # second step, when everything a step launches has been launched once.
        self._warm = False
        self.prev = d.rank - mesh.tp if mesh.pp_rank > 0 else None
        self.next = d.rank + mesh.tp if mesh.pp_rank < mesh.pp - 1 else None
        self._loss = torch.zeros(1, dtype=torch.float32, device=d.device)
        self.pp_bytes = 0
        self.peak_live_microbatches = 0          # most micro-batches whose activations were held at once
        self._step_done = None
        self._sends: list = []
        self.use_graph = bool(use_graph) and d.device.type == "cuda"
        self._graph = None
        self._tok = self._tgt = None

    def _hidden(self) -> torch.Tensor:
        st = self.stage
        return torch.empty(st.rows, st.cfg.d_model, dtype=torch.bfloat16, device=self.d.device)

    def _send(self, t: torch.Tensor, dst: int, group):
        self.pp_bytes += t.numel() * t.element_size()
        return dist.isend(t.contiguous(), dst, group=group)

    def _forward_backward(self, tokens, targets, hooks: bool) -> None:
        """The micro-batches of one step in the configured order; the loss shares accumulate in ``self._loss``."""
        st, n, ddp, m = self.stage, self.n_micro, self.ddp, self.mesh
        ahead = self.post_ahead and self._warm
        ins, outs = {}, {}
        frecv, brecv = {}, {}                                # posted receives: micro-batch -> (buffer, request)

        def post_f(i):
            if self.prev is not None and i < n and i not in frecv:
                x = self._hidden()
                frecv[i] = (x, dist.irecv(x, self.prev, group=m.fwd_prev))

        def post_b(i):
            if self.next is not None and i < n and i not in brecv:
                g = self._hidden()
                brecv[i] = (g, dist.irecv(g, self.next, group=m.bwd_next))

        def forward(i):
            if self.prev is None:
                x = tokens[i]
            else:
                post_f(i)
                if ahead:
                    post_f(i + 1)                            # the next input travels while this micro-batch computes
                x, req = frecv.pop(i)
                req.wait()
                x.requires_grad_(True)
            y = st(x, targets[i] if self.next is None else None)
            if self.next is not None:
                self._sends.append(self._send(y.detach(), self.next, m.fwd_next))
            ins[i], outs[i] = x, y
            self.peak_live_microbatches = max(self.peak_live_microbatches, len(outs))

        def backward(i):
            ddp.hooks_enabled = hooks and i == n - 1         # buckets go to the daemon as the last micro-batch fills them
            if self.next is None:
                loss = outs[i] / n
                self._loss += loss.detach()
                loss.backward()
            else:
                post_b(i)
                if ahead:
                    post_b(i + 1)
                g, req = brecv.pop(i)
                req.wait()
                outs[i].backward(g)
            if self.prev is not None:
                self._sends.append(self._send(ins[i].grad, self.prev, m.bwd_prev))
            del ins[i], outs[i]

        self._loss.zero_()
        if ahead:
            post_f(0)
            post_b(0)
        warm = n if self.schedule == "gpipe" else min(m.pp - 1 - m.pp_rank, n)
        for i in range(warm):
            forward(i)
        for i in range(n - warm):                            # steady state: one forward, one backward
            forward(warm + i)
            backward(i)
        for i in range(n - warm, n):
            backward(i)
        ddp.hooks_enabled = False

    def _capture(self, tokens, targets, warmup: int = 2) -> None:
        """Capture the forward + backward of a whole step (every micro-batch, the tensor-parallel kernels with
        their collectives inside, the pipeline transfers) into one CUDA graph.  The fused kernels and the
        stream-ordered collectives count their calls on the device, so the captured launches stay valid."""
        dev = self.d.device
        self.ddp.ctx.set_hold_on_wait(False)                 # a replayed step is a handful of host calls (see GraphedStep)
        self._tok = tokens.clone() if tokens is not None else None
        self._tgt = targets.clone() if targets is not None else None
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):                          # allocator, staging areas, point-to-point connections
                self._forward_backward(self._tok, self._tgt, hooks=False)
                for w in self._sends:
                    w.wait()
                self._sends = []
                self._warm = True                            # from the second pass on receives are posted ahead
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.d.barrier()
        self.ddp.zero_grads()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._forward_backward(self._tok, self._tgt, hooks=False)
            for w in self._sends:
                w.wait()
            self._sends = []
        torch.cuda.synchronize(dev)
        self.ddp.zero_grads()

    def step(self, tokens: Optional[torch.Tensor], targets: Optional[torch.Tensor]) -> torch.Tensor:
        """``tokens`` / ``targets``: [n_micro, micro_batch, seq] of this replica (tokens are read by the first
        stage, targets by the last).  Returns the mean loss over all replicas as a 1-element tensor on every rank."""
        ddp = self.ddp
        # Eager steps are thousands of launches: keep the host within one step of the GPU (a host far ahead sits
        # blocked in a launch exactly when the GPU reaches the bucket waits of the step before).
        if self._step_done is not None:
            self._step_done.synchronize()
        if self.use_graph:
            if self._graph is None:
                self._capture(tokens, targets)
            if tokens is not None and self._tok is not None:
                self._tok.copy_(tokens, non_blocking=True)
            if targets is not None and self._tgt is not None:
                self._tgt.copy_(targets, non_blocking=True)
            self._graph.replay()
            ddp.submit_all()
        else:
            self._forward_backward(tokens, targets, hooks=True)
        ddp.finish_backward()
        ddp.step()
        for w in self._sends:
            w.wait()
        self._sends = []
        # mean loss over the replicas: the last-stage ranks hold tensor-parallel shares of their replica's loss
        m = self.mesh
        if self.d.world > 1:
            self._loss.mul_(1.0 / m.dp)
            s = torch.cuda.current_stream(self.d.device).cuda_stream if self.d.device.type == "cuda" else 0
            nv.check(nv.lib().ncclAllReduce(self._loss.data_ptr(), self._loss.data_ptr(), 1, nccl_dtype(torch.float32), nv.SUM,
                                            self.d.comm.handle, s), "ncclAllReduce(loss)")
        if self.d.device.type == "cuda":
            self._step_done = torch.cuda.Event()
            self._step_done.record()
        self._warm = True
        return self._loss

    def state_dict(self):
        """This rank's optimizer state (its shard of the weights in fp32 plus the moments)."""
        return self.ddp.state_dict()

    def load_state_dict(self, state) -> None:
        self.ddp.load_state_dict(state)

    def close(self) -> None:
        self.ddp.close()
