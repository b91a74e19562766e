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

Schedule: all micro-batches forward, then all backward (GPipe), gradients accumulated in the flat
buckets; the buckets are released to the daemon from the gradient hooks of the last micro-batch.
"""
from __future__ import annotations

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

    def close(self) -> None:
        for c in (self.tp_group.comm, self.dp_comm, self.stage_comm):
            c.destroy()


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
    return Mesh(tp, pp, dp, tp_rank, pp_rank, dp_rank, TpGroup(tp_comm, pg, d.device), dp_comm, stage_comm)


class HybridTrainer:
    """One optimizer step = ``n_micro`` micro-batches of ``micro_batch`` sequences per replica."""

    def __init__(self, d: Dist, mesh: Mesh, stage: torch.nn.Module, *, n_micro: int, bucket_mb: float = 25.0, lr: float = 0.01,
                 momentum: float = 0.9, weight_decay: float = 0.0, seed: int = 0, daemon_blocks: int = 8, use_graph: bool = False,
                 optimizer: str = "sgd"):
        self.d, self.mesh, self.stage, self.n_micro = d, mesh, stage, n_micro
        params = [p for p in stage.parameters() if p.requires_grad]
        sharded = [p for p in params if not getattr(p, "tp_replicated", False)]
        replicated = [p for p in params if getattr(p, "tp_replicated", False)]
        groups = [{"params": sharded, "comm": mesh.dp_comm, "scale": 1.0 / mesh.dp},
                  {"params": replicated, "comm": mesh.stage_comm, "scale": 1.0 / mesh.dp}]
        self.ddp = DaemonDDP(stage, d, bucket_mb=bucket_mb, lr=lr, momentum=momentum, weight_decay=weight_decay,
                             randomize_order=True, seed=seed, param_groups=groups, daemon_blocks=daemon_blocks, optimizer=optimizer)
        self.ddp.hooks_enabled = False
        if d.device.type == "cuda":
            # the fused GEMM launches need all their CTAs resident together: keep them off the SMs a daemon
            # instance may still hold when the next forward pass starts
            nv.check(nv.lib().dfcclGemmReserveSms(daemon_blocks), "dfcclGemmReserveSms")
        self.prev = d.rank - mesh.tp if mesh.pp_rank > 0 else None
        self.next = d.rank + mesh.tp if mesh.pp_rank < mesh.pp - 1 else None
        self._loss = torch.zeros(1, dtype=torch.float32, device=d.device)
        self.pp_bytes = 0
        self._step_done = None
        self._sends: list = []
        self.use_graph = bool(use_graph) and d.device.type == "cuda"
        self._graph = None
        self._tok = self._tgt = None

    def _hidden(self) -> torch.Tensor:
        st = self.stage
        return torch.empty(st.rows, st.cfg.d_model, dtype=torch.bfloat16, device=self.d.device)

    def _send(self, t: torch.Tensor, dst: int):
        self.pp_bytes += t.numel() * t.element_size()
        return dist.isend(t.contiguous(), dst)

    def _forward_backward(self, tokens, targets, hooks: bool) -> None:
        """All micro-batches forward, then all backward; the loss shares accumulate in ``self._loss``."""
        st, n, ddp = self.stage, self.n_micro, self.ddp
        ins: List[torch.Tensor] = []
        outs: List[torch.Tensor] = []
        for i in range(n):                                   # ---- forward
            if self.prev is None:
                x = tokens[i]
            else:
                x = self._hidden()
                dist.irecv(x, self.prev).wait()
                x.requires_grad_(True)
            y = st(x, targets[i] if self.next is None else None)
            if self.next is not None:
                self._sends.append(self._send(y.detach(), self.next))
            ins.append(x)
            outs.append(y)
        self._loss.zero_()
        for i in range(n):                                   # ---- backward
            ddp.hooks_enabled = hooks and i == n - 1         # buckets go to the daemon as the last micro-batch fills them
            if self.next is None:
                loss = outs[i] / n
                self._loss += loss.detach()
                loss.backward()
            else:
                g = self._hidden()
                dist.irecv(g, self.next).wait()
                outs[i].backward(g)
            if self.prev is not None:
                self._sends.append(self._send(ins[i].grad, self.prev))
            ins[i] = outs[i] = None
        ddp.hooks_enabled = False

    def _capture(self, tokens, targets, warmup: int = 2) -> None:
        """Capture the forward + backward of a whole step (every micro-batch, the tensor-parallel kernels with
        their collectives inside, the pipeline transfers) into one CUDA graph.  The fused kernels and the
        stream-ordered collectives count their calls on the device, so the captured launches stay valid."""
        dev = self.d.device
        if hasattr(self.ddp, "ctx"):
            self.ddp.ctx.set_hold_on_wait(False)             # a replayed step is a handful of host calls (see GraphedStep)
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
        return self._loss

    def close(self) -> None:
        for c in (self.tp_group.comm, self.dp_comm, self.stage_comm):
            c.destroy()


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
    return Mesh(tp, pp, dp, tp_rank, pp_rank, dp_rank, TpGroup(tp_comm, pg, d.device), dp_comm, stage_comm)


class HybridTrainer:
    """One optimizer step = ``n_micro`` micro-batches of ``micro_batch`` sequences per replica."""

    def __init__(self, d: Dist, mesh: Mesh, stage: torch.nn.Module, *, n_micro: int, bucket_mb: float = 25.0, lr: float = 0.01,
                 momentum: float = 0.9, weight_decay: float = 0.0, seed: int = 0, daemon_blocks: int = 8, use_graph: bool = False,
                 optimizer: str = "sgd"):
        self.d, self.mesh, self.stage, self.n_micro = d, mesh, stage, n_micro
        params = [p for p in stage.parameters() if p.requires_grad]
        sharded = [p for p in params if not getattr(p, "tp_replicated", False)]
        replicated = [p for p in params if getattr(p, "tp_replicated", False)]
        groups = [{"params": sharded, "comm": mesh.dp_comm, "scale": 1.0 / mesh.dp},
                  {"params": replicated, "comm": mesh.stage_comm, "scale": 1.0 / mesh.dp}]
        self.ddp = DaemonDDP(stage, d, bucket_mb=bucket_mb, lr=lr, momentum=momentum, weight_decay=weight_decay,
                             randomize_order=True, seed=seed, param_groups=groups, daemon_blocks=daemon_blocks, optimizer=optimizer)
        self.ddp.hooks_enabled = False
        if d.device.type == "cuda":
            # the fused GEMM launches need all their CTAs resident together: keep them off the SMs a daemon
            # instance may still hold when the next forward pass starts
            nv.check(nv.lib().dfcclGemmReserveSms(daemon_blocks), "dfcclGemmReserveSms")
        self.prev = d.rank - mesh.tp if mesh.pp_rank > 0 else None
        self.next = d.rank + mesh.tp if mesh.pp_rank < mesh.pp - 1 else None
        self._loss = torch.zeros(1, dtype=torch.float32, device=d.device)
        self.pp_bytes = 0
        self._step_done = None
        self._sends: list = []
        self.use_graph = bool(use_graph) and d.device.type == "cuda"
        self._graph = None
        self._tok = self._tgt = None

    def _hidden(self) -> torch.Tensor:
        st = self.stage
        return torch.empty(st.rows, st.cfg.d_model, dtype=torch.bfloat16, device=self.d.device)

    def _send(self, t: torch.Tensor, dst: int):
        self.pp_bytes += t.numel() * t.element_size()
        return dist.isend(t.contiguous(), dst)

    def step(self, tokens: Optional[torch.Tensor], targets: Optional[torch.Tensor]) -> torch.Tensor:
        """``tokens`` / ``targets``: [n_micro, micro_batch, seq] of this replica (tokens are read by the first
        stage, targets by the last).  Returns the mean loss over all replicas as a 1-element tensor on every rank."""
        st, n, ddp = self.stage, self.n_micro, self.ddp
        # Eager steps are thousands of launches: a host that runs a whole step ahead sits blocked in a launch
        # (queue full) exactly when the GPU reaches the bucket waits of the previous step, and the daemon's
        # relaunch from its observer thread then queues behind that blocked launch.  Keeping the host within
        # one step of the GPU costs nothing at these step times and removes the dependency.
        if self._step_done is not None:
            self._step_done.synchronize()
        ins: List[torch.Tensor] = []
        outs: List[torch.Tensor] = []
        sends = []
        for i in range(n):                                   # ---- forward
            if self.prev is None:
                x = tokens[i]
            else:
                x = self._hidden()
                dist.irecv(x, self.prev).wait()
                x.requires_grad_(True)
            y = st(x, targets[i] if self.next is None else None)
            if self.next is not None:
                sends.append(self._send(y.detach(), self.next))
            ins.append(x)
            outs.append(y)
        self._loss.zero_()
        for i in range(n):                                   # ---- backward
            ddp.hooks_enabled = i == n - 1                   # buckets go to the daemon as the last micro-batch fills them
            if self.next is None:
                loss = outs[i] / n
                self._loss += loss.detach()
                loss.backward()
            else:
                g = self._hidden()
                dist.irecv(g, self.next).wait()
                outs[i].backward(g)
            if self.prev is not None:
                sends.append(self._send(ins[i].grad, self.prev))
            ins[i] = outs[i] = None
        ddp.hooks_enabled = False
        ddp.finish_backward()
        ddp.step()
        for w in sends:
            w.wait()
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
        return self._loss

    def state_dict(self):
        """This rank's optimizer state (its shard of the weights in fp32 plus the moments)."""
        return self.ddp.state_dict()

    def load_state_dict(self, state) -> None:
        self.ddp.load_state_dict(state)

    def close(self) -> None:
        self.ddp.close()
