"""Tensor parallelism with sequence-parallel activations (Megatron style) on top of this library.

Forward passes run the fused kernels: the column-parallel layer is an all-gather -> GEMM, the
row-parallel layer a GEMM -> reduce-scatter, both one tcgen05 kernel each with the collective
inside (``dfccl_b200.ops.fused_linear``).  The data-gradient GEMMs of the backward passes are the same
two kernels with the roles swapped (the column-parallel layer's is a GEMM -> reduce-scatter, the
row-parallel layer's an all-gather -> GEMM, each on the transposed weight); the weight-gradient
GEMMs contract over the token dimension and stay on cuBLAS.  On the host backend (tests) the layers
fall back to this library's stream-ordered collectives around plain GEMMs.

The reference has no tensor-parallel code; its simulator only generates the group structure of
such jobs (reference: simulator/simulator.py:434-493).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import native as nv
from ..ops.fused_linear import AllGatherGemm, GemmReduceScatter, TpGroup
from ..utils.tensors import nccl_dtype


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream if t.device.type == "cuda" else 0


_OPS: Dict[Tuple, object] = {}


def shared_op(kind, tp: TpGroup, *shape):
    """Layers of the same shape share one fused operator (its heap buffers and rendezvous words):
    calls on one stream are ordered, and the operator's own done-handshake keeps a peer from
    overwriting what another still reads."""
    key = (kind.__name__, id(tp)) + tuple(shape)
    if key not in _OPS:
        _OPS[key] = kind(tp, *shape)
    return _OPS[key]


def _fused(tp: TpGroup) -> bool:
    """Fused kernels on GPUs; collective + plain GEMM on the host backend (tests) and on the comparison arm."""
    return tp.device.type == "cuda" and getattr(tp, "library", "dfccl") == "dfccl"


def _wgrad(gy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """gy^T @ x (the weight gradient: a contraction over the token dimension).  Both operands are stored with the
    contraction index slow, which the tcgen05 kernel reads in place as MN-major operands; shapes it cannot tile go
    to ``torch.matmul``."""
    from ..ops import gemm
    if gy.is_cuda and gemm.gemm_supported(gy.shape[1], x.shape[1], gy.shape[0]):
        return gemm.matmul(gy, x, a_transposed=True, b_transposed=True)
    return gy.t() @ x


def tp_all_gather(tp: TpGroup, x: torch.Tensor) -> torch.Tensor:
    """Concatenate the ranks' tensors along dim 0 with this library's stream-ordered all-gather."""
    if tp.n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] * tp.n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if getattr(tp, "library", "dfccl") == "torch":         # comparison arm: the collective library behind torch.distributed
        dist.all_gather_into_tensor(out, x, group=tp.pg)
        return out
    nv.check(nv.lib().ncclAllGather(x.data_ptr(), out.data_ptr(), x.numel(), nccl_dtype(x.dtype), tp.comm.handle,
                                    _stream(x)), "ncclAllGather")
    return out


def tp_reduce_scatter(tp: TpGroup, x: torch.Tensor) -> torch.Tensor:
    """Sum over ranks, keep this rank's block of dim 0."""
    if tp.n == 1:
        return x
    x = x.contiguous()
    rows = x.shape[0] // tp.n
    out = torch.empty((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if getattr(tp, "library", "dfccl") == "torch":
        dist.reduce_scatter_tensor(out, x, group=tp.pg)
        return out
    nv.check(nv.lib().ncclReduceScatter(x.data_ptr(), out.data_ptr(), out.numel(), nccl_dtype(x.dtype), nv.SUM, tp.comm.handle,
                                        _stream(x)), "ncclReduceScatter")
    return out


class _ColumnFn(torch.autograd.Function):
    """y = all_gather(x_shard) W^T.  Backward: gW = gy^T x_full, gx_shard = reduce_scatter(gy W)."""

    @staticmethod
    def forward(ctx, x_shard, weight, layer):
        ctx.layer = layer
        if layer.op is None:                                # host backend (tests) / comparison arm: collective + plain GEMM
            ctx.save_for_backward(x_shard, weight)
            return tp_all_gather(layer.tp, x_shard) @ weight.t()
        y = layer.op(x_shard, weight)
        # the gathered activations are needed again for the weight gradient: keep a copy (the operator's buffer
        # is shared by every layer of this shape) instead of gathering a second time in the backward pass
        ctx.save_for_backward(layer.op.gathered.clone(), weight)
        return y

    @staticmethod
    def backward(ctx, gy):
        saved, weight = ctx.saved_tensors
        layer = ctx.layer
        tp = layer.tp
        gy = gy.contiguous()
        if layer.op is None:
            x_full = tp_all_gather(tp, saved)
            return tp_reduce_scatter(tp, gy @ weight), gy.t() @ x_full, None
        gw = _wgrad(gy, saved)
        # data gradient with the reduce-scatter inside the GEMM: gx = RS(gy [M, N/n] @ W [N/n, K]); the B operand is W^T,
        # handed over as W itself (stored [contraction, output]: read in place as an MN-major operand)
        gx = layer.bwd_op(gy, weight, w_transposed=True)
        return gx, gw, None


class _RowFn(torch.autograd.Function):
    """y_shard = reduce_scatter(x W^T).  Backward: gy = all_gather(gy_shard), gx = gy W, gW = gy^T x."""

    @staticmethod
    def forward(ctx, x, weight, layer):
        ctx.layer = layer
        ctx.save_for_backward(x, weight)
        if layer.op is None:
            return tp_reduce_scatter(layer.tp, x @ weight.t())
        return layer.op(x, weight)

    @staticmethod
    def backward(ctx, gy_shard):
        x, weight = ctx.saved_tensors
        layer = ctx.layer
        gy_shard = gy_shard.contiguous()
        if layer.op is None:
            gy = tp_all_gather(layer.tp, gy_shard)
            return gy @ weight, gy.t() @ x, None
        # data gradient with the all-gather inside the GEMM: gx = AG(gy_shard) [M, N] @ W [N, K/n], B operand = W^T;
        # the operator's gathered buffer then holds the full output gradient for the weight gradient
        gx = layer.bwd_op(gy_shard, weight, w_transposed=True)
        gw = _wgrad(layer.bwd_op.gathered, x)
        return gx, gw, None


class ColumnParallelLinear(nn.Module):
    """y[M, N/n] = all_gather(x_shard)[M, K] W_local^T + b_local.  Input is sequence-sharded, output is
    feature-sharded."""

    def __init__(self, tp: TpGroup, rows_per_rank: int, full_weight: torch.Tensor, parts: int = 1):
        """``full_weight`` [out, in] is the unsharded weight (identical on every rank); this rank keeps rows
        ``rank`` of each of its ``parts`` equal row groups (3 for a fused q/k/v projection)."""
        super().__init__()
        out_features, in_features = full_weight.shape
        assert out_features % (tp.n * parts) == 0
        self.tp = tp
        nl = out_features // tp.n
        w = full_weight.view(parts, tp.n, out_features // (parts * tp.n), in_features)[:, tp.rank]
        self.weight = nn.Parameter(w.reshape(nl, in_features).to(torch.bfloat16).contiguous())
        self.bias = nn.Parameter(torch.zeros(nl, dtype=torch.bfloat16, device=tp.device))
        self.op = shared_op(AllGatherGemm, tp, rows_per_rank, in_features, nl) if _fused(tp) else None
        self.bwd_op = shared_op(GemmReduceScatter, tp, rows_per_rank * tp.n, nl, in_features) if _fused(tp) else None

    def forward(self, x_shard):
        return _ColumnFn.apply(x_shard, self.weight, self) + self.bias


class RowParallelLinear(nn.Module):
    """y_shard[M/n, N] = reduce_scatter(x[M, K/n] W_local^T) + b.  Input is feature-sharded, output is
    sequence-sharded.  The bias is replicated (its gradient is summed over the group by the caller)."""

    def __init__(self, tp: TpGroup, m: int, full_weight: torch.Tensor):
        super().__init__()
        out_features, in_features = full_weight.shape
        assert in_features % tp.n == 0
        self.tp = tp
        kl = in_features // tp.n
        self.weight = nn.Parameter(full_weight[:, tp.rank * kl:(tp.rank + 1) * kl].to(torch.bfloat16).contiguous())
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=torch.bfloat16, device=tp.device))
        self.bias.tp_replicated = True
        self.op = shared_op(GemmReduceScatter, tp, m, kl, out_features) if _fused(tp) else None
        self.bwd_op = shared_op(AllGatherGemm, tp, m // tp.n, out_features, kl) if _fused(tp) else None

    def forward(self, x):
        return _RowFn.apply(x, self.weight, self) + self.bias
