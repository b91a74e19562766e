"""Stream-ordered collectives of this library on torch tensors.

Thin functional layer over the ``nccl*`` entry points (csrc/src/api/nccl_api.cu): the kernels run on the
current CUDA stream (or synchronously on the host backend), tensors that live in the communicator's
symmetric heap (:class:`dfccl_b200.utils.HeapTensorPool`) are used in place, any other tensor is staged by
the library.  These are the calls the tensor-parallel backward passes use; for collectives that must be
safe under per-rank disordered issue, register them with a :class:`dfccl_b200.native.RankCtx` instead.

Counterpart of the reference's stock entry points (reference: src/collectives/all_reduce.cc:9-16 and
its siblings for the other kinds).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import native as nv
from ..utils.tensors import nccl_dtype

_OPS = {"sum": nv.SUM, "prod": nv.PROD, "max": nv.MAX, "min": nv.MIN, "avg": nv.AVG}


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream if t.device.type == "cuda" else None


def _check(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def all_reduce(comm: nv.Comm, x: torch.Tensor, out: Optional[torch.Tensor] = None, op: str = "sum") -> torch.Tensor:
    """``out = reduce over ranks of x`` (in place when ``out`` is omitted)."""
    out = x if out is None else out
    _check(x, "x"), _check(out, "out")
    nv.check(nv.lib().ncclAllReduce(x.data_ptr(), out.data_ptr(), x.numel(), nccl_dtype(x.dtype), _OPS[op], comm.handle, _stream(x)), "ncclAllReduce")
    return out


def all_gather(comm: nv.Comm, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Concatenation of every rank's ``x`` along dim 0."""
    _check(x, "x")
    if out is None:
        out = torch.empty((x.shape[0] * comm.nranks,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    nv.check(nv.lib().ncclAllGather(x.data_ptr(), _check(out, "out").data_ptr(), x.numel(), nccl_dtype(x.dtype), comm.handle, _stream(x)), "ncclAllGather")
    return out


def reduce_scatter(comm: nv.Comm, x: torch.Tensor, out: Optional[torch.Tensor] = None, op: str = "sum") -> torch.Tensor:
    """Reduce over ranks, keep block ``rank`` of dim 0."""
    _check(x, "x")
    if x.shape[0] % comm.nranks:
        raise ValueError("dim 0 must divide by the number of ranks")
    if out is None:
        out = torch.empty((x.shape[0] // comm.nranks,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    nv.check(nv.lib().ncclReduceScatter(x.data_ptr(), _check(out, "out").data_ptr(), out.numel(), nccl_dtype(x.dtype), _OPS[op], comm.handle, _stream(x)), "ncclReduceScatter")
    return out


def broadcast(comm: nv.Comm, x: torch.Tensor, root: int = 0) -> torch.Tensor:
    """Overwrite ``x`` on every rank with the root's."""
    _check(x, "x")
    nv.check(nv.lib().ncclBroadcast(x.data_ptr(), x.data_ptr(), x.numel(), nccl_dtype(x.dtype), root, comm.handle, _stream(x)), "ncclBroadcast")
    return x


def reduce(comm: nv.Comm, x: torch.Tensor, root: int = 0, out: Optional[torch.Tensor] = None, op: str = "sum") -> Optional[torch.Tensor]:
    """Reduction over ranks delivered to ``root`` (``out`` is only written there)."""
    _check(x, "x")
    if out is None and comm.rank == root:
        out = torch.empty_like(x)
    nv.check(nv.lib().ncclReduce(x.data_ptr(), out.data_ptr() if out is not None else None, x.numel(), nccl_dtype(x.dtype), _OPS[op], root, comm.handle, _stream(x)), "ncclReduce")
    return out
