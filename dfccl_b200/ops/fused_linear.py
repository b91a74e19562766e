"""Tensor-parallel linear layers whose collective runs inside the GEMM kernel.

``AllGatherGemm``   y = all_gather(x_shard) @ W_local^T     (sequence-parallel column-parallel layer)
``GemmReduceScatter`` y_shard = reduce_scatter(x_local @ W_local^T)   (row-parallel layer, sequence-sharded output)

Both drive the fused modes of the tcgen05 GEMM kernel (csrc/src/gemm/tcgen05_gemm.cu): peers' shards are
pulled by communication warps of the GEMM kernel block by block while the tensor cores work on blocks
already present; partial output tiles are stored straight into their owner's memory and reduced there
as they arrive.

When the tensor-parallel group carries a rank context (``TpGroup(..., ctx=...)``) the operators are
*registered* with it under collective ids (``dfcclPrepareFusedGemm``): the context allocates and
exchanges their rendezvous words and receive areas when it is finalized, counts their launches,
reports a wait that ran out through its asynchronous error and keeps its daemon's SMs out of their
grids.  Without a context they own their symmetric-heap buffers themselves and exchange the offsets
over ``torch.distributed`` at construction.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import native as nv
from ..utils.tensors import tensor_from_ptr
from .gemm import BM, BN, BK


class _FusedArgs(C.Structure):
    _fields_ = [
        ("nranks", C.c_int), ("rank", C.c_int), ("rowsPerRank", C.c_int),
        ("peerA", C.c_void_p * 8), ("gathered", C.c_void_p), ("blockReady", C.c_void_p),
        ("slot", C.c_void_p * 8), ("tileFlag", C.c_void_p * 8), ("mySlots", C.c_void_p), ("myTileFlags", C.c_void_p),
        ("reduced", C.c_void_p),
        ("arrive", C.c_void_p), ("done", C.c_void_p), ("peerArrive", C.c_void_p * 8), ("peerDone", C.c_void_p * 8),
        ("doneCount", C.c_void_p), ("epoch", C.c_uint64), ("epochCounter", C.c_void_p), ("mode", C.c_int),
    ]


class TpGroup:
    """A tensor-parallel group: this library's communicator over the group plus the matching
    ``torch.distributed`` group (used only to exchange offsets at construction)."""

    def __init__(self, comm: nv.Comm, pg: Optional["dist.ProcessGroup"], device: torch.device,
                 ctx: Optional[nv.RankCtx] = None, first_id: int = 0):
        """``ctx``: a rank context that is not finalized yet; fused operators of this group register with it under
        consecutive collective ids from ``first_id`` (whoever finalizes the context registers its own collectives
        from ``next_id`` on)."""
        self.comm, self.pg, self.device = comm, pg, device
        self.rank, self.n = comm.rank, comm.nranks
        self.ctx, self.next_id = ctx, first_id
        assert nv.lib().dfcclGemmFusedArgsSize() == C.sizeof(_FusedArgs), "argument block layout mismatch"
        self._base = [comm.peer_base(j) for j in range(self.n)]
        self._mybase = comm.heap_info()[0]

    def take_id(self) -> int:
        i = self.next_id
        self.next_id += 1
        return i

    def alloc(self, nbytes: int, zero: bool = True):
        """Allocate in the symmetric heap; returns (local pointer, [address of every rank's copy as mapped here])."""
        p = self.comm.alloc(max(nbytes, 16))            # heap memory is zeroed on allocation
        off = p - self._mybase
        if self.n > 1:
            offs: List[int] = [0] * self.n
            dist.all_gather_object(offs, off, group=self.pg)
        else:
            offs = [off]
        return p, [self._base[j] + offs[j] for j in range(self.n)]

    def barrier(self):
        if self.n > 1:
            dist.barrier(group=self.pg)


class _Rendezvous:
    def __init__(self, tp: TpGroup):
        n = tp.n
        self.p, peers = tp.alloc(8 * n * 2 + 64)
        self.arrive, self.done = self.p, self.p + 8 * n
        self.peer_arrive = [peers[j] + 8 * tp.rank for j in range(n)]
        self.peer_done = [peers[j] + 8 * n + 8 * tp.rank for j in range(n)]
        self.done_count = torch.zeros(1, dtype=torch.int32, device=tp.device)
        # calls finished so far, counted by the kernel itself: a launch captured in a CUDA graph stays valid on replay
        self.epoch_counter = torch.zeros(1, dtype=torch.int64, device=tp.device)
        self.epoch = 0


class AllGatherGemm:
    """y[M, N] = concat_over_ranks(x_shard)[M, K] @ w[N, K]^T with the all-gather inside the GEMM."""

    def __init__(self, tp: TpGroup, rows_per_rank: int, k: int, n_out: int):
        assert rows_per_rank % BM == 0 and k % BK == 0 and n_out % BN == 0
        self.tp, self.rows, self.k, self.n_out = tp, rows_per_rank, k, n_out
        self.m = rows_per_rank * tp.n
        self.coll_id = None
        if tp.ctx is not None:                          # registered operator: buffers come from the context at finalize
            self.coll_id = tp.take_id()
            tp.ctx.prepare_fused(self.coll_id, tp.comm, nv.FUSED_ALLGATHER_GEMM, rows_per_rank, k, n_out)
            self._gathered = self._shard = None
            return
        gp, peers = tp.alloc(self.m * k * 2)
        self._gathered = tensor_from_ptr(gp, (self.m, k), torch.bfloat16, tp.device)
        self._shard = self._gathered[tp.rank * rows_per_rank:(tp.rank + 1) * rows_per_rank]   # write the input here
        self._peer_shard = [peers[j] + j * rows_per_rank * k * 2 for j in range(tp.n)]
        self.block_ready = torch.zeros(self.m // BM, dtype=torch.int32, device=tp.device)
        self.rv = _Rendezvous(tp)
        self._args = None
        tp.barrier()

    def _bind(self) -> None:
        if self._gathered is None:                      # registered: the context owns the operand (valid once it is finalized)
            sp, gp = self.tp.ctx.fused_operand(self.coll_id)
            self._gathered = tensor_from_ptr(gp, (self.m, self.k), torch.bfloat16, self.tp.device)
            self._shard = self._gathered[self.tp.rank * self.rows:(self.tp.rank + 1) * self.rows]

    @property
    def gathered(self) -> torch.Tensor:
        """The [M, K] operand; complete after a call (the weight gradient reads it)."""
        self._bind()
        return self._gathered

    @property
    def shard(self) -> torch.Tensor:
        """This rank's rows of the operand: writing the input here saves a copy."""
        self._bind()
        return self._shard

    def __call__(self, x_shard: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, w_transposed: bool = False) -> torch.Tensor:
        """``w``: [n_out, k]; with ``w_transposed`` it is given as [k, n_out] and read in place (registered operators)."""
        tp = self.tp
        if out is None:
            out = torch.empty(self.m, self.n_out, dtype=torch.bfloat16, device=tp.device)
        if self.coll_id is not None:
            x_shard, w = x_shard.contiguous(), w.contiguous()
            st = torch.cuda.current_stream(tp.device).cuda_stream if tp.device.type == "cuda" else 0
            tp.ctx.run_fused(self.coll_id, x_shard.data_ptr(), w.data_ptr(), out.data_ptr(), st, w_transposed)
            return out
        if w_transposed:
            w = w.t()
        if x_shard.data_ptr() != self.shard.data_ptr():
            self.shard.copy_(x_shard)
        self.rv.epoch += 1
        a = self._args
        if a is None:                                   # built once: only the epoch changes between calls
            a = self._args = _FusedArgs()
            a.nranks, a.rank, a.rowsPerRank, a.mode = tp.n, tp.rank, self.rows, 1
            for j in range(tp.n):
                a.peerA[j] = self._peer_shard[j]
                a.peerArrive[j] = self.rv.peer_arrive[j]
                a.peerDone[j] = self.rv.peer_done[j]
            a.gathered, a.blockReady = self.gathered.data_ptr(), self.block_ready.data_ptr()
            a.arrive, a.done, a.doneCount = self.rv.arrive, self.rv.done, self.rv.done_count.data_ptr()
            a.epochCounter = self.rv.epoch_counter.data_ptr()
            self._fn, self._sz, self._gp = nv.lib().dfcclGemmFused, C.sizeof(a), self.gathered.data_ptr()
        a.epoch = self.rv.epoch
        w = w.contiguous()
        nv.check(nv.lib().dfcclGemmFused(self.gathered.data_ptr(), w.data_ptr(), out.data_ptr(), self.m, self.n_out, self.k,
                                         C.byref(a), C.sizeof(a), torch.cuda.current_stream(tp.device).cuda_stream), "dfcclGemmFused(ag)")
        return out


class GemmReduceScatter:
    """y_shard[M/n, N] = sum_over_ranks(x[M, K_local] @ w[N, K_local]^T)[my rows] with the reduce-scatter
    inside the GEMM: the epilogue stores partial tiles into their owner's memory, the owner sums them."""

    def __init__(self, tp: TpGroup, m: int, k_local: int, n_out: int):
        assert m % (BM * tp.n) == 0 and k_local % BK == 0 and n_out % BN == 0
        self.tp, self.m, self.k, self.n_out = tp, m, k_local, n_out
        self.rows = m // tp.n
        self.tiles_mine = (self.rows // BM) * (n_out // BN)
        self.coll_id = None
        if tp.ctx is not None:
            self.coll_id = tp.take_id()
            tp.ctx.prepare_fused(self.coll_id, tp.comm, nv.FUSED_GEMM_REDUCESCATTER, self.rows, k_local, n_out)
            return
        sp, speers = tp.alloc(tp.n * self.rows * n_out * 2)
        fp, fpeers = tp.alloc(tp.n * self.tiles_mine * 4)
        self._slots, self._flags = sp, fp
        # where MY partial tiles go in owner j's memory: its slot number tp.rank
        self._slot_at = [speers[j] + tp.rank * self.rows * n_out * 2 for j in range(tp.n)]
        self._flag_at = list(fpeers)
        self.rv = _Rendezvous(tp)
        self._dummy = torch.empty(16, dtype=torch.bfloat16, device=tp.device)
        self._args = None
        tp.barrier()

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, w_transposed: bool = False) -> torch.Tensor:
        tp = self.tp
        if w_transposed and self.coll_id is None:
            w, w_transposed = w.t(), False
        x, w = x.contiguous(), w.contiguous()
        if out is None:
            out = torch.empty(self.rows, self.n_out, dtype=torch.bfloat16, device=tp.device)
        if self.coll_id is not None:
            st = torch.cuda.current_stream(tp.device).cuda_stream if tp.device.type == "cuda" else 0
            tp.ctx.run_fused(self.coll_id, x.data_ptr(), w.data_ptr(), out.data_ptr(), st, w_transposed)
            return out
        if tp.n == 1:
            nv.check(nv.lib().dfcclGemmBf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), self.m, self.n_out, self.k,
                                            torch.cuda.current_stream(tp.device).cuda_stream), "dfcclGemmBf16")
            return out
        self.rv.epoch += 1
        a = self._args
        if a is None:
            a = self._args = _FusedArgs()
            a.nranks, a.rank, a.rowsPerRank, a.mode = tp.n, tp.rank, self.rows, 2
            for j in range(tp.n):
                a.slot[j] = self._slot_at[j]
                a.tileFlag[j] = self._flag_at[j]
                a.peerArrive[j] = self.rv.peer_arrive[j]
                a.peerDone[j] = self.rv.peer_done[j]
            a.mySlots, a.myTileFlags = self._slots, self._flags
            a.arrive, a.done, a.doneCount = self.rv.arrive, self.rv.done, self.rv.done_count.data_ptr()
            a.epochCounter = self.rv.epoch_counter.data_ptr()
        a.epoch, a.reduced = self.rv.epoch, out.data_ptr()
        nv.check(nv.lib().dfcclGemmFused(x.data_ptr(), w.data_ptr(), self._dummy.data_ptr(), self.m, self.n_out, self.k,
                                         C.byref(a), C.sizeof(a), torch.cuda.current_stream(tp.device).cuda_stream), "dfcclGemmFused(rs)")
        return out
