"""Python face of the hand-written tcgen05 GEMM (``csrc/src/gemm/tcgen05_gemm.cu``)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import native as nv

BM, BN, BK = 128, 256, 64


def gemm_supported(m: int, n: int, k: int) -> bool:
    return m > 0 and n > 0 and k > 0 and m % BM == 0 and n % BN == 0 and k % BK == 0


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a @ b.T`` for bf16 ``a [M, K]`` and ``b [N, K]`` (the layout of ``nn.Linear``), computed by
    the library's own tensor-core kernel: TMA-fed shared-memory stages, ``tcgen05.mma`` into tensor
    memory, fp32 accumulation, bf16 result."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and b.is_cuda
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    a, b = a.contiguous(), b.contiguous()
    m, k = a.shape
    n = b.shape[0]
    if not gemm_supported(m, n, k):
        raise ValueError(f"tcgen05 GEMM needs M % {BM} == 0, N % {BN} == 0, K % {BK} == 0, got {m} x {n} x {k}")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    nv.check(nv.lib().dfcclGemmBf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k,
                                    torch.cuda.current_stream(a.device).cuda_stream), "dfcclGemmBf16")
    return out


def matmul(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, *, a_transposed: bool = False,
           b_transposed: bool = False) -> torch.Tensor:
    """``op(a) @ op(b).T`` on the tensor cores, where an operand flagged ``*_transposed`` is *stored* transposed:
    ``a`` as [K, M] and / or ``b`` as [K, N] (row-major, the contraction index slow).  Nothing is copied - the kernel
    describes such an operand to ``tcgen05.mma`` as MN-major.  With both flags this is ``a.T @ b``: the weight gradient
    ``gy.T @ x`` of a linear layer; with ``b_transposed`` alone ``a @ b``: its data gradient ``gy @ W``."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and b.is_cuda and a.dim() == 2 and b.dim() == 2
    a, b = a.contiguous(), b.contiguous()
    k, m = (a.shape if a_transposed else a.shape[::-1])
    kb, n = (b.shape if b_transposed else b.shape[::-1])
    assert k == kb, "contraction lengths differ"
    if not gemm_supported(m, n, k):
        raise ValueError(f"tcgen05 GEMM needs M % {BM} == 0, N % {BN} == 0, K % {BK} == 0, got {m} x {n} x {k}")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    nv.check(nv.lib().dfcclGemmBf16Ex(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, int(a_transposed), int(b_transposed),
                                      torch.cuda.current_stream(a.device).cuda_stream), "dfcclGemmBf16Ex")
    return out


def check_kernels() -> bool:
    """True if no kernel of the GEMM file gave up on a bounded wait since the last check."""
    failed = C.c_int()
    nv.check(nv.lib().dfcclGemmCheck(C.byref(failed)))
    return failed.value == 0
