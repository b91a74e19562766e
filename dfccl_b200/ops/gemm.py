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


def check_kernels() -> bool:
    """True if no kernel of the GEMM file gave up on a bounded wait since the last check."""
    failed = C.c_int()
    nv.check(nv.lib().dfcclGemmCheck(C.byref(failed)))
    return failed.value == 0
