"""Views of symmetric-heap memory as torch tensors (no copy, no ownership)."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np
import torch

from .. import native as nv

_TORCH_TO_NCCL = {
    torch.int8: nv.INT8, torch.uint8: nv.UINT8, torch.int32: nv.INT32, torch.int64: nv.INT64,
    torch.float16: nv.FLOAT16, torch.float32: nv.FLOAT32, torch.float64: nv.FLOAT64, torch.bfloat16: nv.BFLOAT16,
}


def nccl_dtype(dt: torch.dtype) -> int:
    try:
        return _TORCH_TO_NCCL[dt]
    except KeyError:
        raise TypeError(f"{dt} has no collective datatype") from None


class _CudaBlob:
    """Minimal ``__cuda_array_interface__`` provider for a raw device range."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr: int, shape: Sequence[int], dtype: torch.dtype, device) -> torch.Tensor:
    """Tensor over ``prod(shape)`` elements of ``dtype`` starting at device (or host) address ``ptr``.
    The memory stays owned by the heap; the caller keeps it alive."""
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    device = torch.device(device)
    if device.type == "cuda":
        raw = torch.as_tensor(_CudaBlob(ptr, max(nbytes, 1)), device=device)
    else:
        buf = (C.c_uint8 * max(nbytes, 1)).from_address(ptr)
        raw = torch.from_numpy(np.frombuffer(buf, dtype=np.uint8))
    return raw[:nbytes].view(dtype).view(*shape)


class HeapTensorPool:
    """Allocates tensors from a communicator's symmetric heap and frees them together."""

    def __init__(self, comm: nv.Comm, device):
        self.comm, self.device, self._ptrs = comm, torch.device(device), []

    def empty(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(1, n * torch.empty((), dtype=dtype).element_size())
        p = self.comm.alloc(nbytes)
        self._ptrs.append(p)
        return tensor_from_ptr(p, shape, dtype, self.device)

    def zeros(self, shape, dtype):
        return self.empty(shape, dtype).zero_()

    def release(self):
        for p in self._ptrs:
            self.comm.free(p)
        self._ptrs.clear()
