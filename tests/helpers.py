"""Shared helpers for tests that drive several ranks from one process."""
import ctypes as C
import threading
import traceback

import numpy as np

NP_OF = None


def np_dtype(nv, dt):
    table = {nv.INT8: np.int8, nv.UINT8: np.uint8, nv.INT32: np.int32, nv.UINT32: np.uint32, nv.INT64: np.int64,
             nv.UINT64: np.uint64, nv.FLOAT16: np.float16, nv.FLOAT32: np.float32, nv.FLOAT64: np.float64,
             nv.BFLOAT16: np.uint16}
    return table[dt]


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even conversion of float32 to bfloat16 bit patterns."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    rounded = u + 0x7FFF + ((u >> 16) & 1)
    return (rounded >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def host_array(ptr: int, count: int, dtype) -> np.ndarray:
    """numpy view of `count` elements at a raw address (host-backend heap memory)."""
    dt = np.dtype(dtype)
    buf = (C.c_char * (count * dt.itemsize)).from_address(ptr)
    return np.frombuffer(buf, dtype=dt, count=count)


def run_ranks(n, fn, timeout=120):
    """Run fn(rank) on n threads; re-raise the first failure with its traceback."""
    errors = []

    def wrap(r):
        try:
            fn(r)
        except BaseException:
            errors.append((r, traceback.format_exc()))

    ts = [threading.Thread(target=wrap, args=(r,), daemon=True) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout)
    alive = [i for i, t in enumerate(ts) if t.is_alive()]
    if errors:
        raise AssertionError("rank %d failed:\n%s" % errors[0])
    if alive:
        raise AssertionError(f"ranks {alive} did not finish within {timeout}s")
