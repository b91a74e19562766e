"""ctypes binding of ``libdfccl.so`` (the C interface declared in
``csrc/include/dfccl.h``) plus small Python conveniences.

The library is built in-tree on first use if it is missing (``_build.build``).
On a machine with a GPU the CUDA backend is the default and a missing or
unloadable library is an error, never a silent fallback to Python code.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Callable, Dict, List, Optional, Sequence

from . import _build

# ---- enums (values of dfccl.h)
SUCCESS, UNHANDLED_CUDA, SYSTEM_ERROR, INTERNAL_ERROR, INVALID_ARGUMENT, INVALID_USAGE, TIMEOUT, ABORTED = range(8)
SUM, PROD, MAX, MIN, AVG = range(5)
INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, BFLOAT16 = range(10)
ALLREDUCE, ALLGATHER, REDUCESCATTER, BROADCAST, REDUCE = range(5)
ALGO_AUTO, ALGO_ONESHOT, ALGO_TWOSHOT, ALGO_NVLS, ALGO_PUSH = range(5)
BACKEND_CUDA, BACKEND_HOST = 0, 1
COLL_ARENA_BUFFERS = 1
FAULT_NONE, FAULT_DROP_SQE, FAULT_DELAY_SQE_US, FAULT_FREEZE_POLLER = range(4)

DTYPE_SIZE = {INT8: 1, UINT8: 1, INT32: 4, UINT32: 4, INT64: 8, UINT64: 8, FLOAT16: 2, FLOAT32: 4, FLOAT64: 8, BFLOAT16: 2}

CALLBACK = C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p)


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


class CollInfo(C.Structure):
    _fields_ = [("kind", C.c_int), ("count", C.c_size_t), ("inType", C.c_int), ("outType", C.c_int),
                ("op", C.c_int), ("root", C.c_int), ("scale", C.c_float), ("algo", C.c_int), ("nBlocks", C.c_int), ("flags", C.c_int)]


class FusedInfo(C.Structure):
    _fields_ = [("kind", C.c_int), ("rowsPerRank", C.c_int), ("k", C.c_int), ("n", C.c_int)]


FUSED_ALLGATHER_GEMM, FUSED_GEMM_REDUCESCATTER = 1, 2


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "sqesSubmitted", "cqesDelivered", "callbacksRun", "daemonLaunches", "daemonVoluntaryQuits",
        "ctxSwitches", "ctxSaves", "ctxLoads", "waitPolls", "waitTimeouts", "bytesReduced", "bytesCopied",
        "sqFullRetries", "maxSwitchNs", "totalSwitchNs", "deviceEvents", "dataYields", "schedulerPasses",
        "nsTriggers", "nsWalk", "nsQueues", "fusedLaunches")]

    def as_dict(self) -> Dict[str, int]:
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class DfcclError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(f"{what}: {error_string(code)} ({code})")


_lib = None
_lock = threading.Lock()


def lib() -> C.CDLL:
    """Load (building first if necessary) and return the native library."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB
        if os.environ.get("DFCCL_LIBRARY"):             # e.g. a sanitizer build (see _build.build(sanitize=...))
            path = type(path)(os.environ["DFCCL_LIBRARY"])
        elif not path.exists() or os.environ.get("DFCCL_REBUILD") == "1":
            path = _build.build()
        L = C.CDLL(str(path))       # local scope: the nccl* names must not shadow another collective library's
        vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
        sig = {
            "ncclGetVersion": [C.POINTER(i)],
            "ncclGetUniqueId": [C.POINTER(UniqueId)],
            "ncclCommInitRank": [C.POINTER(vp), i, UniqueId, i],
            "ncclCommInitAll": [C.POINTER(vp), i, C.POINTER(i)],
            "dfcclCommInitLoopback": [C.POINTER(vp), i, i],
            "dfcclCommSplit": [vp, i, i, C.POINTER(vp)],
            "ncclCommDestroy": [vp], "ncclCommAbort": [vp],
            "ncclCommGetAsyncError": [vp, C.POINTER(i)],
            "ncclCommCount": [vp, C.POINTER(i)], "ncclCommCuDevice": [vp, C.POINTER(i)], "ncclCommUserRank": [vp, C.POINTER(i)],
            "ncclRedOpCreatePreMulSum": [C.POINTER(i), vp, i, i, vp], "ncclRedOpDestroy": [i, vp],
            "ncclAllReduce": [vp, vp, sz, i, i, vp, vp],
            "ncclReduce": [vp, vp, sz, i, i, i, vp, vp],
            "ncclBroadcast": [vp, vp, sz, i, i, vp, vp],
            "ncclBcast": [vp, sz, i, i, vp, vp],
            "ncclReduceScatter": [vp, vp, sz, i, i, vp, vp],
            "ncclAllGather": [vp, vp, sz, i, vp, vp],
            "ncclSend": [vp, sz, i, i, vp, vp], "ncclRecv": [vp, sz, i, i, vp, vp],
            "ncclGroupStart": [], "ncclGroupEnd": [],
            "dfcclSetBackend": [i], "dfcclGetBackend": [C.POINTER(i)],
            "dfcclMemAlloc": [C.POINTER(vp), sz, vp], "dfcclMemFree": [vp, vp],
            "dfcclHeapInfo": [vp, C.POINTER(vp), C.POINTER(sz), C.POINTER(sz)],
            "dfcclNvlsInit": [vp, sz, C.POINTER(i)], "dfcclNvlsAlloc": [C.POINTER(vp), sz, vp],
            "dfcclNvlsInfo": [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(sz), C.POINTER(sz)],
            "ofcclInitRankCtx": [C.POINTER(vp), i], "dfcclInitRankCtxOnDevice": [C.POINTER(vp), i, i],
            "ofcclFinalizeRankCtx7StartHostThrds": [vp], "ofcclPrepareDone": [vp], "ofcclDestroy": [vp],
            "dfcclPrepare": [C.POINTER(CollInfo), vp, i, vp],
            "ofcclPrepareAllReduce": [sz, i, i, vp, i, vp], "ofcclPrepareReduce": [sz, i, i, i, vp, i, vp],
            "ofcclPrepareReduceScatter": [sz, i, i, vp, i, vp], "ofcclPrepareAllGather": [sz, i, vp, i, vp],
            "ofcclPrepareBroadcast": [sz, i, i, vp, i, vp], "ofcclPrepareBcast": [sz, i, i, vp, i, vp],
            "ofcclRunAllReduce": [vp, vp, i, CALLBACK, vp, vp], "ofcclRunReduce": [vp, vp, i, CALLBACK, vp, vp],
            "ofcclRunReduceScatter": [vp, vp, i, CALLBACK, vp, vp], "ofcclRunAllGather": [vp, vp, i, CALLBACK, vp, vp],
            "ofcclRunBroadcast": [vp, vp, i, CALLBACK, vp, vp], "ofcclRunBcast": [vp, i, CALLBACK, vp, vp],
            "dfcclPrepareFusedGemm": [C.POINTER(FusedInfo), vp, i, vp], "dfcclFusedGemmOperand": [i, vp, C.POINTER(vp), C.POINTER(vp)],
            "dfcclRunFusedGemm": [i, vp, vp, vp, vp, vp], "dfcclRunFusedGemmT": [i, vp, vp, vp, vp, vp],
            "dfcclRun": [vp, vp, i, CALLBACK, vp, vp],
            "dfcclRunOnStream": [vp, vp, i, vp, CALLBACK, vp, vp],
            "dfcclRunDeferred": [vp, vp, i, CALLBACK, vp, vp], "dfcclTriggerOnStream": [i, vp, vp],
            "dfcclStreamWait": [i, vp, vp], "dfcclWait": [i, i, vp], "dfcclWaitAll": [i, vp],
            "dfcclAbort": [vp], "dfcclGetAsyncError": [vp, C.POINTER(i)],
            "dfcclGemmReserveSms": [i], "dfcclSetHoldOnWait": [vp, i], "dfcclGetStats": [vp, C.POINTER(Stats)], "dfcclGetHostStats": [vp, C.POINTER(Stats)], "dfcclTraceDump": [vp, C.c_char_p],
            "dfcclInjectFault": [vp, i, C.c_int64],
            "dfcclFusedSgdStep": [vp, vp, vp, vp, sz, i, C.c_float, C.c_float, C.c_float, i, vp],
            "dfcclFusedAdamWStep": [vp, vp, vp, vp, vp, sz, i, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, i, vp],
            "dfcclOpsWarm": [],
            "dfcclGemmBf16": [vp, vp, vp, i, i, i, vp],
            "dfcclGemmBf16Ex": [vp, vp, vp, i, i, i, i, i, vp],
            "dfcclGemmCheck": [C.POINTER(i)],
            "dfcclGemmPairResident": [C.POINTER(i)],
            "dfcclGemmFused": [vp, vp, vp, i, i, i, vp, sz, vp],
            "dfcclHeapPeerBase": [vp, i, C.POINTER(vp)],
            "dfcclCommTransport": [vp, C.POINTER(i)],
            "dfcclTopoXml": [C.c_char_p, i], "dfcclTopoReset": [], "dfcclTopoGpuCount": [], "dfcclTopoP2pAllowed": [i, i],
            "dfcclTunerChoose": [i, sz, i, i, i, i, C.POINTER(i), C.POINTER(i), C.POINTER(C.c_double)],
            "dfcclTunerPredictUs": [i, i, sz, i, i],
            "dfcclProbePeerCopy": [vp, i, sz, i, i, i, i, i, C.POINTER(C.c_double)],
            "dfcclProbeFlagRoundTrip": [vp, i, i, C.POINTER(C.c_double)],
            "dfcclProbeMemoryOps": [i, C.POINTER(C.c_uint64)],
            "dfcclProbeStreamRoundTrip": [i, i, i, C.POINTER(C.c_double)],
            "dfcclAllReduceNoAlloc": [vp, vp, sz, i, C.c_float, vp],
            "dfcclSetDaemonGeometry": [vp, i, i],
        }
        for name, args in sig.items():
            f = getattr(L, name)
            f.argtypes = args
            f.restype = i
        L.dfcclGemmFusedArgsSize.argtypes = []
        L.dfcclGemmFusedArgsSize.restype = C.c_size_t
        L.ncclGetErrorString.argtypes = [i]
        L.ncclGetErrorString.restype = C.c_char_p
        L.dfcclTunerPredictUs.restype = C.c_double
        L.dfcclTopoReset.restype = None
        L.dfcclParam.argtypes = [C.c_char_p, C.c_longlong]
        L.dfcclParam.restype = C.c_longlong
        L.dfcclLogReset.argtypes = []
        L.dfcclLogReset.restype = None
        L.dfcclLastError.argtypes = []
        L.dfcclLastError.restype = C.c_char_p
        _lib = L
        return L


def error_string(code: int) -> str:
    return lib().ncclGetErrorString(code).decode()


def check(code: int, what: str = "dfccl call") -> None:
    if code != SUCCESS:
        raise DfcclError(code, what)


def set_backend(name: str) -> None:
    check(lib().dfcclSetBackend(BACKEND_HOST if name in ("host", "cpu") else BACKEND_CUDA), "dfcclSetBackend")


def get_backend() -> str:
    b = C.c_int()
    check(lib().dfcclGetBackend(C.byref(b)))
    return "host" if b.value == BACKEND_HOST else "cuda"


def param(name: str, default: int = 0) -> int:
    """Value of a configuration parameter as the library reads it: ``DFCCL_<name>``, then ``NCCL_<name>``, then (for the
    reference's unprefixed scheduler knobs) ``<name>``; the environment first, then ``~/.dfccl.conf``, ``~/.nccl.conf``,
    ``/etc/dfccl.conf``, ``/etc/nccl.conf``; ``k`` / ``m`` / ``g`` suffixes scale byte counts."""
    return int(lib().dfcclParam(name.encode(), default))


def log_reset() -> None:
    """Re-read ``DEBUG``, ``DEBUG_SUBSYS`` and ``DEBUG_FILE`` (they are read once, at the first message)."""
    lib().dfcclLogReset()


def last_error() -> str:
    """Text of the calling thread's most recent warning (what went wrong in the call that just failed)."""
    s = lib().dfcclLastError()
    return s.decode() if s else ""


def topo_xml() -> str:
    """The system topology the library works with (detected, or injected with ``DFCCL_TOPO_FILE``) as XML."""
    n = lib().dfcclTopoXml(None, 0)
    if n < 0:
        raise DfcclError(2, "dfcclTopoXml")
    buf = C.create_string_buffer(n + 1)
    lib().dfcclTopoXml(buf, n + 1)
    return buf.value.decode()


def topo_reset() -> None:
    """Forget the cached topology (the next use detects or loads it again)."""
    lib().dfcclTopoReset()


def topo_gpu_count() -> int:
    return lib().dfcclTopoGpuCount()


def topo_p2p_allowed(a: int, b: int) -> bool:
    """Path policy: may devices ``a`` and ``b`` use one another's memory directly (peer access, ``P2P_DISABLE``, ``P2P_LEVEL``)?"""
    r = lib().dfcclTopoP2pAllowed(a, b)
    if r < 0:
        raise DfcclError(2, "dfcclTopoP2pAllowed")
    return bool(r)


def tuner_choose(kind: int, nbytes: int, nranks: int, max_blocks: int, nvls: bool = False, pinned_algo: int = 0):
    """(schedule, blocks, predicted microseconds) the size -> schedule tuner picks for one collective."""
    algo, nb, us = C.c_int(), C.c_int(), C.c_double()
    check(lib().dfcclTunerChoose(kind, nbytes, nranks, max_blocks, 1 if nvls else 0, pinned_algo, C.byref(algo), C.byref(nb), C.byref(us)),
          "dfcclTunerChoose")
    return algo.value, nb.value, us.value


def tuner_predict_us(kind: int, algo: int, nbytes: int, nranks: int, blocks: int) -> float:
    return float(lib().dfcclTunerPredictUs(kind, algo, nbytes, nranks, blocks))


def get_unique_id() -> bytes:
    uid = UniqueId()
    check(lib().ncclGetUniqueId(C.byref(uid)), "ncclGetUniqueId")
    return C.string_at(C.addressof(uid), 128)       # the whole blob: the c_char field would stop at the first NUL


class Comm:
    """Owning wrapper of an ``ncclComm_t``."""

    def __init__(self, handle: int):
        self.handle = C.c_void_p(handle)
        self._live = True

    @staticmethod
    def init_rank(nranks: int, uid: bytes, rank: int) -> "Comm":
        u = UniqueId()
        C.memmove(C.addressof(u), uid, 128)
        h = C.c_void_p()
        check(lib().ncclCommInitRank(C.byref(h), nranks, u, rank), "ncclCommInitRank")
        return Comm(h.value)

    @staticmethod
    def init_all(ndev: int, devices: Optional[Sequence[int]] = None) -> List["Comm"]:
        arr = (C.c_void_p * ndev)()
        devs = (C.c_int * ndev)(*devices) if devices is not None else None
        check(lib().ncclCommInitAll(arr, ndev, devs), "ncclCommInitAll")
        return [Comm(arr[k]) for k in range(ndev)]

    @staticmethod
    def init_loopback(nranks: int, device: int = 0) -> List["Comm"]:
        arr = (C.c_void_p * nranks)()
        check(lib().dfcclCommInitLoopback(arr, nranks, device), "dfcclCommInitLoopback")
        return [Comm(arr[k]) for k in range(nranks)]

    def split(self, color: int, key: int) -> Optional["Comm"]:
        h = C.c_void_p()
        check(lib().dfcclCommSplit(self.handle, color, key, C.byref(h)), "dfcclCommSplit")
        return Comm(h.value) if h.value else None

    @property
    def rank(self) -> int:
        v = C.c_int()
        check(lib().ncclCommUserRank(self.handle, C.byref(v)))
        return v.value

    @property
    def nranks(self) -> int:
        v = C.c_int()
        check(lib().ncclCommCount(self.handle, C.byref(v)))
        return v.value

    @property
    def device(self) -> int:
        v = C.c_int()
        check(lib().ncclCommCuDevice(self.handle, C.byref(v)))
        return v.value

    def alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        check(lib().dfcclMemAlloc(C.byref(p), nbytes, self.handle), "dfcclMemAlloc")
        return p.value

    def free(self, ptr: int) -> None:
        check(lib().dfcclMemFree(C.c_void_p(ptr), self.handle), "dfcclMemFree")

    def nvls_init(self, nbytes: int = 0) -> bool:
        """Collective: bind ``nbytes`` per member to a switch-multicast object.  False when unavailable."""
        ok = C.c_int(0)
        check(lib().dfcclNvlsInit(self.handle, nbytes, C.byref(ok)), "dfcclNvlsInit")
        return bool(ok.value)

    def nvls_alloc(self, nbytes: int) -> int:
        """Symmetric allocation in the NVLS arena (same sizes, same order on every member)."""
        p = C.c_void_p()
        check(lib().dfcclNvlsAlloc(C.byref(p), nbytes, self.handle), "dfcclNvlsAlloc")
        return p.value

    def nvls_info(self):
        uc, mc, b, u = C.c_void_p(), C.c_void_p(), C.c_size_t(), C.c_size_t()
        check(lib().dfcclNvlsInfo(self.handle, C.byref(uc), C.byref(mc), C.byref(b), C.byref(u)), "dfcclNvlsInfo")
        return uc.value, mc.value, b.value, u.value

    def transport(self) -> str:
        """Transport the members selected together: 'peer' memory, 'shm' (heap in registered host shared memory) or 'net'."""
        k = C.c_int()
        check(lib().dfcclCommTransport(self.handle, C.byref(k)), "dfcclCommTransport")
        return ("peer", "shm", "net")[k.value]

    def peer_base(self, peer: int) -> int:
        b = C.c_void_p()
        check(lib().dfcclHeapPeerBase(self.handle, peer, C.byref(b)), "dfcclHeapPeerBase")
        return b.value

    def heap_info(self):
        base, nbytes, used = C.c_void_p(), C.c_size_t(), C.c_size_t()
        check(lib().dfcclHeapInfo(self.handle, C.byref(base), C.byref(nbytes), C.byref(used)))
        return base.value, nbytes.value, used.value

    def async_error(self) -> int:
        v = C.c_int()
        check(lib().ncclCommGetAsyncError(self.handle, C.byref(v)))
        return v.value

    def destroy(self) -> None:
        if self._live:
            self._live = False
            check(lib().ncclCommDestroy(self.handle), "ncclCommDestroy")


class RankCtx:
    """Owning wrapper of an ``ofcclRankCtx_t`` (register, finalize, submit, destroy)."""

    def __init__(self, rank: int, device: int = -1):
        h = C.c_void_p()
        check(lib().dfcclInitRankCtxOnDevice(C.byref(h), rank, device), "ofcclInitRankCtx")
        self.handle = h
        self._callbacks: Dict[int, object] = {}
        self._live = True

    def prepare(self, coll_id: int, comm: Comm, kind: int, count: int, dtype: int, *, out_dtype: Optional[int] = None,
                op: int = SUM, root: int = 0, scale: float = 1.0, algo: int = ALGO_AUTO, n_blocks: int = 0,
                arena_buffers: bool = False) -> None:
        info = CollInfo(kind, count, dtype, dtype if out_dtype is None else out_dtype, op, root, scale, algo, n_blocks,
                        COLL_ARENA_BUFFERS if arena_buffers else 0)
        check(lib().dfcclPrepare(C.byref(info), comm.handle, coll_id, self.handle), f"dfcclPrepare({coll_id})")

    def prepare_fused(self, coll_id: int, comm: Comm, kind: int, rows_per_rank: int, k: int, n: int) -> None:
        """Register a GEMM fused with its tensor-parallel collective (``FUSED_ALLGATHER_GEMM`` / ``FUSED_GEMM_REDUCESCATTER``)."""
        info = FusedInfo(kind, rows_per_rank, k, n)
        check(lib().dfcclPrepareFusedGemm(C.byref(info), comm.handle, coll_id, self.handle), f"dfcclPrepareFusedGemm({coll_id})")

    def fused_operand(self, coll_id: int):
        """(address of this rank's rows, address of the gathered operand) of a registered all-gather -> GEMM."""
        a, b = C.c_void_p(), C.c_void_p()
        check(lib().dfcclFusedGemmOperand(coll_id, self.handle, C.byref(a), C.byref(b)), f"dfcclFusedGemmOperand({coll_id})")
        return a.value, b.value

    def run_fused(self, coll_id: int, x: int, w: int, out: int, stream: int, w_transposed: bool = False) -> None:
        """``w``: [n, k]; with ``w_transposed`` [k, n] (read in place as an MN-major operand)."""
        fn = lib().dfcclRunFusedGemmT if w_transposed else lib().dfcclRunFusedGemm
        check(fn(coll_id, C.c_void_p(x), C.c_void_p(w), C.c_void_p(out), C.c_void_p(stream), self.handle), f"dfcclRunFusedGemm({coll_id})")

    def set_daemon_geometry(self, blocks: int = 0, threads: int = 0) -> None:
        check(lib().dfcclSetDaemonGeometry(self.handle, blocks, threads), "dfcclSetDaemonGeometry")

    def finalize(self) -> None:
        check(lib().ofcclFinalizeRankCtx7StartHostThrds(self.handle), "ofcclFinalizeRankCtx7StartHostThrds")

    def run(self, coll_id: int, send: int, recv: int, callback: Optional[Callable[[int], None]] = None) -> None:
        cb = CALLBACK(0)
        if callback is not None:
            def tramp(cid, _args, _f=callback):
                _f(cid)
                return 0
            cb = CALLBACK(tramp)
            self._callbacks[coll_id] = cb          # keep the trampoline alive until the next submit of this id
        check(lib().dfcclRun(C.c_void_p(send), C.c_void_p(recv), coll_id, cb, None, self.handle), f"dfcclRun({coll_id})")

    def run_on_stream(self, coll_id: int, send: int, recv: int, stream: int) -> None:
        check(lib().dfcclRunOnStream(C.c_void_p(send), C.c_void_p(recv), coll_id, C.c_void_p(stream), CALLBACK(0), None,
                                     self.handle), f"dfcclRunOnStream({coll_id})")

    def run_deferred(self, coll_id: int, send: int, recv: int) -> None:
        """Publish a submission that ``trigger_on_stream`` (or the replay of a graph that captured it) releases."""
        check(lib().dfcclRunDeferred(C.c_void_p(send), C.c_void_p(recv), coll_id, CALLBACK(0), None, self.handle),
              f"dfcclRunDeferred({coll_id})")

    def trigger_on_stream(self, coll_id: int, stream: int) -> None:
        check(lib().dfcclTriggerOnStream(coll_id, C.c_void_p(stream), self.handle), f"dfcclTriggerOnStream({coll_id})")

    def stream_wait(self, coll_id: int, stream: int) -> None:
        check(lib().dfcclStreamWait(coll_id, C.c_void_p(stream), self.handle), f"dfcclStreamWait({coll_id})")

    def wait(self, coll_id: int, timeout_ms: int = -1) -> int:
        return lib().dfcclWait(coll_id, timeout_ms, self.handle)

    def wait_all(self, timeout_ms: int = -1) -> int:
        return lib().dfcclWaitAll(timeout_ms, self.handle)

    def abort(self) -> None:
        check(lib().dfcclAbort(self.handle))

    def async_error(self) -> int:
        v = C.c_int()
        check(lib().dfcclGetAsyncError(self.handle, C.byref(v)))
        return v.value

    def stats(self) -> Dict[str, int]:
        s = Stats()
        check(lib().dfcclGetStats(self.handle, C.byref(s)), "dfcclGetStats")
        return s.as_dict()

    def set_hold_on_wait(self, on: bool) -> None:
        check(lib().dfcclSetHoldOnWait(self.handle, 1 if on else 0), "dfcclSetHoldOnWait")

    def host_stats(self) -> Dict[str, int]:
        """Host-side counters only; safe while the device is busy."""
        s = Stats()
        check(lib().dfcclGetHostStats(self.handle, C.byref(s)), "dfcclGetHostStats")
        return {k: v for k, v in s.as_dict().items() if k in ("sqesSubmitted", "cqesDelivered", "daemonLaunches", "daemonVoluntaryQuits", "deviceEvents")}

    def trace_dump(self, path: str) -> None:
        check(lib().dfcclTraceDump(self.handle, path.encode()), "dfcclTraceDump")

    def inject_fault(self, fault: int, arg: int) -> None:
        check(lib().dfcclInjectFault(self.handle, fault, arg))

    def destroy(self) -> None:
        if self._live:
            self._live = False
            check(lib().ofcclDestroy(self.handle), "ofcclDestroy")
