"""Reference arm of ``bench.py``: the same ResNet-50 step with the gradient all-reduce done
by the UNMODIFIED reference library (``baseline/_ref/lib/libnccl.so``, built offline from
the reference tree for sm_100) through its own public, stock entry points
(``ncclGetUniqueId`` / ``ncclCommInitRank`` / ``ncclAllReduce``).  Nothing of this
repository's engine is on that path: the model is torchvision's ResNet-50, the optimizer is
``torch.optim.SGD``, buckets are packed and unpacked with plain PyTorch copies, and
``torch.distributed`` (gloo) only carries the unique id and the timing reduction.

Set ``REF_PATH=ofccl`` to drive the reference's register-then-submit interface
(``ofcclPrepareAllReduce`` / ``ofcclRunAllReduce`` with host callbacks) instead of the
stream-ordered one.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

REF_LIB = Path(__file__).resolve().parent / "_ref" / "lib" / "libnccl.so.2.12.12"

NCCL_SUM, NCCL_AVG = 0, 4
NCCL_FLOAT32, NCCL_BFLOAT16 = 7, 9


def reference_unavailable() -> str:
    """Empty string when the reference arm can run, else the reason (one line)."""
    if not REF_LIB.exists():
        return ("reference library not built: pip cannot install the reference (no setup.py / pyproject.toml); "
                "its make build for sm_100 is expected at baseline/_ref/lib/libnccl.so.2.12.12")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # Observed on 2 x B200: the reference's stock ncclAllReduce kernels never completed (both ranks
        # stalled behind them until the 120 s watchdog ended the run; the GPUs still answered).  Its
        # device code is therefore not run again at more than one rank.
        return ("reference ncclAllReduce (NCCL 2.12.12 fork, built for sm_100) hung at 2 ranks on B200; "
                "not run again at N>1 on this pool (record: profiles/reference_arm_n2_hang.txt)")
    return ""


class RefDist:
    """Rank bookkeeping of the reference arm (gloo carries the unique id and the timing reduction)."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.torch_dist = self.world > 1
        if self.torch_dist:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group("gloo", rank=self.rank, world_size=self.world)

    def barrier(self):
        if self.torch_dist:
            import torch.distributed as dist
            dist.barrier()

    def destroy(self):
        if self.torch_dist:
            import torch.distributed as dist
            dist.destroy_process_group()


def make_model(device, classes: int = 1000, tiny: bool = False):
    """torchvision's ResNet-50, bf16 channels-last with fp32 normalisation parameters."""
    import torchvision
    import torch.nn as nn
    net = torchvision.models.resnet50(num_classes=classes) if not tiny else torchvision.models.resnet18(num_classes=classes)
    net = net.to(device).to(memory_format=torch.channels_last).to(torch.bfloat16)
    for m in net.modules():
        if isinstance(m, nn.modules.batchnorm._BatchNorm):
            m.float()
    return net


class _UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


CALLBACK = C.CFUNCTYPE(C.c_int, C.c_int, C.c_void_p)


class ReferenceBackend:
    name = "reference"

    def __init__(self, d):
        self.d = d
        os.environ.setdefault("NCCL_SOCKET_IFNAME", "lo")
        self.path = os.environ.get("REF_PATH", "nccl")
        if self.path == "ofccl":                     # the preemptible path implements Ring + Simple only
            os.environ.setdefault("NCCL_ALGO", "Ring")
            os.environ.setdefault("NCCL_PROTO", "Simple")
        self.lib = C.CDLL(str(REF_LIB), mode=C.RTLD_LOCAL)
        L, vp = self.lib, C.c_void_p
        L.ncclGetUniqueId.argtypes = [C.POINTER(_UniqueId)]
        L.ncclCommInitRank.argtypes = [C.POINTER(vp), C.c_int, _UniqueId, C.c_int]
        L.ncclAllReduce.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
        L.ncclCommDestroy.argtypes = [vp]
        L.ncclGetErrorString.restype = C.c_char_p
        uid = _UniqueId()
        if d.world > 1:
            import torch.distributed as dist
            box = [None]
            if d.rank == 0:
                self._check(L.ncclGetUniqueId(C.byref(uid)), "ncclGetUniqueId")
                box = [C.string_at(C.addressof(uid), 128)]
            dist.broadcast_object_list(box, src=0)
            C.memmove(C.addressof(uid), box[0], 128)
        else:
            self._check(L.ncclGetUniqueId(C.byref(uid)), "ncclGetUniqueId")
        self.comm = vp()
        self._check(L.ncclCommInitRank(C.byref(self.comm), d.world, uid, d.rank), "ncclCommInitRank")
        self.launch_count = 0
        self.opt = None
        self.buckets = []

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"reference {what} failed: {self.lib.ncclGetErrorString(rc).decode()}")

    def attach(self, net):
        params = [p for p in net.parameters() if p.requires_grad]
        self.opt = torch.optim.SGD(params, lr=0.1, momentum=0.9, weight_decay=1e-4, foreach=True)
        limit = int(25.0 * (1 << 20))
        by = {}
        for p in reversed(params):
            by.setdefault(p.dtype, []).append(p)
        for dt, plist in by.items():
            cur, size = [], 0
            for p in plist:
                nb = p.numel() * p.element_size()
                if cur and size + nb > limit:
                    self.buckets.append(self._mk(cur, dt))
                    cur, size = [], 0
                cur.append(p)
                size += nb
            if cur:
                self.buckets.append(self._mk(cur, dt))
        if self.path == "ofccl":
            self._setup_ofccl()

    def _mk(self, plist, dt):
        n = sum(p.numel() for p in plist)
        return {"params": plist, "flat": torch.zeros(n, dtype=dt, device=self.d.device), "dtype": dt, "n": n}

    # ---- register-then-submit path of the reference
    def _setup_ofccl(self):
        L, vp = self.lib, C.c_void_p
        L.ofcclInitRankCtx.argtypes = [C.POINTER(vp), C.c_int]
        L.ofcclPrepareAllReduce.argtypes = [C.c_size_t, C.c_int, C.c_int, vp, C.c_int, vp]
        L.ofcclFinalizeRankCtx7StartHostThrds.argtypes = [vp]
        L.ofcclRunAllReduce.argtypes = [vp, vp, C.c_int, CALLBACK, vp, vp]
        L.ofcclDestroy.argtypes = [vp]
        self.ctx = vp()
        self._check(L.ofcclInitRankCtx(C.byref(self.ctx), self.d.local_rank), "ofcclInitRankCtx")
        self.comms = []
        for i, b in enumerate(self.buckets):       # the reference wants one communicator per collective
            uid = _UniqueId()
            if self.d.world > 1:
                import torch.distributed as dist
                box = [None]
                if self.d.rank == 0:
                    self._check(L.ncclGetUniqueId(C.byref(uid)), "ncclGetUniqueId")
                    box = [C.string_at(C.addressof(uid), 128)]
                dist.broadcast_object_list(box, src=0)
                C.memmove(C.addressof(uid), box[0], 128)
            else:
                self._check(L.ncclGetUniqueId(C.byref(uid)), "ncclGetUniqueId")
            c = vp()
            self._check(L.ncclCommInitRank(C.byref(c), self.d.world, uid, self.d.rank), "ncclCommInitRank")
            self.comms.append(c)
            dt = NCCL_BFLOAT16 if b["dtype"] == torch.bfloat16 else NCCL_FLOAT32
            self._check(L.ofcclPrepareAllReduce(b["n"], dt, NCCL_SUM, c, i, self.ctx), "ofcclPrepareAllReduce")
        self._check(L.ofcclFinalizeRankCtx7StartHostThrds(self.ctx), "ofcclFinalizeRankCtx7StartHostThrds")
        self._done = threading.Semaphore(0)

        def cb(_cid, _args):
            self._done.release()
            return 0
        self._cb = CALLBACK(cb)

    def finish_backward(self):
        from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors
        s = torch.cuda.current_stream()
        for b in self.buckets:
            b["grads"] = [p.grad for p in b["params"]]
            b["flat"] = _flatten_dense_tensors(b["grads"])
        if self.path == "ofccl":
            s.synchronize()                          # no stream argument in that interface: the host orders
            for i, b in enumerate(self.buckets):
                self._check(self.lib.ofcclRunAllReduce(C.c_void_p(b["flat"].data_ptr()), C.c_void_p(b["flat"].data_ptr()), i,
                                                       self._cb, None, self.ctx), "ofcclRunAllReduce")
            for _ in self.buckets:
                self._done.acquire()
            for b in self.buckets:
                b["flat"].div_(self.d.world)
        else:
            for b in self.buckets:
                dt = NCCL_BFLOAT16 if b["dtype"] == torch.bfloat16 else NCCL_FLOAT32
                self._check(self.lib.ncclAllReduce(C.c_void_p(b["flat"].data_ptr()), C.c_void_p(b["flat"].data_ptr()), b["n"], dt,
                                                   NCCL_AVG, self.comm, C.c_void_p(s.cuda_stream)), "ncclAllReduce")
                self.launch_count += 1
        for b in self.buckets:
            for g, synced in zip(b["grads"], _unflatten_dense_tensors(b["flat"], b["grads"])):
                g.copy_(synced)

    def step(self):
        self.opt.step()
        self.opt.zero_grad(set_to_none=False)

    def launches(self):
        return self.launch_count

    def info(self):
        return {"buckets": len(self.buckets), "bucket_mb": 25.0, "path": self.path, "library": str(REF_LIB.name)}

    def close(self):
        torch.cuda.synchronize()
        if self.path == "ofccl":
            self.lib.ofcclDestroy(self.ctx)
        self.lib.ncclCommDestroy(self.comm)
