"""In-tree build of the native library (``dfccl_b200/lib/libdfccl.so``).

Everything is compiled with nvcc for sm_100a only (``-gencode
arch=compute_100a,code=sm_100a``): device code and the host runtime live in the
same shared object, which is loaded through ctypes (``dfccl_b200.lib``).  Objects
are cached under ``dfccl_b200/csrc/build`` and rebuilt when a source or any
header is newer.  ``python -m dfccl_b200._build`` builds from the command line;
``DFCCL_FAST_BUILD=1`` compiles only the float / bfloat16 reduction kernels
(development shortcut, never used for a committed measurement).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = CSRC / "build"
LIBDIR = ROOT / "lib"
LIB = LIBDIR / "libdfccl.so"

SOURCES = [
    "src/common/log.cc", "src/common/param.cc", "src/common/socket.cc",
    "src/bootstrap/bootstrap.cc",
    "src/mem/heap.cu", "src/mem/mcast.cu", "src/topo/topo.cu", "src/net/net_socket.cc", "src/net/net_ring.cu",
    "src/device/datapath.cu", "src/daemon/daemon.cu", "src/daemon/standalone.cu", "src/daemon/daemon_host.cu",
    "src/comm/comm.cu",
    "src/api/nccl_api.cu", "src/api/p2p.cu", "src/api/ofccl_api.cu", "src/api/debug_api.cu",
    "src/ops/optim.cu", "src/api/noalloc.cu", "src/api/probe.cu", "src/gemm/tcgen05_gemm.cu", "src/gemm/tcgen05_gemm_pair.cu",
]

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _flags(verbose: bool) -> list:
    f = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
         "-I", str(CSRC / "include"), "-Wno-deprecated-gpu-targets", "-x", "cu", "-rdc=true"] + ARCH
    if os.environ.get("DFCCL_FAST_BUILD") == "1":
        f.append("-DDF_FAST_BUILD")
    if verbose:
        f += ["-Xptxas", "-v"]
    return f


def _newest_header() -> float:
    return max((p.stat().st_mtime for p in CSRC.rglob("*.h")), default=0.0)


def _compile(src: str, verbose: bool, hdr_time: float, sanitize: str = "") -> Path:
    s = CSRC / src
    o = OBJ / (src.replace("/", "_") + (f".{sanitize}.o" if sanitize else ".fast.o" if os.environ.get("DFCCL_FAST_BUILD") == "1" else ".o"))
    if o.exists() and o.stat().st_mtime > max(s.stat().st_mtime, hdr_time):
        return o
    extra = []
    if src.endswith("device/datapath.cu"):
        # out-of-line device functions do not inherit a kernel's launch bounds: cap them at what
        # a 512-thread block leaves per thread (the reference caps its device code the same way)
        extra = ["-maxrregcount=128"]
    if sanitize:                                     # host code only: the device code is the same as in the plain build
        extra += ["-Xcompiler", f"-fsanitize={sanitize},-fno-omit-frame-pointer,-g", "-DDF_FAST_BUILD"]
    cmd = [nvcc()] + _flags(verbose) + extra + ["-c", str(s), "-o", str(o)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return o


def build(verbose: bool = False, force: bool = False, extra_sources=(), sanitize: str = "") -> Path:
    """Compile what is stale and link ``libdfccl.so``; returns its path.

    ``sanitize="thread"`` or ``"address"`` builds ``libdfccl_<sanitize>.so`` instead, with the host code (the
    runtime, and the scheduler / engine / data path as compiled for the host backend) instrumented by the
    compiler's sanitizer: the race and memory checks of the library run on the CPU twin of the device code."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    hdr = _newest_header()
    srcs = [s for s in list(SOURCES) + list(extra_sources) if (CSRC / s).exists()]
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, hdr, sanitize), srcs))
    lib = LIBDIR / f"libdfccl_{sanitize}.so" if sanitize else LIB
    if lib.exists() and all(lib.stat().st_mtime > o.stat().st_mtime for o in objs):
        return lib
    san = ["-Xcompiler", f"-fsanitize={sanitize}"] if sanitize else []
    cmd = [nvcc(), "-shared", "-rdc=true", "-Xcompiler", "-fPIC", "-o", str(lib)] + san + [str(o) for o in objs] + ARCH + ["-lrt", "-lpthread", "-ldl", "-cudart", "static", "-Xlinker", "-Bsymbolic"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
