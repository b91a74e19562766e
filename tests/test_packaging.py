"""Stand-alone build of the native library (csrc/Makefile): shared library, static archive, pkg-config file and the
binary package; a plain C program links against the STATIC archive and runs register-then-submit on the host backend."""
import os
import shutil
import subprocess
import tarfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "dfccl_b200", "csrc")


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"), reason="needs nvcc")
def test_makefile_builds_archive_package_and_a_c_program_runs(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    build = tmp_path / "build"
    jobs = str(max(2, min(16, os.cpu_count() or 2)))
    p = subprocess.run(["make", "-C", CSRC, "-j", jobs, f"BUILDDIR={build}", f"NVCC={nvcc}", "pkg"], capture_output=True, text=True,
                       timeout=1500)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    for f in ("lib/libdfccl.so", "lib/libdfccl_static.a", "lib/pkgconfig/dfccl.pc"):
        assert (build / f).exists(), f
    pkg = build / "pkg" / "dfccl-0.1.0-cuda-sm100a.tar.xz"
    with tarfile.open(pkg) as t:
        names = set(t.getnames())
    for f in ("lib/libdfccl.so", "lib/libdfccl_static.a", "lib/pkgconfig/dfccl.pc", "include/dfccl.h", "include/dfccl_noalloc.h"):
        assert f"dfccl-0.1.0-cuda-sm100a/{f}" in names, f
    exe = tmp_path / "smoke"
    p = subprocess.run([nvcc, "-Wno-deprecated-gpu-targets", "-x", "c", os.path.join(CSRC, "examples", "host_backend_smoke.c"),
                        "-I", os.path.join(CSRC, "include"), "-L", str(build / "lib"), "-ldfccl_static", "-lpthread", "-ldl", "-lrt",
                        "-o", str(exe)], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "12 callbacks, 0 ranks with wrong results" in p.stdout, p.stdout + p.stderr
