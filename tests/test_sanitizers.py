"""Race and memory checks: the library is rebuilt with the compiler's ThreadSanitizer / AddressSanitizer
(host code only - which includes the scheduler, the engine and the data path as compiled for the host
backend) and a multi-rank scenario runs under it in a child process.  Any report fails the test."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _runtime(name):
    p = subprocess.run(["gcc", f"-print-file-name=lib{name}.so"], capture_output=True, text=True).stdout.strip()
    return p if os.path.isabs(p) and os.path.exists(p) else None


@pytest.mark.parametrize("kind,rt,marker,opts", [
    ("thread", "tsan", "WARNING: ThreadSanitizer", {"TSAN_OPTIONS": "report_signal_unsafe=0 exitcode=0"}),
    ("address", "asan", "ERROR: AddressSanitizer", {"ASAN_OPTIONS": "detect_leaks=0 exitcode=0 verify_asan_link_order=0"}),
])
def test_host_twin_under_sanitizer(kind, rt, marker, opts):
    runtime = _runtime(rt)
    if runtime is None:
        pytest.skip(f"lib{rt} is not installed")
    sys.path.insert(0, ROOT)
    from dfccl_b200 import _build
    lib = _build.build(sanitize=kind)
    env = dict(os.environ, LD_PRELOAD=runtime, DFCCL_LIBRARY=str(lib), **opts)
    env.pop("DFCCL_FORCE_NET", None)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "sanitizer_case.py")], env=env, capture_output=True, text=True, timeout=900)
    out = p.stdout + p.stderr
    assert "CASE OK" in out, out[-4000:]
    assert marker not in out, out[out.index(marker):][:6000]
