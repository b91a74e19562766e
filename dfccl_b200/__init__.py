"""dfccl_b200: a Blackwell-native deadlock-free collective library.

``native``     ctypes binding of the C interface (nccl*, ofccl*, dfccl*)
``simulator``  issue-order deadlock models and the daemon-preemption model
``parallel``   data / tensor / pipeline parallel building blocks on top of the daemon
``models``     ResNet-50 and GPT-2 used by the benchmarks
``ops``        fused compute + collective operators
"""
__version__ = "0.1.0"

import os as _os

# A kernel that CUDA loads lazily takes its first launch through a module load, which can wait for the
# device to go idle.  If that happens while a stream is parked on a completion word that only the daemon
# sets, and the daemon in turn needs a (re)launch from its observer thread, the two wait for each other.
# Loading every kernel when its module is loaded removes the case.  Only effective when the package is
# imported before the process creates its CUDA context; an explicit setting of the variable wins.
_os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
