"""dfccl_b200: a Blackwell-native deadlock-free collective library.

``native``     ctypes binding of the C interface (nccl*, ofccl*, dfccl*)
``simulator``  issue-order deadlock models and the daemon-preemption model
``parallel``   data / tensor / pipeline parallel building blocks on top of the daemon
``models``     ResNet-50 and GPT-2 used by the benchmarks
``ops``        fused compute + collective operators
"""
__version__ = "0.1.0"
