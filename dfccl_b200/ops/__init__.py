from .gemm import matmul_nt, gemm_supported
from . import collectives
