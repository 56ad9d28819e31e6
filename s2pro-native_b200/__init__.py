"""Python host-side mirror of the s2pro-b200 C ABI (ctypes).

The product is the C library ``libs2pro_b200.so`` (C11 host code + hand-written
sm_100a CUDA).  This package only binds it for tests and the benchmark driver:
same entry-point names, argument meaning and status codes as the C header
``include/s2p_b200_abi.h``.  There is no Python or CPU fallback: loading fails
loudly when the library has not been built.
"""
from .capi import (  # noqa: F401
    LIB_PATH, S2PError, check, lib, load_library, Linear, Tensor, ModelOpts, SamplingCfg, VqPart,
    GEMM_BF16, GEMM_INT8, STATUS_NAMES, Stats,
)
