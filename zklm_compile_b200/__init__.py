"""zkb200 — B200-native backend for zk_ml_prover's sumcheck hot path.

The package is a thin host-side mirror of the reference's prover interface over the C ABI in
`include/zkb200.h`; all arithmetic runs in hand-written sm_100a CUDA kernels
(`zklm_compile_b200/csrc`).  Importing it does not need a GPU; using it does.
"""
from ._lib import ZkbError, build, lib, LIB_PATH  # noqa: F401
from .sumcheck import *  # noqa: F401,F403
