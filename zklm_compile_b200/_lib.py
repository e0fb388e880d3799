"""ctypes binding of libzkb200.so — the only way the package reaches the GPU.

There is no CPU path: if the shared library is missing this module raises, and every call
that needs a device returns a nonzero status which is raised as `ZkbError`.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
# ZKB200_LIB selects another build of the same library (e.g. an instrumented one); there is still no fallback.
LIB_PATH = os.environ.get("ZKB200_LIB") or os.path.join(_HERE, "libzkb200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "zkb200.h")

u32p = C.POINTER(C.c_uint32)
u8p = C.POINTER(C.c_uint8)


class ZkbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"zkb200 status {code}: {msg}")
        self.code = code


def build(verbose: bool = False) -> str:
    """Compile the CUDA library in-tree for sm_100a (nvcc cross-compiles without a GPU)."""
    subprocess.run(["make", "-C", os.path.join(_HERE, "csrc")] + ([] if verbose else ["-s"]), check=True)
    return LIB_PATH


_lib = None

# The per-layer proofs run on one CUDA stream each; the default of 8 hardware work queues would
# make streams share a queue and serialise behind each other.  Must be set before CUDA starts.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `make -C zklm_compile_b200/csrc` "
                "(there is no fallback implementation)")
        L = C.CDLL(LIB_PATH)
        L.zkb_last_error.restype = C.c_char_p
        L.zkb_last_error.argtypes = [C.c_void_p]
        L.zkb_launch_count.restype = C.c_uint64
        L.zkb_launch_count.argtypes = [C.c_void_p]
        L.zkb_ctx_destroy.restype = None
        L.zkb_ctx_destroy.argtypes = [C.c_void_p]
        L.zkb_tr_free.restype = None
        L.zkb_tr_free.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def check(ctx_handle, status: int):
    if status != 0:
        msg = lib().zkb_last_error(ctx_handle).decode(errors="replace") if ctx_handle else ""
        raise ZkbError(status, msg)
