"""Weights in the reference's wire format, resident on the GPU (mirror of the server's preload step,
rust/zk_ml_prover/src/server.rs:33-94, over zkb_weightset_* of the C ABI)."""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import _lib
from ._lib import check, u32p
from .sumcheck import Context, DeviceBuffer


def preload_block(matrices) -> bytes:
    """The preload block a client of the reference's server sends: [count u32] then per matrix
    [name_len u32][name][m u32][n u32][m * n u32 LE].  `matrices`: iterable of (name, 2-D uint32 array)."""
    matrices = list(matrices)
    parts = [struct.pack("<I", len(matrices))]
    for name, w in matrices:
        w = np.ascontiguousarray(w, dtype="<u4")
        nb = name.encode() if isinstance(name, str) else bytes(name)
        parts += [struct.pack("<I", len(nb)), nb, struct.pack("<II", w.shape[0], w.shape[1]), w.tobytes()]
    return b"".join(parts)


class WeightSet:
    def __init__(self, ctx: Context, block: bytes):
        self.ctx = ctx
        self.h = C.c_void_p()
        used = C.c_size_t()
        buf = np.frombuffer(block, dtype=np.uint8)
        check(ctx.h, _lib.lib().zkb_weightset_preload(ctx.h, buf.ctypes.data_as(C.POINTER(C.c_uint8)), C.c_size_t(buf.size), C.byref(self.h),
                                                       C.byref(used)))
        self.consumed = used.value

    def __len__(self):
        return int(_lib.lib().zkb_weightset_count(self.h))

    @property
    def nbytes(self) -> int:
        fn = _lib.lib().zkb_weightset_bytes
        fn.restype = C.c_uint64
        fn.argtypes = [C.c_void_p]
        return int(fn(self.h))

    def get(self, name: str):
        """(device buffer, m, n, commit_weights_fast root) of the matrix of that name."""
        p = u32p()
        m, n = C.c_size_t(), C.c_size_t()
        root = (C.c_uint8 * 32)()
        check(self.ctx.h, _lib.lib().zkb_weightset_get(self.h, name.encode(), C.byref(p), C.byref(m), C.byref(n), root))
        addr = C.cast(p, C.c_void_p).value
        return DeviceBuffer.wrap(self.ctx, addr, m.value * n.value), m.value, n.value, bytes(root)

    def close(self):
        if self.h.value and self.ctx.h.value:
            _lib.lib().zkb_weightset_destroy.restype = None
            _lib.lib().zkb_weightset_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
