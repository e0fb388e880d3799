"""One sumcheck split over several GPUs, one process per GPU.

Rank g holds the table elements j with j mod world == g.  Folding is MSB-first, so until only
`world` elements are left every round is local to a GPU except for its partial sums, which the
round kernels exchange over NVLink themselves (peer-mapped mailboxes); the host's part is the
one-time exchange of the mailbox handles, done here with torch.distributed."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, u32p
from .sumcheck import _KINDS, Context, DeviceBuffer, SumcheckProof, Transcript


def slice_for_rank(table, world: int, rank: int, width: int = 1) -> np.ndarray:
    """The slice rank `rank` owns: elements j with j mod world == rank (elements of `width` words)."""
    a = np.ascontiguousarray(table, dtype=np.uint32).reshape(-1, width)
    return np.ascontiguousarray(a[rank::world]).reshape(-1)


class Exchange:
    """Mailboxes of one rank, connected to its peers' (see include/zkb200.h, zkb_xch_*)."""

    def __init__(self, ctx: Context, world: int, rank: int, gather_handles=None, timeout_ms: int = None, loopback: bool = False):
        self.ctx, self.world, self.rank = ctx, world, rank
        self.h = C.c_void_p()
        check(ctx.h, _lib.lib().zkb_xch_create(ctx.h, C.c_uint32(world), C.c_uint32(rank), C.byref(self.h)))
        if timeout_ms:
            check(ctx.h, _lib.lib().zkb_xch_set_timeout_ms(self.h, C.c_uint32(timeout_ms)))
        if world > 1 and loopback:       # peers that never answer: only for exercising the time-out path
            check(ctx.h, _lib.lib().zkb_xch_connect_loopback(self.h))
        elif world > 1:
            mine = (C.c_uint8 * 64)()
            check(ctx.h, _lib.lib().zkb_xch_handle(self.h, mine))
            handles = (gather_handles or _gather_with_torch)(bytes(mine), world)
            if len(handles) != world or any(len(b) != 64 for b in handles):
                raise ValueError("expected one 64-byte handle per rank")
            blob = (C.c_uint8 * (64 * world)).from_buffer_copy(b"".join(handles))
            check(ctx.h, _lib.lib().zkb_xch_connect(self.h, blob))

    def close(self):
        if self.h.value:
            _lib.lib().zkb_xch_destroy.restype = None
            _lib.lib().zkb_xch_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _gather_with_torch(mine: bytes, world: int):
    import torch.distributed as dist
    out = [None] * world
    dist.all_gather_object(out, mine)
    return out


def sumcheck_prove_split(kind: int, local_tables, num_vars: int, transcript: Transcript, xch: Exchange):
    """`sumcheck_prove` for tables of 2^num_vars elements given as this rank's slices."""
    widths, epr, w = _KINDS[kind]
    ctx = transcript.ctx
    n_local = (1 << num_vars) // xch.world
    on_dev = all(isinstance(t, DeviceBuffer) for t in local_tables)
    keep, ptrs = [], (u32p * 3)()
    for i, (t, wd) in enumerate(zip(local_tables, widths)):
        if on_dev:
            if t.n != n_local * wd:
                raise ValueError(f"table {i}: expected {n_local * wd} u32, got {t.n}")
            ptrs[i] = t.ptr
        else:
            a = np.ascontiguousarray(t, dtype=np.uint32)
            if a.size != n_local * wd:
                raise ValueError(f"table {i}: expected {n_local * wd} u32, got {a.size}")
            keep.append(a)
            ptrs[i] = a.ctypes.data_as(u32p)
    polys = np.zeros((num_vars, epr, w) if w == 4 else (num_vars, epr), np.uint32)
    chal = np.zeros((num_vars, w) if w == 4 else (num_vars,), np.uint32)
    fin = np.zeros((max(2, len(widths)), w), np.uint32)
    check(ctx.h, _lib.lib().zkb_sumcheck_prove_split(
        ctx.h, xch.h, transcript.h, C.c_int32(kind), ptrs, C.c_uint32(num_vars), C.c_int32(1 if on_dev else 0),
        polys.ctypes.data_as(u32p), chal.ctypes.data_as(u32p), fin.ctypes.data_as(u32p)))
    finals = [fin[i] if w == 4 else int(fin[i, 0]) for i in range(fin.shape[0])]
    return (SumcheckProof(polys, chal), *finals)
