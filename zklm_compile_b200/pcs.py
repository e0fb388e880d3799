"""Host-side mirror of the reference's Merkle tree and Basefold commitment over the C ABI
(rust/zk_ml_prover/src/proving/pcs.rs, basefold.rs).  Results are the reference's values or
the bincode bytes of its proof structs."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, u32p
from .protocols import _a, _proof_call, log2_ceil
from .sumcheck import Context, DeviceBuffer, Transcript

NODE_BLAKE3, NODE_AES_MMO = 0, 1


def _src(values):
    if isinstance(values, DeviceBuffer):
        return values, values.ptr, values.n, 1
    a, pa = _a(values)
    return a, pa, a.size, 0


def merkle_root(ctx: Context, values, node_hash: int = NODE_BLAKE3) -> bytes:
    """MerkleTree::new(values).root(), pcs.rs:143-201."""
    keep, p, n, dev = _src(values)
    out = (C.c_uint8 * 16)()
    check(ctx.h, _lib.lib().zkb_merkle_root(ctx.h, p, C.c_size_t(n), C.c_int32(dev), C.c_int32(node_hash), out))
    return bytes(out)


def merkle_layers(ctx: Context, values, node_hash: int = NODE_BLAKE3) -> bytes:
    """All internal layers, parents of the leaves first (pcs.rs:156-196)."""
    keep, p, n, dev = _src(values)
    h = log2_ceil(n)
    return _proof_call(ctx, _lib.lib().zkb_merkle_layers, ctx.h, p, C.c_size_t(n), C.c_int32(dev), C.c_int32(node_hash),
                       cap=16 << h)


def merkle_batch_open(ctx: Context, values, indices, node_hash: int = NODE_BLAKE3) -> bytes:
    """MerkleTree::batch_open, pcs.rs:290-337 -> bincode(BatchMerkleProof)."""
    keep, p, n, dev = _src(values)
    idx = np.ascontiguousarray(indices, dtype=np.uint64)
    return _proof_call(ctx, _lib.lib().zkb_merkle_batch_open, ctx.h, p, C.c_size_t(n), C.c_int32(dev), C.c_int32(node_hash),
                       idx.ctypes.data_as(C.POINTER(C.c_uint64)), C.c_size_t(idx.size))


def basefold_tables(ctx: Context, log_n: int):
    """generate_tables(log_n, table_seed(log_n)), basefold.rs:106-143 -> (t_flat, w_flat)."""
    total = (1 << log_n) - 1
    t = np.zeros(total, np.uint32)
    w = np.zeros(total, np.uint32)
    check(ctx.h, _lib.lib().zkb_basefold_tables(ctx.h, C.c_uint32(log_n), t.ctypes.data_as(u32p), w.ctypes.data_as(u32p)))
    return t, w


def basefold_encode(ctx: Context, coeffs, out: DeviceBuffer = None):
    """encode, basefold.rs:169-238 (coefficients zero-padded to a power of two, at least 2).
    With `out` (a device buffer of 2 * 2^log_n words) the codeword stays on the device."""
    keep, p, n, dev = _src(coeffs)
    if out is not None:
        assert out.n >= 2 << log2_ceil(n)
        check(ctx.h, _lib.lib().zkb_basefold_encode(ctx.h, p, C.c_size_t(n), C.c_int32(dev), out.ptr, C.c_int32(1)))
        return out
    cw = np.zeros(2 << log2_ceil(n), np.uint32)
    check(ctx.h, _lib.lib().zkb_basefold_encode(ctx.h, p, C.c_size_t(n), C.c_int32(dev), cw.ctypes.data_as(u32p), C.c_int32(0)))
    return cw


def basefold_commit_and_prove(ctx: Context, tr: Transcript, coeffs, point, node_hash: int = NODE_BLAKE3) -> bytes:
    """commit_and_prove, basefold.rs:368-396 -> bincode(BasefoldCommitment) || bincode(BasefoldOpeningProof)."""
    keep, p, n, dev = _src(coeffs)
    if dev:
        assert isinstance(point, DeviceBuffer)
        pp, npt = point.ptr, point.n
    else:
        pt, pp = _a(point)
        npt = pt.size
    return _proof_call(ctx, _lib.lib().zkb_basefold_commit_and_prove, ctx.h, tr.h, p, C.c_size_t(n), pp, C.c_uint32(npt),
                       C.c_int32(dev), C.c_int32(node_hash), cap=1 << 22)


def basefold_verify_opening(ctx: Context, tr: Transcript, blob: bytes, point, claimed: int, node_hash: int = NODE_BLAKE3) -> bool:
    """verify_opening, basefold.rs:611-748, on the bytes basefold_commit_and_prove returns.  The caller
    absorbs the commitment root (blob[:16]) into `tr` first, as the reference's callers do."""
    pt, pp = _a(point)
    ok = C.c_int32(0)
    buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
    check(ctx.h, _lib.lib().zkb_basefold_verify_opening(ctx.h, tr.h, buf, C.c_size_t(len(blob)), pp, C.c_uint32(pt.size),
                                                        C.c_uint32(int(claimed)), C.c_int32(node_hash), C.byref(ok)))
    return bool(ok.value)


def basefold_batch_verify_opening(ctx: Context, tr: Transcript, blob: bytes, node_hash: int = NODE_BLAKE3) -> bool:
    """batch_verify_opening, basefold.rs:959-1137, on the bytes BasefoldBatch.prove returns."""
    ok = C.c_int32(0)
    buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
    check(ctx.h, _lib.lib().zkb_basefold_batch_verify_opening(ctx.h, tr.h, buf, C.c_size_t(len(blob)), C.c_int32(node_hash), C.byref(ok)))
    return bool(ok.value)


class BasefoldBatch:
    """Batch Basefold over polynomials of possibly different sizes (basefold.rs:1144-1378).

    Construction is `batch_precommit_multi_height`: every polynomial is encoded (with the largest one's tables) and its
    Merkle tree built, both kept in device memory - the transcript-independent half, done once at load time.  `prove(tr)` is
    `batch_prove_with_precommit`: one fold chain over the rho-weighted sum of the codewords, the smaller ones joining when the
    chain reaches their length.  With `individual_openings` (equal sizes only) the result is `batch_commit_and_prove`
    (basefold.rs:801-956).  Returns bincode(Vec<BasefoldCommitment>) (input order) || bincode(BasefoldBatchProof)."""

    def __init__(self, ctx: Context, polys, log_ns, node_hash: int = NODE_BLAKE3):
        self.ctx = ctx
        self.h = C.c_void_p()
        k = len(polys)
        keep = [_src(p) for p in polys]
        dev = [d for _, _, _, d in keep]
        if any(dev) and not all(dev):
            raise ValueError("the polynomials are either all DeviceBuffers or all host arrays")
        self._keep = keep if all(dev) and k else None             # device polynomials are borrowed, not copied
        ptrs = (u32p * max(k, 1))(*[p for _, p, _, _ in keep])
        ns = (C.c_size_t * max(k, 1))(*[n for _, _, n, _ in keep])
        lns = (C.c_uint32 * max(k, 1))(*[int(x) for x in log_ns])
        check(ctx.h, _lib.lib().zkb_basefold_batch_precommit(ctx.h, ptrs, ns, lns, C.c_size_t(k), C.c_int32(int(all(dev) and k > 0)),
                                                             C.c_int32(node_hash), C.byref(self.h)))
        self.k = k

    def commitment(self, i: int):
        root = (C.c_uint8 * 16)()
        n = C.c_uint64(); ln = C.c_uint64()
        check(self.ctx.h, _lib.lib().zkb_basefold_batch_commitment(self.h, C.c_size_t(i), root, C.byref(n), C.byref(ln)))
        return bytes(root), n.value, ln.value

    @property
    def device_bytes(self) -> int:
        f = _lib.lib().zkb_basefold_batch_device_bytes
        f.restype = C.c_uint64
        return int(f(self.h))

    def prove(self, tr: Transcript, individual_openings: bool = False) -> bytes:
        return _proof_call(self.ctx, _lib.lib().zkb_basefold_batch_prove, self.h, tr.h, C.c_int32(int(individual_openings)), cap=1 << 22)

    def close(self):
        if self.h.value and self.ctx.h.value:
            _lib.lib().zkb_basefold_batch_destroy.restype = None
            _lib.lib().zkb_basefold_batch_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
