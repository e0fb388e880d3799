"""Host-side mirror of the reference's sumcheck interface over the C ABI.

Names, argument order and return shapes follow rust/zk_ml_prover/src/proving/sumcheck.rs:
`Transcript` (:110-206), `prove_product*` / `prove_triple*` / `prove_product_ones*`
(:211-978, :1204-1435) and `prove_product_ef_mixed` (rust/zk_ml_prover/src/proving/matmul.rs:889-944).
Tables may be numpy arrays (copied to the device inside the call) or `DeviceBuffer`s.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import u32p, u8p, check

P = (1 << 31) - 1

SC_PRODUCT, SC_TRIPLE, SC_PRODUCT_ONES, SC_PRODUCT_EF, SC_PRODUCT_EF_FULL, SC_PRODUCT_EF_MIXED, \
    SC_TRIPLE_EF_FULL, SC_PRODUCT_ONES_EF_FULL = range(8)

# kind -> (input widths, stored evals per round, output width)
_KINDS = {
    SC_PRODUCT: ((1, 1), 3, 1),
    SC_TRIPLE: ((1, 1, 1), 4, 1),
    SC_PRODUCT_ONES: ((1,), 2, 1),
    SC_PRODUCT_EF: ((1, 1), 2, 4),
    SC_PRODUCT_EF_FULL: ((4, 4), 3, 4),
    SC_PRODUCT_EF_MIXED: ((4, 1), 3, 4),
    SC_TRIPLE_EF_FULL: ((4, 4, 4), 3, 4),
    SC_PRODUCT_ONES_EF_FULL: ((4,), 2, 4),
}


class Context:
    """One GPU + one CUDA stream (replaces the reference's MetalContext/MetalKernels singletons,
    rust/zk_ml_prover/src/gpu/metal_device.rs:47-77)."""

    def __init__(self, device: int = 0):
        self.h = C.c_void_p()
        st = _lib.lib().zkb_ctx_create(C.c_int32(device), C.byref(self.h))
        if st != 0:
            raise _lib.ZkbError(st, f"zkb_ctx_create(device={device}) failed (no CUDA device?)")
        self.device = device

    def close(self):
        if getattr(self, "h", None) and self.h.value:
            _lib.lib().zkb_ctx_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        check(self.h, _lib.lib().zkb_ctx_sync(self.h))

    def set_shared(self, on: bool = True):
        """This context runs next to many others on the same GPU: use launch shapes that leave half
        of every SM free (see zkb_ctx_set_shared in include/zkb200.h)."""
        check(self.h, _lib.lib().zkb_ctx_set_shared(self.h, C.c_int32(1 if on else 0)))

    def trim(self):
        """Give the context's scratch arena back to the device (the next proof allocates it again)."""
        check(self.h, _lib.lib().zkb_ctx_trim(self.h))

    @property
    def scratch_bytes(self) -> int:
        fn = _lib.lib().zkb_ctx_scratch_bytes
        fn.restype = C.c_uint64
        fn.argtypes = [C.c_void_p]
        return int(fn(self.h))

    OPT_PLAIN_TAIL, OPT_SINGLE_CTA_THREADS, OPT_PIPE_THREADS, OPT_NO_FUSED_FOLD, OPT_FOLD2_VEC, OPT_BASEFOLD_IN_ORDER, OPT_MATVEC_PREFETCH_ROWS, OPT_MATVEC_RING, OPT_SHARED_SM_HASH, OPT_ATTENTION_THREADS = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9

    def set_option(self, option: int, value: int):
        """Tuning options for measurements (zkb_ctx_set_option in include/zkb200.h); 0 = built-in choice."""
        check(self.h, _lib.lib().zkb_ctx_set_option(self.h, C.c_int32(option), C.c_int32(value)))

    @property
    def stream(self) -> int:
        """The context's cudaStream_t as an integer handle."""
        fn = _lib.lib().zkb_ctx_stream
        fn.restype = C.c_void_p
        fn.argtypes = [C.c_void_p]
        return fn(self.h) or 0

    def timer_start(self):
        check(self.h, _lib.lib().zkb_timer_start(self.h))

    def timer_stop_ms(self) -> float:
        ms = C.c_float()
        check(self.h, _lib.lib().zkb_timer_stop_ms(self.h, C.byref(ms)))
        return ms.value

    def profile(self, on: bool):
        check(self.h, _lib.lib().zkb_profile_enable(self.h, C.c_int32(1 if on else 0)))

    def profile_read(self):
        buf = (C.c_float * 256)()
        n = C.c_size_t()
        check(self.h, _lib.lib().zkb_profile_read(self.h, buf, C.c_size_t(256), C.byref(n)))
        return [buf[i] for i in range(min(n.value, 256))]

    def profile_ranges(self):
        """{tag: (ms, algorithmic bytes, launches)} for the bracketed matrix kernels since the last call."""
        ms = (C.c_double * 2)()
        by = (C.c_double * 2)()
        cnt = (C.c_uint64 * 2)()
        check(self.h, _lib.lib().zkb_profile_ranges(self.h, ms, by, cnt))
        return {"fold_eq_matvec": (ms[0], by[0], cnt[0]), "matvec_forward": (ms[1], by[1], cnt[1])}

    def trace(self, on: bool):
        """Launch trace: an event behind every launch of this context (also inside layer graphs)."""
        check(self.h, _lib.lib().zkb_trace_enable(self.h, C.c_int32(1 if on else 0)))

    def trace_dump(self, path: str, base: "Context | None" = None):
        """Write `index,site,ms` lines; ms counts from the first traced launch of `base` (default: own)."""
        check(self.h, _lib.lib().zkb_trace_dump(self.h, base.h if base is not None else None, path.encode()))

    @property
    def launches(self) -> int:
        return int(_lib.lib().zkb_launch_count(self.h))

    def upload(self, arr) -> "DeviceBuffer":
        a = np.ascontiguousarray(arr, dtype=np.uint32)
        buf = DeviceBuffer(self, a.size, a.shape)
        check(self.h, _lib.lib().zkb_buf_upload_u32(self.h, a.ctypes.data_as(u32p), C.c_size_t(a.size), buf.ptr))
        return buf

    def pinned_u32(self, n_u32: int) -> np.ndarray:
        """numpy view of page-locked host memory (freed with the process, or earlier by host_free)."""
        p = C.c_void_p()
        check(self.h, _lib.lib().zkb_host_alloc(self.h, C.c_size_t(n_u32 * 4), C.byref(p)))
        return np.ctypeslib.as_array(C.cast(p, u32p), shape=(n_u32,))

    def host_free(self, arr: np.ndarray):
        """Release an array obtained from pinned_u32; the array must not be used afterwards."""
        check(self.h, _lib.lib().zkb_host_free(self.h, C.c_void_p(arr.ctypes.data)))

    def alloc(self, n_u32: int, shape=None) -> "DeviceBuffer":
        return DeviceBuffer(self, n_u32, shape or (n_u32,))


class DeviceBuffer:
    """u32 device array (replaces GpuBuffer, rust/zk_ml_prover/src/gpu/metal_buffer.rs:9-53)."""

    def __init__(self, ctx: Context, n_u32: int, shape):
        self.ctx = ctx
        self.n = int(n_u32)
        self.shape = tuple(shape)
        self.ptr = u32p()
        check(ctx.h, _lib.lib().zkb_buf_alloc(ctx.h, C.c_size_t(self.n), C.byref(self.ptr)))

    @classmethod
    def wrap(cls, ctx: "Context", address: int, n_u32: int) -> "DeviceBuffer":
        """View of `n_u32` words of device memory owned by somebody else (e.g. a tensor another
        library received into); never freed by this object."""
        b = cls.__new__(cls)
        b.ctx, b.n, b.shape = ctx, int(n_u32), (int(n_u32),)
        b.ptr = C.cast(C.c_void_p(address), u32p)
        b._borrowed = True
        return b

    def download(self) -> np.ndarray:
        out = np.empty(self.n, np.uint32)
        check(self.ctx.h, _lib.lib().zkb_buf_download_u32(self.ctx.h, self.ptr, C.c_size_t(self.n), out.ctypes.data_as(u32p)))
        return out.reshape(self.shape)

    def free(self):
        if getattr(self, "_borrowed", False):
            self.ptr = u32p()
            return
        if self.ptr and self.ctx.h.value:
            check(self.ctx.h, _lib.lib().zkb_buf_free(self.ctx.h, self.ptr))
            self.ptr = u32p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Transcript:
    """Device-resident Fiat-Shamir transcript (sumcheck.rs:110-206)."""

    def __init__(self, ctx: Context, label: bytes):
        self.ctx = ctx
        self.h = C.c_void_p()
        lab = (C.c_uint8 * max(len(label), 1)).from_buffer_copy(label if label else b"\0")
        check(ctx.h, _lib.lib().zkb_tr_new(ctx.h, lab, C.c_size_t(len(label)), C.byref(self.h)))

    def __del__(self):
        try:
            if self.h.value and self.ctx.h.value:
                _lib.lib().zkb_tr_free(self.h)
                self.h = C.c_void_p()
        except Exception:
            pass

    def absorb(self, v: int):
        check(self.ctx.h, _lib.lib().zkb_tr_absorb_u32(self.h, C.c_uint32(int(v))))

    def absorb_many(self, values):
        if isinstance(values, DeviceBuffer):
            check(self.ctx.h, _lib.lib().zkb_tr_absorb_many_dev(self.h, values.ptr, C.c_size_t(values.n)))
            return
        a = np.ascontiguousarray(values, dtype=np.uint32)
        check(self.ctx.h, _lib.lib().zkb_tr_absorb_many(self.h, a.ctypes.data_as(u32p), C.c_size_t(a.size)))

    def absorb_bytes(self, b: bytes):
        arr = (C.c_uint8 * max(len(b), 1)).from_buffer_copy(b if b else b"\0")
        check(self.ctx.h, _lib.lib().zkb_tr_absorb_bytes(self.h, arr, C.c_size_t(len(b))))

    def absorb_ef(self, v):
        for x in np.asarray(v, dtype=np.uint32).reshape(4):
            self.absorb(int(x))

    def squeeze(self) -> int:
        o = C.c_uint32()
        check(self.ctx.h, _lib.lib().zkb_tr_squeeze(self.h, C.byref(o)))
        return o.value

    def squeeze_many(self, n: int):
        return [self.squeeze() for _ in range(n)]

    def squeeze_ef(self) -> np.ndarray:
        o = np.zeros(4, np.uint32)
        check(self.ctx.h, _lib.lib().zkb_tr_squeeze_ef(self.h, o.ctypes.data_as(u32p)))
        return o

    def export_state(self) -> bytes:
        buf = (C.c_uint8 * 112)()
        check(self.ctx.h, _lib.lib().zkb_tr_export(self.h, buf))
        return bytes(buf)

    def import_state(self, state: bytes):
        buf = (C.c_uint8 * 112).from_buffer_copy(state)
        check(self.ctx.h, _lib.lib().zkb_tr_import(self.h, buf))


@dataclass
class SumcheckProof:
    """`SumcheckProof` / `SumcheckProofEF` (sumcheck.rs:57-65, 99-107): `round_polys[round]` holds
    the stored evaluations (EF ones as rows of 4 u32), `challenges[round]` the challenge."""
    round_polys: np.ndarray
    challenges: np.ndarray


def sumcheck_prove(kind: int, tables, num_vars: int, transcript: Transcript):
    widths, epr, w = _KINDS[kind]
    ctx = transcript.ctx
    n = 1 << num_vars
    on_dev = all(isinstance(t, DeviceBuffer) for t in tables)
    keep, ptrs = [], (u32p * 3)()
    for i, (t, wd) in enumerate(zip(tables, widths)):
        if on_dev:
            if t.n != n * wd:
                raise ValueError(f"table {i}: expected {n * wd} u32, got {t.n}")
            ptrs[i] = t.ptr
        else:
            if isinstance(t, DeviceBuffer):
                raise ValueError("tables must be all host arrays or all DeviceBuffers")
            a = np.ascontiguousarray(t, dtype=np.uint32)
            if a.size != n * wd:
                raise ValueError(f"table {i}: expected {n * wd} u32, got {a.size}")
            keep.append(a)
            ptrs[i] = a.ctypes.data_as(u32p)
    polys = np.zeros((num_vars, epr, w) if w == 4 else (num_vars, epr), np.uint32)
    chal = np.zeros((num_vars, w) if w == 4 else (num_vars,), np.uint32)
    fin = np.zeros((max(2, len(widths)), w), np.uint32)
    check(ctx.h, _lib.lib().zkb_sumcheck_prove(
        ctx.h, transcript.h, C.c_int32(kind), ptrs, C.c_uint32(num_vars), C.c_int32(1 if on_dev else 0),
        polys.ctypes.data_as(u32p), chal.ctypes.data_as(u32p), fin.ctypes.data_as(u32p)))
    finals = [fin[i] if w == 4 else int(fin[i, 0]) for i in range(fin.shape[0])]
    return (SumcheckProof(polys, chal), *finals)


# ---- the reference's entry points -------------------------------------------------------------
def prove_product(f, g, num_vars, transcript):
    """sumcheck.rs:211-272; also stands in for prove_product_parallel / _gpu / _best (:389-482, :625-710, :815-828)."""
    return sumcheck_prove(SC_PRODUCT, [f, g], num_vars, transcript)


prove_product_parallel = prove_product
prove_product_best = prove_product


def prove_triple(f, g, h, num_vars, transcript):
    """sumcheck.rs:277-354; also prove_triple_parallel / _gpu / _best (:487-619, :714-812, :831-845)."""
    return sumcheck_prove(SC_TRIPLE, [f, g, h], num_vars, transcript)


prove_triple_parallel = prove_triple
prove_triple_best = prove_triple


def prove_product_ones(g, num_vars, transcript):
    """sumcheck.rs:857-902; also _parallel / _best (:906-978).  Returns (proof, 1, g(s))."""
    return sumcheck_prove(SC_PRODUCT_ONES, [g], num_vars, transcript)


prove_product_ones_parallel = prove_product_ones
prove_product_ones_best = prove_product_ones


def prove_product_ef(f, g, num_vars, transcript):
    """sumcheck.rs:1204-1258 — base-field tables, EF challenges, compressed [s0, s2] messages."""
    return sumcheck_prove(SC_PRODUCT_EF, [f, g], num_vars, transcript)


def prove_product_ef_full(f, g, num_vars, transcript):
    """sumcheck.rs:1262-1315 — EF tables, full [s0, s1, s2] messages."""
    return sumcheck_prove(SC_PRODUCT_EF_FULL, [f, g], num_vars, transcript)


def prove_product_ef_mixed(f_ef, g_base, num_vars, transcript):
    """matmul.rs:889-944 — f in EF, g in the base field, full messages."""
    return sumcheck_prove(SC_PRODUCT_EF_MIXED, [f_ef, g_base], num_vars, transcript)


def prove_triple_ef_full(f, g, h, num_vars, transcript):
    """sumcheck.rs:1318-1384 — EF tables, stored [s0, s2, s3]."""
    return sumcheck_prove(SC_TRIPLE_EF_FULL, [f, g, h], num_vars, transcript)


def prove_product_ones_ef_full(g, num_vars, transcript):
    """sumcheck.rs:1389-1435 — f == 1, stored [s0, s2]."""
    return sumcheck_prove(SC_PRODUCT_ONES_EF_FULL, [g], num_vars, transcript)
