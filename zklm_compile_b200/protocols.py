"""Host-side mirror of the reference's sub-protocol provers over the C ABI.

Each `prove_*` returns the proof as the reference's bincode bytes (the layout of the serde
structs in rust/zk_ml_prover/src/proving/*.rs), so two implementations can be compared byte
for byte.  Names and argument order follow the reference functions cited per function.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, u32p
from .sumcheck import Context, DeviceBuffer, Transcript


def _a(x):
    a = np.ascontiguousarray(x, dtype=np.uint32)
    return a, a.ctypes.data_as(u32p)


def log2_ceil(n: int) -> int:
    """rust/zk_ml_prover/src/field/common.rs:16-21"""
    return 1 if n <= 1 else (n - 1).bit_length()


def _proof_call(ctx: Context, fn, *args, cap: int = 1 << 22) -> bytes:
    buf = (C.c_uint8 * cap)()
    n = C.c_size_t()
    st = fn(*args, buf, C.c_size_t(cap), C.byref(n))
    if st == 7 and n.value > cap:
        return _proof_call(ctx, fn, *args, cap=n.value)
    check(ctx.h, st)
    return C.string_at(buf, n.value)


def commit_weights_fast(ctx: Context, weights) -> bytes:
    """weight_commitment.rs:82-107 -> 32-byte root."""
    out = (C.c_uint8 * 32)()
    if isinstance(weights, DeviceBuffer):
        check(ctx.h, _lib.lib().zkb_commit_weights_fast(ctx.h, weights.ptr, C.c_size_t(weights.n), C.c_int32(1), out))
    else:
        w, pw = _a(weights)
        check(ctx.h, _lib.lib().zkb_commit_weights_fast(ctx.h, pw, C.c_size_t(w.size), C.c_int32(0), out))
    return bytes(out)


def eq_evals(ctx: Context, r) -> np.ndarray:
    """m31_ops.rs:30-50"""
    a, pa = _a(r)
    out = np.zeros(1 << a.size, np.uint32)
    check(ctx.h, _lib.lib().zkb_eq_evals(ctx.h, pa, C.c_uint32(a.size), C.c_int32(0), out.ctypes.data_as(u32p)))
    return out


def eq_evals_ef(ctx: Context, r) -> np.ndarray:
    """m31_ops.rs:175-191; r is (k, 4)."""
    a, pa = _a(r)
    k = a.size // 4
    out = np.zeros((1 << k, 4), np.uint32)
    check(ctx.h, _lib.lib().zkb_eq_evals(ctx.h, pa, C.c_uint32(k), C.c_int32(1), out.ctypes.data_as(u32p)))
    return out


def mle_evaluate(ctx: Context, evals, point) -> int:
    """m31_ops.rs:11-26; evals: host array or DeviceBuffer of n <= 2^k values, point: k coordinates."""
    pt, pp = _a(point)
    out = C.c_uint32()
    if isinstance(evals, DeviceBuffer):
        pe, n, on = evals.ptr, evals.n, 1
    else:
        e, pe = _a(evals)
        n, on = e.size, 0
    check(ctx.h, _lib.lib().zkb_mle_eval_base(ctx.h, pe, C.c_size_t(n), pp, C.c_uint32(pt.size), C.c_int32(on), C.byref(out)))
    return out.value


def mle_evaluate_ef(ctx: Context, evals, point, evals_ef: bool = False) -> np.ndarray:
    """m31_ops.rs:155-171; point is (k, 4); with evals_ef the table holds EF elements (n, 4)."""
    pt, pp = _a(point)
    w = 4 if evals_ef else 1
    out = np.zeros(4, np.uint32)
    if isinstance(evals, DeviceBuffer):
        pe, n, on = evals.ptr, evals.n // w, 1
    else:
        e, pe = _a(evals)
        n, on = e.size // w, 0
    check(ctx.h, _lib.lib().zkb_mle_eval_ef(ctx.h, pe, C.c_size_t(n), C.c_int32(int(evals_ef)), pp, C.c_uint32(pt.size // 4), C.c_int32(on),
                                             out.ctypes.data_as(u32p)))
    return out


def batch_inverse(ctx: Context, vals, ef: bool = False):
    """lookup.rs:322-345 (ef=False) / :348-368 (ef=True).  Host array in, host array out; a
    DeviceBuffer is inverted in place (as the reference's Metal hook does, lookup.rs:491-542)."""
    fn = _lib.lib().zkb_batch_inverse_ef if ef else _lib.lib().zkb_batch_inverse_base
    w = 4 if ef else 1
    if isinstance(vals, DeviceBuffer):
        check(ctx.h, fn(ctx.h, vals.ptr, C.c_size_t(vals.n // w), C.c_int32(1), vals.ptr))
        return vals
    v, pv = _a(vals)
    out = np.zeros_like(v)
    check(ctx.h, fn(ctx.h, pv, C.c_size_t(v.size // w), C.c_int32(0), out.ctypes.data_as(u32p)))
    return out


def requantize_lookup(ctx: Context, raw, table_out: DeviceBuffer = None):
    """transformer/mod.rs:293-324 (+ the activation lookup of qwen.rs:286-316 when a table is given).
    Returns q, or (q, table[q])."""
    r, pr = _a(raw)
    q = np.zeros(r.size, np.uint32)
    t = np.zeros(r.size, np.uint32) if table_out is not None else None
    check(ctx.h, _lib.lib().zkb_requantize_lookup(ctx.h, pr, C.c_size_t(r.size), C.c_int32(0), table_out.ptr if table_out is not None else None,
                                                   C.c_uint32(table_out.n if table_out is not None else 0), q.ctypes.data_as(u32p),
                                                   t.ctypes.data_as(u32p) if t is not None else None))
    return q if t is None else (q, t)


def fold_eq_matvec(ctx: Context, w_flat, m: int, n: int, r_point, ef: bool = False) -> np.ndarray:
    """matmul.rs:76-128 (ef=False) / :743-835 (ef=True)."""
    r, pr = _a(r_point)
    log_m = r.size // (4 if ef else 1)
    n_pad = 1 << log2_ceil(n)
    out = np.zeros((n_pad, 4) if ef else n_pad, np.uint32)
    if isinstance(w_flat, DeviceBuffer):
        pw, on = w_flat.ptr, 1
    else:
        w, pw = _a(w_flat)
        on = 0
    check(ctx.h, _lib.lib().zkb_fold_eq_matvec(ctx.h, pw, C.c_size_t(m), C.c_size_t(n), pr, C.c_uint32(log_m), C.c_int32(int(ef)),
                                                C.c_int32(on), out.ctypes.data_as(u32p)))
    return out


def matmul_forward(ctx: Context, w_flat, x, m: int, n: int) -> np.ndarray:
    """transformer/mod.rs:140-163"""
    xv, px = _a(x)
    y = np.zeros(m, np.uint32)
    if isinstance(w_flat, DeviceBuffer):
        pw, on = w_flat.ptr, 1
    else:
        w, pw = _a(w_flat)
        on = 0
    check(ctx.h, _lib.lib().zkb_matvec_forward(ctx.h, pw, px, C.c_size_t(m), C.c_size_t(n), C.c_int32(on), y.ctypes.data_as(u32p)))
    return y


def rmsnorm_forward(ctx: Context, x, gamma):
    """transformer/mod.rs:245-288 -> (output, perturbed_input, delta)."""
    xv, px = _a(x)
    g, pg = _a(gamma)
    out = np.zeros(xv.size, np.uint32)
    xu = np.zeros(xv.size, np.uint32)
    delta = C.c_int32()
    check(ctx.h, _lib.lib().zkb_rmsnorm_forward(ctx.h, px, pg, C.c_size_t(xv.size), out.ctypes.data_as(u32p), xu.ctypes.data_as(u32p),
                                                 C.byref(delta)))
    return out, xu, delta.value


BIND_BLAKE3, BIND_PCS, BIND_PCS_FULL = 0, 1, 2


def prove_matmul_succinct_ef(w_flat, x_vals, y_vals, m: int, n: int, transcript: Transcript, bind_mode: int = BIND_BLAKE3,
                             node_hash: int = 0) -> bytes:
    """matmul.rs:963-997 -> SuccinctMatmulProofEF.  bind_mode selects what the reference fixes at
    compile time (bind_weights_ef, matmul.rs:360-453): default build, feature pcs, feature pcs-full."""
    ctx = transcript.ctx
    x, px = _a(x_vals)
    y, py = _a(y_vals)
    if isinstance(w_flat, DeviceBuffer):
        pw, on = w_flat.ptr, 1
    else:
        w, pw = _a(w_flat)
        on = 0
    return _proof_call(ctx, _lib.lib().zkb_prove_matmul_succinct_ef_bind, ctx.h, transcript.h, pw, px, py, C.c_size_t(m), C.c_size_t(n),
                       C.c_int32(on), C.c_int32(bind_mode), C.c_int32(node_hash))


def prove_matmul_succinct(w_flat, x_vals, y_vals, m: int, n: int, transcript: Transcript) -> bytes:
    """matmul.rs:482-511 (base-field challenges) -> SuccinctMatmulProof."""
    ctx = transcript.ctx
    x, px = _a(x_vals)
    y, py = _a(y_vals)
    if isinstance(w_flat, DeviceBuffer):
        pw, on = w_flat.ptr, 1
    else:
        w, pw = _a(w_flat)
        on = 0
    return _proof_call(ctx, _lib.lib().zkb_prove_matmul_succinct, ctx.h, transcript.h, pw, px, py, C.c_size_t(m), C.c_size_t(n),
                       C.c_int32(on))


def prove_mle_eval_bound(weights, point, label: bytes, root: bytes, transcript: Transcript) -> bytes:
    """weight_commitment.rs:437-447 (label = b"" gives prove_mle_eval_no_merkle, :177-206) -> MleEvalProof."""
    ctx = transcript.ctx
    w, pw = _a(weights)
    pt, pp = _a(point)
    lab = (C.c_uint8 * max(1, len(label))).from_buffer_copy(label or b"\0")
    rt = (C.c_uint8 * 32).from_buffer_copy(root or bytes(32))
    return _proof_call(ctx, _lib.lib().zkb_prove_mle_eval, ctx.h, transcript.h, pw, C.c_size_t(w.size), pp, C.c_uint32(pt.size),
                       lab, C.c_size_t(len(label)), rt)


def _elementwise_base(is_add, a, b, c, point, transcript):
    ctx = transcript.ctx
    av, pa = _a(a)
    bv, pb = _a(b)
    cv, pc = _a(c)
    pt, pp = _a(point)
    return _proof_call(ctx, _lib.lib().zkb_prove_elementwise, ctx.h, transcript.h, C.c_int32(is_add), pa, pb, pc, C.c_size_t(av.size),
                       pp, C.c_uint32(pt.size))


def prove_hadamard(a, b, c, point, transcript: Transcript) -> bytes:
    """elementwise.rs:50-98 (base-field challenges) -> HadamardProof."""
    return _elementwise_base(0, a, b, c, point, transcript)


def prove_add(a, b, c, point, transcript: Transcript) -> bytes:
    """elementwise.rs:189-235 (base-field challenges) -> AddProof."""
    return _elementwise_base(1, a, b, c, point, transcript)


def _elementwise(is_add, a, b, c, point, transcript):
    ctx = transcript.ctx
    av, pa = _a(a)
    bv, pb = _a(b)
    cv, pc = _a(c)
    pt, pp = _a(point)
    return _proof_call(ctx, _lib.lib().zkb_prove_elementwise_ef, ctx.h, transcript.h, C.c_int32(is_add), pa, pb, pc, C.c_size_t(av.size),
                       pp, C.c_uint32(pt.size // 4))


def prove_hadamard_ef(a, b, c, point, transcript: Transcript) -> bytes:
    """elementwise.rs:429-480 -> HadamardProofEF."""
    return _elementwise(0, a, b, c, point, transcript)


def prove_add_ef(a, b, c, point, transcript: Transcript) -> bytes:
    """elementwise.rs:545-595 -> AddProofEF."""
    return _elementwise(1, a, b, c, point, transcript)


def prove_rmsnorm_ef(x, gamma, y, perturbation_delta: int, transcript: Transcript) -> bytes:
    """rmsnorm.rs:512-667 -> RmsNormProofEF."""
    ctx = transcript.ctx
    xv, px = _a(x)
    g, pg = _a(gamma)
    yv, py = _a(y)
    return _proof_call(ctx, _lib.lib().zkb_prove_rmsnorm_ef, ctx.h, transcript.h, px, pg, py, C.c_size_t(xv.size),
                       C.c_int32(perturbation_delta))


def prove_rmsnorm(x, gamma, y, perturbation_delta: int, transcript: Transcript) -> bytes:
    """rmsnorm.rs:96-246 (base-field challenges) -> RmsNormProof."""
    ctx = transcript.ctx
    xv, px = _a(x)
    g, pg = _a(gamma)
    yv, py = _a(y)
    return _proof_call(ctx, _lib.lib().zkb_prove_rmsnorm, ctx.h, transcript.h, px, pg, py, C.c_size_t(xv.size),
                       C.c_int32(perturbation_delta))


def prove_lookup_ef(table_outputs, inputs, outputs, transcript: Transcript) -> bytes:
    """lookup.rs:643-762 -> LookupProofEF.  Raises ZkbError with the reference's panic messages
    (status 3: LogUp identity failed, status 4: alpha collision)."""
    ctx = transcript.ctx
    t, pt = _a(table_outputs)
    i, pi = _a(inputs)
    o, po = _a(outputs)
    return _proof_call(ctx, _lib.lib().zkb_prove_lookup_ef, ctx.h, transcript.h, pt, C.c_size_t(t.size), pi, po, C.c_size_t(i.size))


def prove_lookup(table_outputs, inputs, outputs, transcript: Transcript) -> bytes:
    """lookup.rs:432-604 (base-field challenges) -> LookupProof; same error statuses as prove_lookup_ef."""
    ctx = transcript.ctx
    t, pt = _a(table_outputs)
    i, pi = _a(inputs)
    o, po = _a(outputs)
    return _proof_call(ctx, _lib.lib().zkb_prove_lookup, ctx.h, transcript.h, pt, C.c_size_t(t.size), pi, po, C.c_size_t(i.size))


def fold_eq_matvec_ef_noalloc(w_dev: DeviceBuffer, m: int, n: int, eq_dev: DeviceBuffer, out_dev: DeviceBuffer, stream=None):
    """Weight fold for callers that may not allocate GPU memory while running (fixed memory
    plans, hosts that forbid cudaMalloc after start-up).  All three buffers are device memory
    the caller already owns; the library's own scratch is a fixed 512 KiB array, so the padded
    column count is limited to 16384.  Work is enqueued on `stream` (default stream if None);
    calls must not overlap on the GPU."""
    err = C.create_string_buffer(256)
    fn = _lib.lib().zkb_fold_eq_matvec_ef_noalloc
    st = fn(w_dev.ptr, C.c_size_t(m), C.c_size_t(n), eq_dev.ptr, out_dev.ptr, C.c_void_p(stream), err, C.c_size_t(256))
    if st != 0:
        raise _lib.ZkbError(st, err.value.decode(errors="replace"))
