"""Row-decomposed attention at seq_len >= 2, mirroring rust/zk_ml_prover/src/proving/attention.rs.

`prove_row_attention` has the reference's argument order (attention.rs:116-125) and returns the
bincode image of its RowAttentionProof; `row_attention_forward` is the op's forward pass
(pipeline/forward.rs:233-276).  Both run on the GPU (one CTA per (head, row)); there is no CPU path.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, u32p
from .sumcheck import Context, DeviceBuffer, Transcript


def _ptr(x):
    if isinstance(x, DeviceBuffer):
        return x, x.ptr, True
    a = np.ascontiguousarray(x, dtype=np.uint32)
    return a, a.ctypes.data_as(u32p), False


def _inputs(q, k, v, exp_table):
    keep = [_ptr(a) for a in (q, k, v, exp_table)]
    dev = [d for _, _, d in keep]
    if any(dev) and not all(dev):
        raise ValueError("q, k, v and the table are either all DeviceBuffers or all host arrays")
    n_table = keep[3][0].n if dev[3] else keep[3][0].size
    return keep, [p for _, p, _ in keep], int(all(dev)), n_table


def row_attention_forward(ctx: Context, q, k, v, num_heads: int, seq_len: int, d_head: int, exp_table, num_kv_heads: int = 0) -> np.ndarray:
    """out[h][i] = softmax_table(Q[h][i] K[g]^T) V[g] over M31, g = h (forward.rs:233-276) or, with num_kv_heads,
    g = h // (num_heads // num_kv_heads) (forward.rs:594-640)."""
    keep, ptrs, on_dev, n_table = _inputs(q, k, v, exp_table)
    n = num_heads * seq_len * d_head
    if on_dev:
        out = DeviceBuffer(ctx, n, (n,))
        check(ctx.h, _lib.lib().zkb_row_attention_gqa_forward(ctx.h, *ptrs[:3], C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len),
                                                              C.c_size_t(d_head), ptrs[3], C.c_size_t(n_table), C.c_int32(1), out.ptr))
        return out
    out = np.zeros(n, np.uint32)
    check(ctx.h, _lib.lib().zkb_row_attention_gqa_forward(ctx.h, *ptrs[:3], C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len),
                                                          C.c_size_t(d_head), ptrs[3], C.c_size_t(n_table), C.c_int32(0), out.ctypes.data_as(u32p)))
    return out


def prove_row_attention(q, k, v, num_heads: int, seq_len: int, d_head: int, exp_table, transcript: Transcript, want_output: bool = False,
                        num_kv_heads: int = 0):
    """attention.rs:116-276 -> bincode(RowAttentionProof) [, the op's output]."""
    ctx = transcript.ctx
    keep, ptrs, on_dev, n_table = _inputs(q, k, v, exp_table)
    n = num_heads * seq_len * d_head
    out = None
    pout = u32p()
    if want_output:
        if on_dev:
            out = DeviceBuffer(ctx, n, (n,)); pout = out.ptr
        else:
            out = np.zeros(n, np.uint32); pout = out.ctypes.data_as(u32p)
    cap = proof_size_bound(num_heads, seq_len, d_head)
    buf = (C.c_uint8 * cap)()
    ln = C.c_size_t()
    st = _lib.lib().zkb_prove_row_attention_gqa(ctx.h, transcript.h, *ptrs[:3], C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len),
                                                C.c_size_t(d_head), ptrs[3], C.c_size_t(n_table), C.c_int32(on_dev), pout, buf, C.c_size_t(cap), C.byref(ln))
    check(ctx.h, st)
    proof = C.string_at(buf, ln.value)
    return (proof, out) if want_output else proof


def prove_row_attention_gqa(q, k, v, num_q_heads: int, num_kv_heads: int, seq_len: int, d_head: int, exp_table, transcript: Transcript,
                            want_output: bool = False):
    """attention.rs:386-500, the reference's argument order."""
    return prove_row_attention(q, k, v, num_q_heads, seq_len, d_head, exp_table, transcript, want_output, num_kv_heads)


def verify_row_attention(proof: bytes, k, v, num_heads: int, seq_len: int, d_head: int, transcript: Transcript, num_kv_heads: int = 0) -> bool:
    """attention.rs:279-385 (GQA: :503-590) on bincode(RowAttentionProof); as in the reference, q and the exp table are not needed."""
    ctx = transcript.ctx
    kk, pk, dk = _ptr(k); vv, pv, dv = _ptr(v)
    if dk != dv:
        raise ValueError("k and v are either both DeviceBuffers or both host arrays")
    ok = C.c_int32(0)
    buf = (C.c_uint8 * len(proof)).from_buffer_copy(proof)
    check(ctx.h, _lib.lib().zkb_verify_row_attention(ctx.h, transcript.h, buf, C.c_size_t(len(proof)), pk, pv, C.c_size_t(num_heads),
                                                     C.c_size_t(num_kv_heads), C.c_size_t(seq_len), C.c_size_t(d_head), C.c_int32(int(dk)), C.byref(ok)))
    return bool(ok.value)


def proof_size_bound(num_heads: int, seq_len: int, d_head: int) -> int:
    """Upper bound of the bincode size, for callers that allocate the output buffer themselves."""
    ls = max(1, (seq_len - 1).bit_length()); ld = max(1, (d_head - 1).bit_length())
    per_row = 4 * (6 * seq_len + d_head) + 16 * (7 * ls + 3 * ld + 8) * 4 + 1024      # six vectors of seq_len words, one of d_head, five sumchecks
    return num_heads * seq_len * per_row + 64
