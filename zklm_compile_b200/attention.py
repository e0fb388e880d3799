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
    """attention.rs:116-276 -> bincode(RowAttentionProof) [, the op's output].
    `transcript` may be a Context instead of a Transcript: then only the rows are proved and the caller absorbs the dimensions and
    every row's scores and outputs into its own transcript (`caller_transcript_stream` gives that byte stream)."""
    ctx = transcript.ctx if isinstance(transcript, Transcript) else transcript
    tr_h = transcript.h if isinstance(transcript, Transcript) else None
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
    buf = getattr(ctx, "_attention_out", None)            # the output buffer is kept with the context: a fresh one of this size costs
    if buf is None or len(buf) < cap:                     # a millisecond of page faults, comparable to the rows' proof itself
        buf = ctx._attention_out = (C.c_uint8 * cap)()
    ln = C.c_size_t()
    st = _lib.lib().zkb_prove_row_attention_gqa(ctx.h, tr_h, *ptrs[:3], C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len),
                                                C.c_size_t(d_head), ptrs[3], C.c_size_t(n_table), C.c_int32(on_dev), pout, buf, C.c_size_t(len(buf)), C.byref(ln))
    check(ctx.h, st)
    proof = C.string_at(buf, ln.value)
    return (proof, out) if want_output else proof


def prove_row_attention_gqa(q, k, v, num_q_heads: int, num_kv_heads: int, seq_len: int, d_head: int, exp_table, transcript: Transcript,
                            want_output: bool = False):
    """attention.rs:386-500, the reference's argument order."""
    return prove_row_attention(q, k, v, num_q_heads, seq_len, d_head, exp_table, transcript, want_output, num_kv_heads)


def verify_row_attention(proof: bytes, k, v, num_heads: int, seq_len: int, d_head: int, transcript: Transcript, num_kv_heads: int = 0) -> bool:
    """attention.rs:279-385 (GQA: :503-590) on bincode(RowAttentionProof); as in the reference, q and the exp table are not needed.
    `transcript` may be a Context: the rows are checked and the caller's transcript is left to the caller."""
    ctx = transcript.ctx if isinstance(transcript, Transcript) else transcript
    tr_h = transcript.h if isinstance(transcript, Transcript) else None
    kk, pk, dk = _ptr(k); vv, pv, dv = _ptr(v)
    if dk != dv:
        raise ValueError("k and v are either both DeviceBuffers or both host arrays")
    ok = C.c_int32(0)
    buf = (C.c_uint8 * len(proof)).from_buffer_copy(proof)
    check(ctx.h, _lib.lib().zkb_verify_row_attention(ctx.h, tr_h, buf, C.c_size_t(len(proof)), pk, pv, C.c_size_t(num_heads),
                                                     C.c_size_t(num_kv_heads), C.c_size_t(seq_len), C.c_size_t(d_head), C.c_int32(int(dk)), C.byref(ok)))
    return bool(ok.value)


def caller_transcript_stream(proof: bytes, num_heads: int, seq_len: int, d_head: int, num_kv_heads: int = 0) -> bytes:
    """What the caller's transcript absorbs around a row-attention proof (attention.rs:140-143, 254-265; GQA :403-406): the dimensions as
    u32 LE, then every row's scores and outputs, read from the proof bytes.  For callers that keep their transcript on the host."""
    import struct
    out = [struct.pack("<I", num_heads)]
    if num_kv_heads:
        out.append(struct.pack("<I", num_kv_heads))
    out.append(struct.pack("<II", seq_len, d_head))
    at = 8
    u64 = lambda: struct.unpack_from("<Q", proof, at)[0]

    def skip_vec():
        nonlocal at
        n = u64(); at += 8 + 4 * n

    def skip_sumcheck():
        nonlocal at
        rounds = u64(); at += 8
        for _ in range(rounds):
            skip_vec()
        skip_vec()

    for _ in range(num_heads):
        at += 8                                            # rows of this head
        for _ in range(seq_len):
            skip_sumcheck(); at += 8; skip_vec(); skip_vec()                   # score_proof
            at += 2 * (32 + 8 + 8 + 4); skip_sumcheck(); at += 16               # lookup: commitments, sumcheck, finals, alpha, beta
            skip_vec(); skip_vec(); skip_vec(); at += 32                        # inputs, outputs, multiplicities, digest
            at += 4; skip_sumcheck(); at += 8; skip_sumcheck(); at += 12 + 4    # sum, sum proof + finals, output proof + finals, inv_s
            skip_vec(); skip_vec()                                              # e_values, y_values
            skip_sumcheck(); at += 8; skip_vec(); skip_vec()                   # output_proof
            n = u64(); scores = proof[at + 8:at + 8 + 4 * n]; at += 8 + 4 * n
            skip_vec()                                                          # attn_weights
            n = u64(); outp = proof[at + 8:at + 8 + 4 * n]; at += 8 + 4 * n
            out.append(scores); out.append(outp)
    return b"".join(out)


def proof_size_bound(num_heads: int, seq_len: int, d_head: int) -> int:
    """Upper bound of the bincode size, for callers that allocate the output buffer themselves."""
    ls = max(1, (seq_len - 1).bit_length()); ld = max(1, (d_head - 1).bit_length())
    per_row = 4 * (6 * seq_len + d_head) + 16 * (7 * ls + 3 * ld + 8) * 4 + 1024      # six vectors of seq_len words, one of d_head, five sumchecks
    return num_heads * seq_len * per_row + 64
