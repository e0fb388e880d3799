// "Transcript script" kernel: a short list of absorb / squeeze operations executed by one
// warp in a single launch (lane 0 runs the SHA-256 chain, the other lanes stage device data
// into shared memory), so that the protocol glue between sumchecks costs one launch instead
// of one per operation.  Mirrors Transcript::{absorb, absorb_many, absorb_bytes, squeeze,
// squeeze_ef} (rust/zk_ml_prover/src/proving/sumcheck.rs:121-204).
#pragma once
#include "transcript.cuh"
#include "blake3.cuh"

namespace zkb {

struct ByteChunk { unsigned char b[256]; };

__global__ void tr_init_kernel(TrState* st) {
    u32 h[8];
    tr_iv(h);
    for (int i = 0; i < 8; i++) st->h[i] = h[i];
    st->buflen = 0; st->_pad = 0; st->total = 0;
    for (int i = 0; i < 64; i++) st->buf[i] = 0;
}
__global__ void tr_absorb_bytes_kernel(TrState* st, ByteChunk c, u32 n) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    Tr tr;
    tr_load(tr, st, trbuf);
    tr_absorb_bytes(tr, c.b, n);
    tr_store(tr, st);
}
// One warp: lanes expand the message schedules, lane 0 runs the hash chain.
__global__ void __launch_bounds__(32) tr_absorb_words_kernel(TrState* st, const u32* __restrict__ v, size_t n) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ u32 tile[512];
    __shared__ u32 kw[32 * SHA_KW_STRIDE];
    Tr tr;
    tr.buf = trbuf; tr.buflen = 0; tr.total = 0;
    if (threadIdx.x == 0) tr_load(tr, st, trbuf);
    __syncwarp();
    tr_absorb_stream_warp(tr, (u32)n, [=](u32 g) -> u32 { return v[g]; }, tile, kw);
    if (threadIdx.x == 0) tr_store(tr, st);
}
__global__ void tr_squeeze_kernel(TrState* st, u32* out, u32 count) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    Tr tr;
    tr_load(tr, st, trbuf);
    for (u32 i = 0; i < count; i++) out[i] = tr_squeeze(tr);
    tr_store(tr, st);
}


enum TrOpKind : u32 {
    TROP_BYTES = 0,        // absorb `n` bytes stored inline at `inline_off`
    TROP_WORDS_DEV = 1,    // absorb `n` u32 from device memory, then (pad - n) zero words
    TROP_PAIRS_DEV = 2,    // absorb a[i], b[i] interleaved, i < n (LogUp statement, lookup.rs:655-658)
    TROP_SQUEEZE = 3,      // squeeze `n` base-field challenges to ptr
    TROP_BYTES_DEV = 4,    // absorb `n` bytes from device memory (word aligned, n % 4 == 0)
    TROP_WORD_DEV_N = 5,   // absorb the u32 count stored at ptr[0] (device-resident length)
    TROP_BYTES_DEV_N = 6   // absorb ptr[0] bytes stored from ptr + 1 on (device-resident, any length below 256)
};
struct TrOp {
    u32 kind;
    u32 n;
    u32 pad;          // TROP_WORDS_DEV: total words including zero padding
    u32 inline_off;   // TROP_BYTES
    const u32* ptr;   // device source / squeeze destination
    const u32* ptr2;  // TROP_PAIRS_DEV second array
};
constexpr int TRSCRIPT_MAX_OPS = 12;
constexpr int TRSCRIPT_INLINE = 256;
struct TrScript {
    TrOp ops[TRSCRIPT_MAX_OPS];
    unsigned char inl[TRSCRIPT_INLINE];
    u32 nops;
};

constexpr int TRSCRIPT_THREADS = 64;      // warp 0 advances the transcript, warp 1 prefetches and expands (see tr_absorb_stream_2w)
__global__ void __launch_bounds__(TRSCRIPT_THREADS) tr_script_kernel(TrState* st, TrScript sc) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ u32 tile[2 * 512];
    __shared__ u32 kw[2 * 32 * SHA_KW_STRIDE];
    __shared__ u32 bc[1];
    ZKB_STAMP_BEGIN
    Tr tr;
    tr.buf = trbuf; tr.buflen = 0; tr.total = 0;
    if (threadIdx.x == 0) tr_load(tr, st, trbuf);
    for (u32 o = 0; o < sc.nops; o++) {
        const TrOp& op = sc.ops[o];
        if (op.kind == TROP_BYTES) {
            if (threadIdx.x == 0) tr_absorb_bytes(tr, sc.inl + op.inline_off, op.n);
        } else if (op.kind == TROP_SQUEEZE) {
            if (threadIdx.x == 0) {
                u32* dst = const_cast<u32*>(op.ptr);
                for (u32 i = 0; i < op.n; i++) dst[i] = tr_squeeze(tr);
            }
        } else if (op.kind == TROP_WORD_DEV_N) {
            if (threadIdx.x == 0) tr_absorb_u32(tr, op.ptr[0]);
        } else if (op.kind == TROP_BYTES_DEV_N) {
            if (threadIdx.x == 0) {
                u32 nb = op.ptr[0];
                if (nb > 255) nb = 255;
                tr_absorb_bytes(tr, reinterpret_cast<const unsigned char*>(op.ptr + 1), nb);
            }
        } else {
            // streamed absorbs: total logical words
            u32 total = op.kind == TROP_WORDS_DEV ? op.pad : (op.kind == TROP_PAIRS_DEV ? 2 * op.n : op.n / 4);
            const u32 kind = op.kind, n = op.n;
            const u32* p1 = op.ptr;
            const u32* p2 = op.ptr2;
            tr_absorb_stream_2w(tr, total, [=](u32 g) -> u32 {
                if (kind == TROP_WORDS_DEV) return g < n ? p1[g] : 0u;
                if (kind == TROP_PAIRS_DEV) return (g & 1) ? p2[g >> 1] : p1[g >> 1];
                return p1[g];
            }, reinterpret_cast<u32*>(trbuf), tile, kw, bc);
        }
    }
    if (threadIdx.x == 0) tr_store(tr, st);
    ZKB_STAMP_END(st, 0);
}

// blake3(prefix || words) by one CTA, result to `root_out` (8 words); optionally absorbed into
// the transcript right away.  `n_words_dev` (if non-null) overrides n_words with a
// device-resident length (LogUp's number of active table entries).
__global__ void __launch_bounds__(1024) b3_commit_kernel(B3Prefix pre, const u32* __restrict__ words, u32 n_words,
                                                         const u32* n_words_dev, u32* cvs_scratch, u32* root_out, TrState* absorb_into) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    if (n_words_dev) n_words = n_words_dev[0];
    b3_hash_block(pre, words, n_words, cvs_scratch);
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; i++) root_out[i] = cvs_scratch[i];
        if (absorb_into) {
            Tr tr;
            tr_load(tr, absorb_into, trbuf);
            for (int i = 0; i < 8; i++) tr_absorb_u32(tr, cvs_scratch[i]);
            tr_store(tr, absorb_into);
        }
    }
}

// Large buffers: chunk chaining values by the whole grid, then one merge launch per level.
__global__ void b3_chunks_kernel(B3Prefix pre, const u32* __restrict__ words, size_t n_words, u32* cvs) {
    size_t total = pre.len + n_words * 4;
    size_t n_chunks = total == 0 ? 1 : (total + 1023) / 1024;
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += (size_t)gridDim.x * blockDim.x) {
        u32 cv[8];
        b3_chunk_cv(pre, words, total, c, n_chunks == 1, cv);
        for (int i = 0; i < 8; i++) cvs[c * 8 + i] = cv[i];
    }
}
__global__ void b3_merge_kernel(const u32* __restrict__ in, size_t n, u32* out) {
    size_t pairs = n / 2, next = (n + 1) / 2;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < next; t += (size_t)gridDim.x * blockDim.x) {
        u32 o[8];
        if (t < pairs) b3_parent(in + 2 * t * 8, in + (2 * t + 1) * 8, next == 1, o);
        else for (int i = 0; i < 8; i++) o[i] = in[2 * t * 8 + i];
        for (int i = 0; i < 8; i++) out[t * 8 + i] = o[i];
    }
}

}  // namespace zkb
