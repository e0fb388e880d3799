// BLAKE3 on the device, for the reference's blake3-based commitments
// (commit_weights_fast, rust/zk_ml_prover/src/proving/weight_commitment.rs:82-107: blake3 of an
// ASCII prefix followed by the little-endian u32 buffer).
//
// The hashed stream is  prefix (0..63 bytes) || words[0..n) as LE bytes.  Chunks (1024 stream
// bytes) are independent until the tree, so one thread compresses one chunk; chunk chaining
// values are then merged level by level (adjacent pairs; an odd last node is carried up
// unchanged), which is BLAKE3's left-full binary tree.
#pragma once
#include "m31.cuh"

namespace zkb {

__constant__ u32 B3_IV[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                             0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
enum : u32 { B3_CHUNK_START = 1, B3_CHUNK_END = 2, B3_PARENT = 4, B3_ROOT = 8 };

__device__ __forceinline__ u32 b3_rotr(u32 x, int n) { return __funnelshift_r(x, x, n); }

#define B3_G(a, b, c, d, mx, my)            \
    a = a + b + (mx); d = b3_rotr(d ^ a, 16); \
    c = c + d;        b = b3_rotr(b ^ c, 12); \
    a = a + b + (my); d = b3_rotr(d ^ a, 8);  \
    c = c + d;        b = b3_rotr(b ^ c, 7);

// Compression; returns the first 8 output words (the chaining value / the first 32 digest bytes).
// Chaining value and message travel by value, in registers: through pointers they would live in
// local memory, one more round trip per block for a thread that hashes a chunk alone.
struct B3Cv { u32 v[8]; };
struct B3Msg { u32 w[16]; };
__device__ __noinline__ B3Cv b3_compress(B3Cv cv, B3Msg m, u32 counter_lo, u32 counter_hi, u32 blen, u32 flags) {
    u32 s0 = cv.v[0], s1 = cv.v[1], s2 = cv.v[2], s3 = cv.v[3], s4 = cv.v[4], s5 = cv.v[5], s6 = cv.v[6], s7 = cv.v[7];
    u32 s8 = 0x6a09e667u, s9 = 0xbb67ae85u, s10 = 0x3c6ef372u, s11 = 0xa54ff53au;
    u32 s12 = counter_lo, s13 = counter_hi, s14 = blen, s15 = flags;
    u32 w[16];
#pragma unroll
    for (int i = 0; i < 16; i++) w[i] = m.w[i];
#pragma unroll
    for (int r = 0; r < 7; r++) {
        B3_G(s0, s4, s8, s12, w[0], w[1]);   B3_G(s1, s5, s9, s13, w[2], w[3]);
        B3_G(s2, s6, s10, s14, w[4], w[5]);  B3_G(s3, s7, s11, s15, w[6], w[7]);
        B3_G(s0, s5, s10, s15, w[8], w[9]);  B3_G(s1, s6, s11, s12, w[10], w[11]);
        B3_G(s2, s7, s8, s13, w[12], w[13]); B3_G(s3, s4, s9, s14, w[14], w[15]);
        if (r < 6) {
            u32 t[16] = {w[2], w[6], w[3], w[10], w[7], w[0], w[4], w[13], w[1], w[11], w[12], w[5], w[9], w[14], w[15], w[8]};
#pragma unroll
            for (int i = 0; i < 16; i++) w[i] = t[i];
        }
    }
    B3Cv o;
    o.v[0] = s0 ^ s8;  o.v[1] = s1 ^ s9;  o.v[2] = s2 ^ s10; o.v[3] = s3 ^ s11;
    o.v[4] = s4 ^ s12; o.v[5] = s5 ^ s13; o.v[6] = s6 ^ s14; o.v[7] = s7 ^ s15;
    return o;
}

struct B3Prefix { unsigned char b[64]; u32 len; };

// Stream byte at position s (s < total): prefix bytes first, then the words as LE bytes.
__device__ __forceinline__ u32 b3_stream_byte(const B3Prefix& pre, const u32* __restrict__ words, size_t s) {
    if (s < pre.len) return pre.b[s];
    size_t d = s - pre.len;
    return (words[d >> 2] >> (8 * (d & 3))) & 0xffu;
}
// Stream word (4 bytes from position s, zero past `total`).
__device__ __forceinline__ u32 b3_stream_word(const B3Prefix& pre, const u32* __restrict__ words, size_t s, size_t total) {
    if (s >= pre.len && s + 4 <= total) {
        size_t d = s - pre.len;
        u32 sh = (u32)(d & 3);
        const u32* p = words + (d >> 2);
        if (sh == 0) return p[0];
        return __funnelshift_r(p[0], p[1], 8 * sh);
    }
    u32 w = 0;
#pragma unroll
    for (int k = 0; k < 4; k++)
        if (s + k < total) w |= b3_stream_byte(pre, words, s + k) << (8 * k);
    return w;
}

// The 16 message words of the block that starts at stream position bs.  A block that lies wholly
// inside the words (all but the first and the last of a vector) is 17 independent loads and 16
// independent funnel shifts; per-word position arithmetic would be a dependent chain of its own,
// and a lone thread pays about 11 cycles for every dependent instruction.
__device__ __forceinline__ B3Msg b3_block_words(const B3Prefix& pre, const u32* __restrict__ words, size_t bs, size_t total) {
    B3Msg m;
    if (bs >= pre.len && bs + 64 <= total) {
        const size_t d = bs - pre.len;
        const u32 sh = (u32)(d & 3) * 8;
        const u32* p = words + (d >> 2);
        if (sh == 0) {
#pragma unroll
            for (int k = 0; k < 16; k++) m.w[k] = p[k];
        } else {
            u32 t[17];
#pragma unroll
            for (int k = 0; k < 17; k++) t[k] = p[k];      // p[16] exists: byte d + 63 is inside the words
#pragma unroll
            for (int k = 0; k < 16; k++) m.w[k] = __funnelshift_r(t[k], t[k + 1], sh);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 16; k++) m.w[k] = b3_stream_word(pre, words, bs + 4 * k, total);
    }
    return m;
}

// Chaining value of chunk `ci` (or the root digest when it is the only chunk).  The message words
// of block b + 1 are fetched before block b is compressed, so that the 16 blocks of a chunk cost
// one exposed memory latency, not sixteen.
__device__ inline void b3_chunk_cv(const B3Prefix& pre, const u32* __restrict__ words, size_t total, size_t ci, bool only_chunk, u32* out8) {
    B3Cv cv;
#pragma unroll
    for (int i = 0; i < 8; i++) cv.v[i] = B3_IV[i];
    size_t start = ci * 1024;
    size_t len = total - start < 1024 ? total - start : 1024;
    u32 nblocks = len == 0 ? 1u : (u32)((len + 63) / 64);
    B3Msg cur = b3_block_words(pre, words, start, total), nxt = cur;
    for (u32 b = 0; b < nblocks; b++) {
        if (b + 1 < nblocks) nxt = b3_block_words(pre, words, start + (size_t)(b + 1) * 64, total);
        u32 blen = (u32)(len - (size_t)b * 64 < 64 ? len - (size_t)b * 64 : 64);
        u32 fl = (b == 0 ? B3_CHUNK_START : 0) | (b + 1 == nblocks ? B3_CHUNK_END : 0);
        if (only_chunk && b + 1 == nblocks) fl |= B3_ROOT;
        cv = b3_compress(cv, cur, (u32)ci, (u32)(ci >> 32), blen, fl);
        cur = nxt;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) out8[i] = cv.v[i];
}

__device__ __forceinline__ void b3_parent(const u32* left8, const u32* right8, bool root, u32* out8) {
    B3Msg m;
    B3Cv cv;
#pragma unroll
    for (int i = 0; i < 8; i++) { m.w[i] = left8[i]; m.w[8 + i] = right8[i]; cv.v[i] = B3_IV[i]; }
    cv = b3_compress(cv, m, 0, 0, 64, B3_PARENT | (root ? B3_ROOT : 0));
#pragma unroll
    for (int i = 0; i < 8; i++) out8[i] = cv.v[i];
}

// Whole hash by one CTA: `cvs` is scratch for n_chunks * 8 words in global memory.  Result (8 LE
// words = 32 digest bytes) in cvs[0..8) after the call; all threads must call.  Up to
// B3_SMEM_CHUNKS chunk values are merged in shared memory (a level is then two CTA barriers, not
// two round trips to L2).
constexpr int B3_SMEM_CHUNKS = 128;
__device__ inline void b3_hash_block(const B3Prefix& pre, const u32* __restrict__ words, size_t n_words, u32* cvs) {
    __shared__ u32 cvs_sh[B3_SMEM_CHUNKS * 8];
    size_t total = pre.len + n_words * 4;
    size_t n_chunks = total == 0 ? 1 : (total + 1023) / 1024;
    u32* lv = n_chunks <= (size_t)B3_SMEM_CHUNKS ? cvs_sh : cvs;
    for (size_t c = threadIdx.x; c < n_chunks; c += blockDim.x) {
        u32 cv[8];
        b3_chunk_cv(pre, words, total, c, n_chunks == 1, cv);
#pragma unroll
        for (int i = 0; i < 8; i++) lv[c * 8 + i] = cv[i];
    }
    __syncthreads();
    size_t n = n_chunks;
    while (n > 1) {
        size_t pairs = n / 2, next = (n + 1) / 2;
        u32 outv[8];
        // each thread merges pair t -> slot t; read before anyone overwrites (two-phase)
        for (size_t base = 0; base < next; base += blockDim.x) {
            size_t t = base + threadIdx.x;
            bool act = t < next;
            if (act) {
                if (t < pairs) b3_parent(lv + 2 * t * 8, lv + (2 * t + 1) * 8, next == 1, outv);
                else {
#pragma unroll
                    for (int i = 0; i < 8; i++) outv[i] = lv[2 * t * 8 + i];
                }
            }
            __syncthreads();
            if (act) {
#pragma unroll
                for (int i = 0; i < 8; i++) lv[t * 8 + i] = outv[i];
            }
            __syncthreads();
        }
        n = next;
    }
    if (lv != cvs) {
        if (threadIdx.x < 8) cvs[threadIdx.x] = lv[threadIdx.x];
        __syncthreads();
    }
}

}  // namespace zkb
