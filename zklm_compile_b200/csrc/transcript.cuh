// Device-resident Fiat-Shamir transcript: a SHA-256 stream that lives in global memory and is
// advanced by one thread of whichever kernel finishes a protocol step, so challenges never
// travel to the host.  Mirrors the reference `Transcript`
// (rust/zk_ml_prover/src/proving/sumcheck.rs:110-206):
//   new(label)      stream = label bytes
//   absorb(u32)     4 little-endian bytes; absorb_bytes(raw)
//   squeeze()       d = SHA-256(stream); stream := d; first of the four little-endian u64
//                   windows of d below 2^64 - 4, reduced mod p
//   squeeze_ef()    four squeezes -> (re c0, im c0, re c1, im c1)
#pragma once
#include "m31.cuh"

namespace zkb {

#ifdef ZKB_STAMP
// Experiment build only: start / end time stamps of the serial hash kernels, by transcript.
struct StampRec { const void* key; unsigned long long t0, t1; unsigned kind, smid; };
constexpr unsigned STAMP_CAP = 1u << 16;
__device__ StampRec g_stamps[STAMP_CAP];
__device__ unsigned g_stamp_n;
__device__ __forceinline__ unsigned long long stamp_now() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void stamp_put(const void* key, unsigned kind, unsigned long long t0) {
    unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    unsigned i = atomicAdd(&g_stamp_n, 1u);
    if (i < STAMP_CAP) g_stamps[i] = StampRec{key, t0, stamp_now(), kind, smid};
}
#define ZKB_STAMP_BEGIN unsigned long long stamp_t0 = stamp_now();
#define ZKB_STAMP_END(key, kind) do { if (threadIdx.x == 0) stamp_put(key, kind, stamp_t0); } while (0)
#else
#define ZKB_STAMP_BEGIN
#define ZKB_STAMP_END(key, kind) do { } while (0)
#endif


// Global-memory image of the stream.  `buf` holds the bytes not yet compressed.
struct TrState {
    u32 h[8];
    u32 buflen;      // 0..63
    u32 _pad;
    u64 total;       // bytes absorbed into the current SHA-256 stream
    unsigned char buf[64];
};

__constant__ u32 SHA_K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

__device__ __forceinline__ u32 rotr32(u32 x, int n) { return __funnelshift_r(x, x, n); }
__device__ __forceinline__ u32 bswap32(u32 x) { return __byte_perm(x, 0, 0x0123); }

// One SHA-256 compression.  The chaining value travels in registers (by value), the message
// block is read from 16 little-endian words of shared memory and byte-swapped on the fly; the
// 64 rounds are fully unrolled with the working variables renamed instead of moved, and the
// message schedule is kept in a 16-register window.  One thread runs this; the rounds are a
// strict dependency chain, so the remaining lever is instruction count, not parallelism.
struct Sha8 { u32 v[8]; };

// One round.  A lone warp issues an integer instruction about every two cycles (measured on B200:
// eight independent lop3 or shf per iteration run at 2.0 - 2.2 cycles each, a dependent one at 4.4),
// so a compression is bound by its instruction count, not by the dependency chain: the boolean
// functions are single lop3 instructions, and the additions are written as multiply-adds by one in
// the association  x = h + kw + ch,  e' = x + d + s1,  a' = x + maj + s0 + s1,  which ptxas places
// best (30.6 cycles per round against 33.8 for the textbook form).
__device__ __forceinline__ u32 sha_xor3(u32 a, u32 b, u32 c) { u32 r; asm("lop3.b32 %0, %1, %2, %3, 0x96;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r; }
__device__ __forceinline__ u32 sha_ch(u32 e, u32 f, u32 g) { u32 r; asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(r) : "r"(e), "r"(f), "r"(g)); return r; }
__device__ __forceinline__ u32 sha_maj(u32 a, u32 b, u32 c) { u32 r; asm("lop3.b32 %0, %1, %2, %3, 0xE8;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r; }
__device__ __forceinline__ u32 sha_add(u32 a, u32 b) { u32 r; asm("mad.lo.u32 %0, %1, 1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r; }
#define ZKB_SHA_RND(a, b, c, d, e, f, g, h, kw)                                   \
    {                                                                             \
        const u32 ch_ = sha_ch(e, f, g);                                          \
        const u32 mj_ = sha_maj(a, b, c);                                         \
        const u32 s1_ = sha_xor3(rotr32(e, 6), rotr32(e, 11), rotr32(e, 25));     \
        const u32 s0_ = sha_xor3(rotr32(a, 2), rotr32(a, 13), rotr32(a, 22));     \
        const u32 x_ = sha_add(sha_add(h, (kw)), ch_);                            \
        const u32 z_ = sha_add(x_, mj_);                                          \
        d = sha_add(sha_add(x_, d), s1_);                                         \
        h = sha_add(sha_add(z_, s0_), s1_);                                       \
    }
#define ZKB_SHA_SCHED(i) \
    (w[(i) & 15] += (rotr32(w[((i) + 1) & 15], 7) ^ rotr32(w[((i) + 1) & 15], 18) ^ (w[((i) + 1) & 15] >> 3)) + w[((i) + 9) & 15] + \
                    (rotr32(w[((i) + 14) & 15], 17) ^ rotr32(w[((i) + 14) & 15], 19) ^ (w[((i) + 14) & 15] >> 10)))

__device__ __noinline__ Sha8 sha256_compress(Sha8 hin, const u32* __restrict__ blk) {
    u32 w[16];
#pragma unroll
    for (int i = 0; i < 16; i++) w[i] = bswap32(blk[i]);
    u32 a = hin.v[0], b = hin.v[1], c = hin.v[2], d = hin.v[3], e = hin.v[4], f = hin.v[5], g = hin.v[6], h = hin.v[7];
#define ZKB_SHA_RND8(k0, i)                                                 \
    ZKB_SHA_RND(a, b, c, d, e, f, g, h, SHA_K[(k0) + (i)] + w[(i)]);         \
    ZKB_SHA_RND(h, a, b, c, d, e, f, g, SHA_K[(k0) + (i) + 1] + w[(i) + 1]); \
    ZKB_SHA_RND(g, h, a, b, c, d, e, f, SHA_K[(k0) + (i) + 2] + w[(i) + 2]); \
    ZKB_SHA_RND(f, g, h, a, b, c, d, e, SHA_K[(k0) + (i) + 3] + w[(i) + 3]); \
    ZKB_SHA_RND(e, f, g, h, a, b, c, d, SHA_K[(k0) + (i) + 4] + w[(i) + 4]); \
    ZKB_SHA_RND(d, e, f, g, h, a, b, c, SHA_K[(k0) + (i) + 5] + w[(i) + 5]); \
    ZKB_SHA_RND(c, d, e, f, g, h, a, b, SHA_K[(k0) + (i) + 6] + w[(i) + 6]); \
    ZKB_SHA_RND(b, c, d, e, f, g, h, a, SHA_K[(k0) + (i) + 7] + w[(i) + 7]);
    ZKB_SHA_RND8(0, 0)
    ZKB_SHA_RND8(0, 8)
    // Rounds 16..63 as a loop of three 16-round bodies (the schedule window and the renamed working
    // variables both come back to the same registers every 16 rounds): the loop body stays in the
    // instruction cache next to whatever else runs on the SM, a fully unrolled compression does not.
#pragma unroll 1
    for (int k0 = 16; k0 < 64; k0 += 16) {
#pragma unroll
        for (int j = 0; j < 8; j++) ZKB_SHA_SCHED(j);
        ZKB_SHA_RND8(k0, 0)
#pragma unroll
        for (int j = 8; j < 16; j++) ZKB_SHA_SCHED(j);
        ZKB_SHA_RND8(k0, 8)
    }
#undef ZKB_SHA_RND8
    Sha8 o;
    o.v[0] = hin.v[0] + a; o.v[1] = hin.v[1] + b; o.v[2] = hin.v[2] + c; o.v[3] = hin.v[3] + d;
    o.v[4] = hin.v[4] + e; o.v[5] = hin.v[5] + f; o.v[6] = hin.v[6] + g; o.v[7] = hin.v[7] + h;
    return o;
}

// The 64 rounds alone, with K[t] + W[t] read from shared memory.  The message schedule of a
// block depends only on the block, not on the chaining value, so when many known blocks are
// absorbed in a row the lanes of a warp expand 32 schedules side by side and one lane then runs
// only the (inherently serial) rounds.
constexpr int SHA_KW_STRIDE = 65;    // padded so 32 lanes writing their own row do not share a bank
__device__ __noinline__ Sha8 sha256_rounds(Sha8 hin, const u32* __restrict__ kw) {
    u32 a = hin.v[0], b = hin.v[1], c = hin.v[2], d = hin.v[3], e = hin.v[4], f = hin.v[5], g = hin.v[6], h = hin.v[7];
#pragma unroll 1
    for (int i = 0; i < 64; i += 16) {
#pragma unroll
        for (int j = 0; j < 16; j += 8) {
            ZKB_SHA_RND(a, b, c, d, e, f, g, h, kw[i + j]);
            ZKB_SHA_RND(h, a, b, c, d, e, f, g, kw[i + j + 1]);
            ZKB_SHA_RND(g, h, a, b, c, d, e, f, kw[i + j + 2]);
            ZKB_SHA_RND(f, g, h, a, b, c, d, e, kw[i + j + 3]);
            ZKB_SHA_RND(e, f, g, h, a, b, c, d, kw[i + j + 4]);
            ZKB_SHA_RND(d, e, f, g, h, a, b, c, kw[i + j + 5]);
            ZKB_SHA_RND(c, d, e, f, g, h, a, b, kw[i + j + 6]);
            ZKB_SHA_RND(b, c, d, e, f, g, h, a, kw[i + j + 7]);
        }
    }
    Sha8 o;
    o.v[0] = hin.v[0] + a; o.v[1] = hin.v[1] + b; o.v[2] = hin.v[2] + c; o.v[3] = hin.v[3] + d;
    o.v[4] = hin.v[4] + e; o.v[5] = hin.v[5] + f; o.v[6] = hin.v[6] + g; o.v[7] = hin.v[7] + h;
    return o;
}
// Lane-local: expand the schedule of one block (16 big-endian words) into K + W.
__device__ __forceinline__ void sha256_expand_kw(const u32* __restrict__ blk_be, u32* kw) {
    u32 w[16];
#pragma unroll
    for (int i = 0; i < 16; i++) { w[i] = blk_be[i]; kw[i] = SHA_K[i] + w[i]; }
#pragma unroll
    for (int i = 16; i < 64; i++) { ZKB_SHA_SCHED(i); kw[i] = SHA_K[i] + w[i & 15]; }
}

// Working copy used by the single thread that advances the transcript.  `buf` points to
// TR_SCRATCH_BYTES of 16-byte-aligned shared memory: the 64-byte message block followed by 64
// words for the expanded schedule (K + W) of the block being compressed.
constexpr int TR_SCRATCH_BYTES = 64 + 64 * 4;

struct Tr {
    u32 h[8];
    u32 buflen;
    u64 total;
    unsigned char* buf;
};

__device__ __forceinline__ void tr_iv(u32 h[8]) {
    h[0] = 0x6a09e667u; h[1] = 0xbb67ae85u; h[2] = 0x3c6ef372u; h[3] = 0xa54ff53au;
    h[4] = 0x510e527fu; h[5] = 0x9b05688cu; h[6] = 0x1f83d9abu; h[7] = 0x5be0cd19u;
}
__device__ __forceinline__ void tr_load(Tr& t, const TrState* g, unsigned char* scratch) {
#pragma unroll
    for (int i = 0; i < 8; i++) t.h[i] = g->h[i];
    t.buflen = g->buflen;
    t.total = g->total;
    t.buf = scratch;
    const u32* src = reinterpret_cast<const u32*>(g->buf);
    u32* dst = reinterpret_cast<u32*>(scratch);
#pragma unroll
    for (int i = 0; i < 16; i++) dst[i] = src[i];
}
__device__ __forceinline__ void tr_store(const Tr& t, TrState* g) {
#pragma unroll
    for (int i = 0; i < 8; i++) g->h[i] = t.h[i];
    g->buflen = t.buflen;
    g->total = t.total;
    u32* dst = reinterpret_cast<u32*>(g->buf);
    const u32* src = reinterpret_cast<const u32*>(t.buf);
#pragma unroll
    for (int i = 0; i < 16; i++) dst[i] = src[i];
}
__device__ __forceinline__ void tr_flush_block(Tr& t) {
    Sha8 h;
#pragma unroll
    for (int i = 0; i < 8; i++) h.v[i] = t.h[i];
    // Measured on B200 (one thread, ~11 cycles between dependent instructions): the fused
    // schedule + rounds below takes ~3030 cycles, expanding first and then running the rounds ~3830.
    h = sha256_compress(h, reinterpret_cast<const u32*>(t.buf));
#pragma unroll
    for (int i = 0; i < 8; i++) t.h[i] = h.v[i];
    t.buflen = 0;
}
__device__ __forceinline__ void tr_absorb_byte(Tr& t, unsigned char c) {
    t.buf[t.buflen++] = c;
    t.total++;
    if (t.buflen == 64) tr_flush_block(t);
}
__device__ __forceinline__ void tr_absorb_u32(Tr& t, u32 v) {
    if ((t.buflen & 3) == 0) {           // aligned fast path: one word store
        *reinterpret_cast<u32*>(t.buf + t.buflen) = v;
        t.buflen += 4;
        t.total += 4;
        if (t.buflen == 64) tr_flush_block(t);
    } else {
        tr_absorb_byte(t, (unsigned char)v);
        tr_absorb_byte(t, (unsigned char)(v >> 8));
        tr_absorb_byte(t, (unsigned char)(v >> 16));
        tr_absorb_byte(t, (unsigned char)(v >> 24));
    }
}
// N words at once; when the stream is word-aligned (the common case) this is N plain stores
// plus at most one compression, instead of N rounds of per-byte bookkeeping.
template <int N>
__device__ __forceinline__ void tr_absorb_words(Tr& t, const u32* w) {
    static_assert(N <= 16, "at most one block boundary inside");
    if ((t.buflen & 3) == 0) {
        u32* bw = reinterpret_cast<u32*>(t.buf);
        const u32 pos = t.buflen >> 2;
        const u32 room = 16 - pos;                     // words that still fit into the open block (1..16)
#pragma unroll
        for (int i = 0; i < N; i++) if ((u32)i < room) bw[pos + i] = w[i];
        if ((u32)N >= room) {
            t.buflen = 64;
            tr_flush_block(t);
#pragma unroll
            for (int i = 0; i < N; i++) if ((u32)i >= room) bw[i - room] = w[i];
            t.buflen = ((u32)N - room) << 2;
        } else {
            t.buflen = (pos + N) << 2;
        }
        t.total += 4 * N;
    } else {
#pragma unroll
        for (int i = 0; i < N; i++) tr_absorb_u32(t, w[i]);
    }
}
__device__ __forceinline__ void tr_absorb_fe(Tr& t, Fe v) {
    u32 w[4] = {v.x, v.y, v.z, v.w};
    tr_absorb_words<4>(t, w);
}
__device__ __forceinline__ void tr_absorb_el(Tr& t, Fp v) { tr_absorb_u32(t, v.v); }
__device__ __forceinline__ void tr_absorb_el(Tr& t, Fe v) { tr_absorb_fe(t, v); }
__device__ inline void tr_absorb_bytes(Tr& t, const unsigned char* p, u32 n) {
    for (u32 i = 0; i < n; i++) tr_absorb_byte(t, p[i]);
}

// Pad, compress, and restart the stream with the 32-byte digest as its first bytes.  Written
// without loops whose trip count depends on the position: on a lone thread every dependent
// instruction costs about 11 cycles, so the zero fill is fourteen predicated stores, not a counted loop.
__device__ __forceinline__ void tr_finalize_reseed(Tr& t, u32 digest_be[8]) {
    u64 bits = t.total * 8;
    u32 n = t.buflen;
    u32* bw = reinterpret_cast<u32*>(t.buf);
    if ((n & 3) == 0) {
        bw[n >> 2] = 0x00000080u;                      // 0x80 and three zero bytes
        n += 4;
    } else {
        t.buf[n++] = 0x80;
        while (n & 3) t.buf[n++] = 0;
    }
    u32 first = n >> 2;                                // first word still to be zeroed
    if (n > 56) {
#pragma unroll
        for (u32 i = 14; i < 16; i++) if (i >= first) bw[i] = 0;
        tr_flush_block(t);
        first = 0;
    }
#pragma unroll
    for (u32 i = 0; i < 14; i++) if (i >= first) bw[i] = 0;
    bw[14] = bswap32((u32)(bits >> 32));
    bw[15] = bswap32((u32)bits);
    tr_flush_block(t);
#pragma unroll
    for (int i = 0; i < 8; i++) digest_be[i] = t.h[i];
    tr_iv(t.h);
#pragma unroll
    for (int i = 0; i < 8; i++) bw[i] = bswap32(digest_be[i]);   // digest bytes in stream order
    t.buflen = 32;
    t.total = 32;
}
__device__ __forceinline__ u32 tr_squeeze(Tr& t) {
    for (int guard = 0; guard < 64; guard++) {        // all four windows rejecting has probability 2^-248
        u32 d[8];
        if (t.buflen == 32 && t.total == 32) {
            // stream == one 32-byte digest (the state right after a squeeze): the padded block is fixed
            u32* bw = reinterpret_cast<u32*>(t.buf);
            bw[8] = 0x00000080u;
#pragma unroll
            for (int i = 9; i < 15; i++) bw[i] = 0;
            bw[15] = 0x00010000u;                     // 256 bits, big-endian
            tr_flush_block(t);
#pragma unroll
            for (int i = 0; i < 8; i++) d[i] = t.h[i];
            tr_iv(t.h);
#pragma unroll
            for (int i = 0; i < 8; i++) bw[i] = bswap32(d[i]);
            t.buflen = 32;
        } else {
            tr_finalize_reseed(t, d);
        }
#pragma unroll
        for (int c = 0; c < 4; c++) {
            u64 raw = (u64)bswap32(d[2 * c]) | ((u64)bswap32(d[2 * c + 1]) << 32);
            if (raw < 0xfffffffffffffffcull) return red64(raw);
        }
    }
    return 0;
}
__device__ __forceinline__ Fe tr_squeeze_fe(Tr& t) {
    Fe r;
    r.x = tr_squeeze(t); r.y = tr_squeeze(t); r.z = tr_squeeze(t); r.w = tr_squeeze(t);
    return r;
}
__device__ __forceinline__ void tr_squeeze_el(Tr& t, Fp& r) { r.v = tr_squeeze(t); }
__device__ __forceinline__ void tr_squeeze_el(Tr& t, Fe& r) { r = tr_squeeze_fe(t); }

// Warp-cooperative absorb of `total` u32 words produced by load(g), g in [0, total) (any lane may
// call load).  `tr` is meaningful in lane 0 only; tile (512 words) and kw (32 * SHA_KW_STRIDE
// words) are shared-memory scratch.  Must be called by all 32 lanes of one warp.
template <class Load>
__device__ __forceinline__ void tr_absorb_stream_warp_aligned(Tr& tr, u32 total, Load load, u32* bufw, u32 have, u32* tile, u32* kw) {
    const int lane = threadIdx.x & 31;
    u32 pos = 0;
    while (have + (total - pos) >= 16) {
        u32 nb = (have + (total - pos)) / 16;
        if (nb > 32) nb = 32;
        for (u32 j = lane; j < nb * 16; j += 32) tile[j] = bswap32(j < have ? bufw[j] : load(pos + j - have));
        __syncwarp();
        if ((u32)lane < nb) sha256_expand_kw(tile + lane * 16, kw + lane * SHA_KW_STRIDE);
        __syncwarp();
        if (lane == 0) {
            Sha8 h;
#pragma unroll
            for (int i = 0; i < 8; i++) h.v[i] = tr.h[i];
            for (u32 b = 0; b < nb; b++) h = sha256_rounds(h, kw + b * SHA_KW_STRIDE);
#pragma unroll
            for (int i = 0; i < 8; i++) tr.h[i] = h.v[i];
        }
        __syncwarp();
        pos += nb * 16 - have;
        have = 0;
    }
    const u32 rest = total - pos;
    for (u32 j = lane; j < rest; j += 32) bufw[have + j] = load(pos + j);
    __syncwarp();
    if (lane == 0) { tr.buflen = (have + rest) * 4; tr.total += (u64)total * 4; }
}
// A stream that holds 4 * have + s bytes (s = 1..3) takes the words shifted by s bytes: stream word i
// is the funnel shift of data words i - 1 and i, the s pending bytes standing in for word -1, and the
// top s bytes of the last word stay pending.  The blocks are then hashed exactly like aligned ones.
template <class Load>
__device__ __forceinline__ void tr_absorb_stream_warp(Tr& tr, u32 total, Load load, u32* tile, u32* kw) {
    const int lane = threadIdx.x & 31;
    __syncwarp();                      // lane 0's earlier writes to the stream buffer become visible
    const u32 buflen = __shfl_sync(0xffffffffu, tr.buflen, 0);
    u32* bufw = reinterpret_cast<u32*>(__shfl_sync(0xffffffffu, (unsigned long long)tr.buf, 0));
    const u32 s = buflen & 3, have = buflen >> 2;
    if (s == 0) { tr_absorb_stream_warp_aligned(tr, total, load, bufw, have, tile, kw); return; }
    if (total == 0) return;
    const u32 sh = 8 * s;
    const u32 pend = bufw[have] << (32 - sh);
    __syncwarp();
    tr_absorb_stream_warp_aligned(tr, total, [=](u32 g) -> u32 { return __funnelshift_l(g ? load(g - 1) : pend, load(g), sh); },
                                  bufw, have, tile, kw);
    if (lane == 0) {
        bufw[tr.buflen >> 2] = load(total - 1) >> (32 - sh);
        tr.buflen += s;
    }
    __syncwarp();
}

// The same absorb for a CTA of two warps with the loads and the schedule expansion taken off the
// hash chain: while lane 0 of warp 0 runs the rounds of one batch (up to 32 blocks, about 35 us),
// warp 1 fetches the next batch's words and expands its schedules into the other half of the
// double-buffered scratch; the two meet at a CTA barrier per batch.  Called by all 64 threads with
// identical arguments; `tr` is meaningful in thread 0; `bufw` is the stream buffer (shared
// memory) that tr.buf points to; tile holds 2 x 512 words, kw 2 x 32 x SHA_KW_STRIDE, bc 1 word.
template <class Load>
__device__ __forceinline__ void tr_absorb_stream_2w_aligned(Tr& tr, u32 total, Load load, u32* bufw, u32 have, u32* tile, u32* kw) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto produce = [&](u32 slot, u32 have_, u32 pos, u32 nb) {   // warp 1: words [pos, ...) after `have_` buffered ones
        u32* t = tile + slot * 512;
        u32* k = kw + slot * 32 * SHA_KW_STRIDE;
        for (u32 j = lane; j < nb * 16; j += 32) t[j] = bswap32(j < have_ ? bufw[j] : load(pos + j - have_));
        __syncwarp();
        if ((u32)lane < nb) sha256_expand_kw(t + lane * 16, k + lane * SHA_KW_STRIDE);
    };
    u32 pos = 0;
    u32 nb = (have + total) / 16;
    if (nb > 32) nb = 32;
    if (nb && warp == 1) produce(0, have, 0, nb);
    __syncthreads();
    u32 slot = 0;
    while (nb) {
        const u32 next_pos = pos + nb * 16 - have;
        u32 next_nb = (total - next_pos) / 16;
        if (next_nb > 32) next_nb = 32;
        if (warp == 1) {
            if (next_nb) produce(slot ^ 1, 0, next_pos, next_nb);
        } else if (lane == 0) {
            const u32* k = kw + slot * 32 * SHA_KW_STRIDE;
            Sha8 h;
#pragma unroll
            for (int i = 0; i < 8; i++) h.v[i] = tr.h[i];
            for (u32 b = 0; b < nb; b++) h = sha256_rounds(h, k + b * SHA_KW_STRIDE);
#pragma unroll
            for (int i = 0; i < 8; i++) tr.h[i] = h.v[i];
        }
        __syncthreads();
        pos = next_pos; have = 0; nb = next_nb; slot ^= 1;
    }
    const u32 rest = total - pos;      // fewer than 16 - have words: they stay in the stream buffer
    if (warp == 0) for (u32 j = lane; j < rest; j += 32) bufw[have + j] = load(pos + j);
    if (threadIdx.x == 0) { tr.buflen = (have + rest) * 4; tr.total += (u64)total * 4; }
    __syncthreads();
}
template <class Load>
__device__ __forceinline__ void tr_absorb_stream_2w(Tr& tr, u32 total, Load load, u32* bufw, u32* tile, u32* kw, u32* bc) {
    if (threadIdx.x == 0) bc[0] = tr.buflen;
    __syncthreads();                   // also: thread 0's earlier writes to the stream buffer become visible
    const u32 buflen = bc[0];
    const u32 s = buflen & 3, have = buflen >> 2;
    if (s == 0) { tr_absorb_stream_2w_aligned(tr, total, load, bufw, have, tile, kw); return; }
    if (total == 0) { __syncthreads(); return; }
    // byte-misaligned stream (a label of odd length in front, for instance): the same pipeline over funnel-shifted words
    const u32 sh = 8 * s;
    const u32 pend = bufw[have] << (32 - sh);
    __syncthreads();                   // every thread holds the pending bytes before the buffer is written again
    tr_absorb_stream_2w_aligned(tr, total, [=](u32 g) -> u32 { return __funnelshift_l(g ? load(g - 1) : pend, load(g), sh); },
                                bufw, have, tile, kw);
    if (threadIdx.x == 0) {
        bufw[tr.buflen >> 2] = load(total - 1) >> (32 - sh);
        tr.buflen += s;
    }
    __syncthreads();
}

}  // namespace zkb
