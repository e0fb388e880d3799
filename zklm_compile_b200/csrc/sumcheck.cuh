// Sumcheck round kernels: fold the tables with the previous challenge and, in the same pass,
// accumulate the next round polynomial; the CTA that finishes last adds up the per-CTA
// partials, advances the device transcript and publishes the next challenge.
//
// Protocols covered (reference: rust/zk_ml_prover/src/proving/sumcheck.rs):
//   PRODUCT  sum f g      s0 = sum f0 g0, s1 = sum f1 g1, s2 = sum (2f1-f0)(2g1-g0)   (:211-272, :1204-1315)
//   TRIPLE   sum f g h    s0..s3 at t = 0,1,2,3                                      (:277-354, :1318-1384)
//   ONES     sum g        s0 = sum g0, s1 = sum g1, s2 = 2 s1 - s0                    (:857-902, :1389-1435)
// with base-field (Fp) or extension-field (Fe) challenges.  Tables are folded MSB-first: the
// pair of index j is (j, j + half).
//
// State between launches: tables of `size` elements plus a challenge that is still to be
// folded in ("pending").  A round launch with FOLD reads the size-4h tables, writes the
// size-2h folded tables (quarter j pairs with j + 2h -> lo, j + h with j + 3h -> hi; thread j
// is the only reader and writer of those six slots, so in-place folding is race-free) and
// reduces over the h pairs (lo, hi).  Round 0 has nothing to fold and only reduces.
#pragma once
#include "m31.cuh"
#include "transcript.cuh"
#include "exchange.cuh"

namespace zkb {

enum ScKind { SC_PRODUCT = 0, SC_TRIPLE = 1, SC_ONES = 2 };

template <int KIND> struct ScTraits;
template <> struct ScTraits<SC_PRODUCT> { static constexpr int NT = 2, NACC = 3, NABS = 3; };
template <> struct ScTraits<SC_TRIPLE>  { static constexpr int NT = 3, NACC = 4, NABS = 4; };
template <> struct ScTraits<SC_ONES>    { static constexpr int NT = 1, NACC = 2, NABS = 3; };

template <class T> struct Width;
template <> struct Width<Fp> { static constexpr int W = 1; };
template <> struct Width<Fe> { static constexpr int W = 4; };

template <bool C, class A, class B> struct Sel { typedef A type; };
template <class A, class B> struct Sel<false, A, B> { typedef B type; };

constexpr int SC_MAX_GRID = 2048;   // upper bound on CTAs of a round launch (sizes `partials`)
constexpr int SC_TAIL_THREADS = 1024;

struct ScTables {
    const void* src[3];
    void* dst[3];
};

// Per-sumcheck device bookkeeping.
struct ScIO {
    TrState* tr;            // device transcript, advanced in place
    u32* partials;          // [SC_MAX_GRID][16]
    unsigned int* counter;  // ticket for "last CTA done"; left at 0
    u32* polys;             // [num_vars][NABS][W]: every absorbed evaluation s_0.. of every round
    u32* chal;              // [num_vars][W]
    u32* fin;               // [NT][W]
    const u32* dyn_nv;      // tail only, optional: num_vars read from device memory (LogUp)
    u32* status;            // optional status word (see check_zero_sum)
    u32* post_out;          // optional destination of the post-squeezed challenges
    u32 post_squeezes;      // base-field squeezes performed right after the final evaluations
    u32 check_zero_sum;     // nonzero: flag status = 3 unless round 0 has s0 + s1 == 0 (LogUp identity)
    // Sumcheck split over several GPUs (see exchange.cuh): the tables given to the kernels are
    // this GPU's slice, `round` counts global rounds, the first xch_local_vars rounds are local
    // ones whose sums are exchanged, then the per-GPU remainders are gathered and the last
    // log2(world) rounds run identically on every GPU.  Null for an ordinary sumcheck.
    const ScXch* xch;
    u32 xch_local_vars;
};
__device__ __forceinline__ bool is_zero_el(Fp a) { return a.v == 0; }
__device__ __forceinline__ bool is_zero_el(Fe a) { return (a.x | a.y | a.z | a.w) == 0; }

// ---- small conversions ---------------------------------------------------------------------
__device__ __forceinline__ void to_words(Fp a, u32* w) { w[0] = a.v; }
__device__ __forceinline__ void to_words(Fe a, u32* w) { w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; }
__device__ __forceinline__ void from_words(Fp& a, const u32* w) { a.v = w[0]; }
__device__ __forceinline__ void from_words(Fe& a, const u32* w) { a = Fe{w[0], w[1], w[2], w[3]}; }
__device__ __forceinline__ void widen_to(Fp a, Fp& o) { o = a; }
__device__ __forceinline__ void widen_to(Fp a, Fe& o) { o = fe_from(a); }
__device__ __forceinline__ void widen_to(Fe a, Fe& o) { o = a; }
template <class T> __device__ __forceinline__ T zero_of();
template <> __device__ __forceinline__ Fp zero_of<Fp>() { return fp_zero(); }
template <> __device__ __forceinline__ Fe zero_of<Fe>() { return fe_zero(); }

template <class T> __device__ __forceinline__ T ld_el(const void* base, size_t i) {
    return ld_fe(reinterpret_cast<const T*>(base) + i);
}
template <class T> __device__ __forceinline__ void st_el(void* base, size_t i, T v) {
    st_fe(reinterpret_cast<T*>(base) + i, v);
}

// ---- per-pair accumulation -----------------------------------------------------------------
template <int KIND, class T>
__device__ __forceinline__ void sc_accumulate(T* acc, const T* lo, const T* hi) {
    if constexpr (KIND == SC_PRODUCT) {
        acc[0] = acc[0] + lo[0] * lo[1];
        acc[1] = acc[1] + hi[0] * hi[1];
        acc[2] = acc[2] + dbl_minus(hi[0], lo[0]) * dbl_minus(hi[1], lo[1]);
    } else if constexpr (KIND == SC_TRIPLE) {
        acc[0] = acc[0] + lo[0] * lo[1] * lo[2];
        acc[1] = acc[1] + hi[0] * hi[1] * hi[2];
        T f2 = dbl_minus(hi[0], lo[0]), g2 = dbl_minus(hi[1], lo[1]), h2 = dbl_minus(hi[2], lo[2]);
        acc[2] = acc[2] + f2 * g2 * h2;
        // value at t = 3: x2 + (x1 - x0) = 3 x1 - 2 x0 (sumcheck.rs:316-321, 1356-1359)
        T f3 = f2 + (hi[0] - lo[0]), g3 = g2 + (hi[1] - lo[1]), h3 = h2 + (hi[2] - lo[2]);
        acc[3] = acc[3] + f3 * g3 * h3;
    } else {
        acc[0] = acc[0] + lo[0];
        acc[1] = acc[1] + hi[0];
    }
}

// One (optionally folding) pass of the calling CTA(s) over pairs j in [j0, half) step `stride`.
template <int KIND, class SrcT, class ChalT, bool FOLD>
__device__ __forceinline__ void sc_pass(const ScTables& tb, size_t half, ChalT r, size_t j0, size_t stride,
                                        typename Sel<FOLD, ChalT, SrcT>::type* acc) {
    typedef typename Sel<FOLD, ChalT, SrcT>::type AccT;
    constexpr int NT = ScTraits<KIND>::NT;
    for (size_t j = j0; j < half; j += stride) {
        AccT lo[NT], hi[NT];
#pragma unroll
        for (int t = 0; t < NT; t++) {
            if constexpr (FOLD) {
                SrcT a = ld_el<SrcT>(tb.src[t], j), b = ld_el<SrcT>(tb.src[t], j + 2 * half);
                SrcT c = ld_el<SrcT>(tb.src[t], j + half), d = ld_el<SrcT>(tb.src[t], j + 3 * half);
                ChalT l = lerp(a, b, r), h = lerp(c, d, r);
                st_el<ChalT>(tb.dst[t], j, l);
                st_el<ChalT>(tb.dst[t], j + half, h);
                widen_to(l, lo[t]);
                widen_to(h, hi[t]);
            } else {
                SrcT a = ld_el<SrcT>(tb.src[t], j), b = ld_el<SrcT>(tb.src[t], j + half);
                widen_to(a, lo[t]);
                widen_to(b, hi[t]);
            }
        }
        sc_accumulate<KIND, AccT>(acc, lo, hi);
    }
}

// Sum `nw` canonical words per thread across the CTA; result valid in thread 0 (and in red[] row 0).
template <int NWORDS>
__device__ __forceinline__ void block_sum_words(u32* v, u32* red /* [32][NWORDS] shared */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int k = 0; k < NWORDS; k++) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v[k] = add31(v[k], __shfl_down_sync(0xffffffffu, v[k], off));
    }
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < NWORDS; k++) red[warp * NWORDS + k] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < NWORDS; k++) {
            u32 x = lane < nwarps ? red[lane * NWORDS + k] : 0u;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) x = add31(x, __shfl_down_sync(0xffffffffu, x, off));
            v[k] = x;
        }
    }
    __syncthreads();
}

// Thread 0: turn the summed accumulators into the round message, advance the transcript,
// emit the stored evaluations and the challenge.
template <int KIND, class AccT, class ChalT>
__device__ __forceinline__ ChalT sc_finish_round(const u32* words, const ScIO& io, u32 round, Tr& tr) {
    constexpr int NACC = ScTraits<KIND>::NACC, NABS = ScTraits<KIND>::NABS;
    constexpr int WA = Width<AccT>::W, WC = Width<ChalT>::W;
    ChalT s[4];
#pragma unroll
    for (int k = 0; k < NACC; k++) {
        AccT a;
        from_words(a, words + k * WA);
        widen_to(a, s[k]);
    }
    if constexpr (KIND == SC_ONES) s[2] = s[1] + s[1] - s[0];
    if (io.check_zero_sum && round == 0 && !is_zero_el(s[0] + s[1])) atomicExch(io.status, 3u);
    u32* out = io.polys + (size_t)round * NABS * WC;
    u32 msg[NABS * WC];
#pragma unroll
    for (int k = 0; k < NABS; k++) to_words(s[k], msg + k * WC);
    tr_absorb_words<NABS * WC>(tr, msg);
#pragma unroll
    for (int k = 0; k < NABS * WC; k++) out[k] = msg[k];
    ChalT r;
    tr_squeeze_el(tr, r);
    to_words(r, io.chal + (size_t)round * WC);
    return r;
}

// ---- multi-CTA round launch ----------------------------------------------------------------
template <int KIND, class SrcT, class ChalT, bool FOLD>
__global__ void __launch_bounds__(256) sc_round_kernel(ScTables tb, size_t half, u32 round, ScIO io) {
    typedef typename Sel<FOLD, ChalT, SrcT>::type AccT;
    constexpr int NACC = ScTraits<KIND>::NACC, WA = Width<AccT>::W, NW = NACC * WA;
    __shared__ u32 red[32 * 16];
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ bool is_last;

    ChalT r = zero_of<ChalT>();
    if constexpr (FOLD) from_words(r, io.chal + (size_t)(round - 1) * Width<ChalT>::W);

    AccT acc[NACC];
#pragma unroll
    for (int k = 0; k < NACC; k++) acc[k] = zero_of<AccT>();
    sc_pass<KIND, SrcT, ChalT, FOLD>(tb, half, r, (size_t)blockIdx.x * blockDim.x + threadIdx.x,
                                     (size_t)gridDim.x * blockDim.x, acc);
    u32 w[NW];
#pragma unroll
    for (int k = 0; k < NACC; k++) to_words(acc[k], w + k * WA);
    block_sum_words<NW>(w, red);

    if (threadIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < NW; k++) io.partials[(size_t)blockIdx.x * 16 + k] = w[k];
        __threadfence();
        unsigned int ticket = atomicAdd(io.counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();

    u32 t[NW];
#pragma unroll
    for (int k = 0; k < NW; k++) t[k] = 0;
    for (u32 b = threadIdx.x; b < gridDim.x; b += blockDim.x) {
#pragma unroll
        for (int k = 0; k < NW; k++) t[k] = add31(t[k], __ldcg(io.partials + (size_t)b * 16 + k));
    }
    block_sum_words<NW>(t, red);
    if (io.xch && threadIdx.x < 32) xch_allreduce_warp<NW>(*io.xch, io.xch->seq + round, t);
    if (threadIdx.x == 0) {
        Tr tr;
        tr_load(tr, io.tr, trbuf);
        sc_finish_round<KIND, AccT, ChalT>(t, io, round, tr);
        tr_store(tr, io.tr);
        *io.counter = 0;
    }
}

// ---- product sumcheck over base-field tables: the two bandwidth-critical launches --------------
// Round 0 (nothing to fold) and round 1 (fold the first EF challenge into base-field tables)
// of PRODUCT sumchecks whose inputs are M31 vectors.  Four consecutive pair indices per thread
// (16-byte loads), products accumulated unreduced in 64 bits.
//
// Round 1 never multiplies in EF per element.  With lo = a + r (b - a), hi = c + r (d - c) the
// three sums are quadratics in r with base-field coefficients,
//     sum lo_f lo_g = A0 + r A1 + r^2 A2,   A0 = sum a_f a_g, A1 = sum (a_f e_g + a_g e_f), A2 = sum e_f e_g
// (e = b - a), likewise for hi (c, d - c) and for 2 hi - lo; the nine coefficient sums are
// reduced like any other partial and the finishing CTA evaluates the quadratics once.
__device__ __forceinline__ u64 fold62(u64 t) { return (u64)((u32)t & ZKB_P) + (u32)(t >> 31); }   // t < 2^63 -> < 2^33, same residue
__device__ __forceinline__ void ld4(const void* base, size_t j, u32* o) {
    uint4 t = *reinterpret_cast<const uint4*>(reinterpret_cast<const u32*>(base) + j);
    o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
}

// WRITE = false (with FOLD): the folded tables are not materialised - the launch only produces
// the round message (the fused launch below folds two challenges at once from the base tables).
template <class ChalT, bool FOLD, bool WRITE = true>
__global__ void __launch_bounds__(256) sc_product_base_kernel(ScTables tb, size_t half, u32 round, ScIO io) {
    constexpr int NACC = FOLD ? 9 : 3;
    __shared__ u32 red[32 * 16];
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ bool is_last;
    Fe r = fe_zero();
    if constexpr (FOLD) from_words(r, io.chal + (size_t)(round - 1) * 4);

    u64 acc[NACC];
#pragma unroll
    for (int k = 0; k < NACC; k++) acc[k] = 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x * 4;
    for (size_t j = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; j < half; j += stride) {
        if constexpr (!FOLD) {
            u32 f0[4], f1[4], g0[4], g1[4];
            ld4(tb.src[0], j, f0); ld4(tb.src[0], j + half, f1);
            ld4(tb.src[1], j, g0); ld4(tb.src[1], j + half, g1);
#pragma unroll
            for (int v = 0; v < 4; v++) {
                u32 f2 = sub31(add31(f1[v], f1[v]), f0[v]), g2 = sub31(add31(g1[v], g1[v]), g0[v]);
                acc[0] += fold62((u64)f0[v] * g0[v]);
                acc[1] += fold62((u64)f1[v] * g1[v]);
                acc[2] += fold62((u64)f2 * g2);
            }
        } else {
            u32 fa[4], fb[4], fc[4], fd[4], ga[4], gb[4], gc[4], gd[4];
            ld4(tb.src[0], j, fa); ld4(tb.src[0], j + 2 * half, fb); ld4(tb.src[0], j + half, fc); ld4(tb.src[0], j + 3 * half, fd);
            ld4(tb.src[1], j, ga); ld4(tb.src[1], j + 2 * half, gb); ld4(tb.src[1], j + half, gc); ld4(tb.src[1], j + 3 * half, gd);
#pragma unroll
            for (int v = 0; v < 4; v++) {
                const u32 ef = sub31(fb[v], fa[v]), eg = sub31(gb[v], ga[v]);       // lo = a + r e
                const u32 hf = sub31(fd[v], fc[v]), hg = sub31(gd[v], gc[v]);       // hi = c + r h
                if constexpr (WRITE) {      // folded tables (EF = base + r * base)
                    Fe lf = r * Fp{ef}; lf.x = add31(lf.x, fa[v]);
                    Fe lg = r * Fp{eg}; lg.x = add31(lg.x, ga[v]);
                    Fe uf = r * Fp{hf}; uf.x = add31(uf.x, fc[v]);
                    Fe ug = r * Fp{hg}; ug.x = add31(ug.x, gc[v]);
                    st_el<Fe>(tb.dst[0], j + v, lf); st_el<Fe>(tb.dst[0], j + half + v, uf);
                    st_el<Fe>(tb.dst[1], j + v, lg); st_el<Fe>(tb.dst[1], j + half + v, ug);
                }
                // coefficient sums
                acc[0] += fold62((u64)fa[v] * ga[v]);
                acc[1] += fold62((u64)fa[v] * eg + (u64)ga[v] * ef);
                acc[2] += fold62((u64)ef * eg);
                acc[3] += fold62((u64)fc[v] * gc[v]);
                acc[4] += fold62((u64)fc[v] * hg + (u64)gc[v] * hf);
                acc[5] += fold62((u64)hf * hg);
                const u32 pf = sub31(add31(fc[v], fc[v]), fa[v]), pg = sub31(add31(gc[v], gc[v]), ga[v]);   // 2 hi - lo at r = 0
                const u32 qf = sub31(add31(hf, hf), ef), qg = sub31(add31(hg, hg), eg);                     // its slope in r
                acc[6] += fold62((u64)pf * pg);
                acc[7] += fold62((u64)pf * qg + (u64)pg * qf);
                acc[8] += fold62((u64)qf * qg);
            }
        }
    }
    u32 w[NACC];
#pragma unroll
    for (int k = 0; k < NACC; k++) w[k] = red64(acc[k]);
    block_sum_words<NACC>(w, red);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < NACC; k++) io.partials[(size_t)blockIdx.x * 16 + k] = w[k];
        __threadfence();
        unsigned int ticket = atomicAdd(io.counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    u32 t[NACC];
#pragma unroll
    for (int k = 0; k < NACC; k++) t[k] = 0;
    for (u32 b = threadIdx.x; b < gridDim.x; b += blockDim.x) {
#pragma unroll
        for (int k = 0; k < NACC; k++) t[k] = add31(t[k], __ldcg(io.partials + (size_t)b * 16 + k));
    }
    block_sum_words<NACC>(t, red);
    if (io.xch && threadIdx.x < 32) xch_allreduce_warp<NACC>(*io.xch, io.xch->seq + round, t);
    if (threadIdx.x == 0) {
        Tr tr;
        tr_load(tr, io.tr, trbuf);
        if constexpr (FOLD) {
            const Fe r2 = r * r;
            u32 ew[12];
#pragma unroll
            for (int k = 0; k < 3; k++) {
                Fe s = r * Fp{t[3 * k + 1]} + r2 * Fp{t[3 * k + 2]};
                s.x = add31(s.x, t[3 * k]);
                to_words(s, ew + 4 * k);
            }
            sc_finish_round<SC_PRODUCT, Fe, Fe>(ew, io, round, tr);
        } else {
            sc_finish_round<SC_PRODUCT, Fp, ChalT>(t, io, round, tr);
        }
        tr_store(tr, io.tr);
        *io.counter = 0;
    }
}

// ---- product sumcheck over base-field tables: two challenges folded in one pass -----------------
// Rounds 0 and 1 only need the base tables (round 1's message comes from the coefficient sums
// above), so the first extension-field tables that are ever written are the ones folded with BOTH
// r_0 and r_1: a quarter of the input length instead of a half.  For the table index
// i = j + q0 E + q1 2E + q2 4E (E = an eighth of the table, j < E) the two folds give
//     T2[j + q0 E] = t00 + r0 (t01 - t00) + r1 (t10 - t00) + r0 r1 (t11 - t10 - t01 + t00),  t_{q1 q2} = T[i],
// three EF x base products whose coordinates are summed in 64 bits and folded once.  In the same
// pass the message of round 2 is accumulated over the pairs (T2[j], T2[j + E]).  Against folding
// round by round this launch and the one before it move 24 N bytes instead of 48 N (N = table length).
__device__ __forceinline__ Fe fold2_el(u32 t00, u32 t01, u32 t10, u32 t11, Fe r0, Fe r1, Fe r01) {
    const u32 b = sub31(t01, t00), c = sub31(t10, t00), d = sub31(sub31(t11, t10), b);
    Fe o;
    o.x = red64((u64)r0.x * b + (u64)r1.x * c + (u64)r01.x * d + t00);
    o.y = red64((u64)r0.y * b + (u64)r1.y * c + (u64)r01.y * d);
    o.z = red64((u64)r0.z * b + (u64)r1.z * c + (u64)r01.z * d);
    o.w = red64((u64)r0.w * b + (u64)r1.w * c + (u64)r01.w * d);
    return o;
}
template <int VEC> struct LdVec;
template <> struct LdVec<1> { static __device__ __forceinline__ void ld(const u32* p, u32* o) { o[0] = *p; } };
template <> struct LdVec<2> { static __device__ __forceinline__ void ld(const u32* p, u32* o) { uint2 t = *reinterpret_cast<const uint2*>(p); o[0] = t.x; o[1] = t.y; } };
template <> struct LdVec<4> { static __device__ __forceinline__ void ld(const u32* p, u32* o) { uint4 t = *reinterpret_cast<const uint4*>(p); o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w; } };

// tables: 8 E base-field words each; dst: 2 E extension-field elements each; `round` is the round
// whose message is produced (2); challenges of rounds round-2 and round-1 are read from io.chal.
template <int VEC>
__global__ void __launch_bounds__(256) sc_product_base_fold2_kernel(ScTables tb, size_t E, u32 round, ScIO io) {
    __shared__ u32 red[32 * 16];
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ bool is_last;
    Fe r0, r1;
    from_words(r0, io.chal + (size_t)(round - 2) * 4);
    from_words(r1, io.chal + (size_t)(round - 1) * 4);
    const Fe r01 = r0 * r1;
    Fe acc[3] = {fe_zero(), fe_zero(), fe_zero()};
    const size_t stride = (size_t)gridDim.x * blockDim.x * VEC;
    for (size_t j = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; j < E; j += stride) {
        Fe lo[2][VEC], hi[2][VEC];
#pragma unroll
        for (int t = 0; t < 2; t++) {
            const u32* src = reinterpret_cast<const u32*>(tb.src[t]) + j;
            u32 q[8][VEC];
#pragma unroll
            for (int k = 0; k < 8; k++) LdVec<VEC>::ld(src + (size_t)k * E, q[k]);
#pragma unroll
            for (int v = 0; v < VEC; v++) {
                // q index = q0 + 2 q1 + 4 q2: t_{q1 q2} of the lower element is q[2 q1 + 4 q2], of the upper one q[1 + 2 q1 + 4 q2]
                lo[t][v] = fold2_el(q[0][v], q[4][v], q[2][v], q[6][v], r0, r1, r01);
                hi[t][v] = fold2_el(q[1][v], q[5][v], q[3][v], q[7][v], r0, r1, r01);
                st_el<Fe>(tb.dst[t], j + v, lo[t][v]);
                st_el<Fe>(tb.dst[t], j + E + v, hi[t][v]);
            }
        }
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            acc[0] = acc[0] + lo[0][v] * lo[1][v];
            acc[1] = acc[1] + hi[0][v] * hi[1][v];
            acc[2] = acc[2] + dbl_minus(hi[0][v], lo[0][v]) * dbl_minus(hi[1][v], lo[1][v]);
        }
    }
    u32 w[12];
#pragma unroll
    for (int k = 0; k < 3; k++) to_words(acc[k], w + 4 * k);
    block_sum_words<12>(w, red);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < 12; k++) io.partials[(size_t)blockIdx.x * 16 + k] = w[k];
        __threadfence();
        unsigned int ticket = atomicAdd(io.counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    u32 t[12];
#pragma unroll
    for (int k = 0; k < 12; k++) t[k] = 0;
    for (u32 b = threadIdx.x; b < gridDim.x; b += blockDim.x) {
#pragma unroll
        for (int k = 0; k < 12; k++) t[k] = add31(t[k], __ldcg(io.partials + (size_t)b * 16 + k));
    }
    block_sum_words<12>(t, red);
    if (io.xch && threadIdx.x < 32) xch_allreduce_warp<12>(*io.xch, io.xch->seq + round, t);
    if (threadIdx.x == 0) {
        Tr tr;
        tr_load(tr, io.tr, trbuf);
        sc_finish_round<SC_PRODUCT, Fe, Fe>(t, io, round, tr);
        tr_store(tr, io.tr);
        *io.counter = 0;
    }
}

// ---- single-CTA tail: all remaining rounds and the final evaluations -------------------------
// Entry state: tables in tb.src (type SrcT) of `size` elements; if `pending`, the challenge
// of round `round - 1` still has to be folded in.  Runs rounds round .. num_vars-1, then folds
// the last challenge into the two remaining elements of each table and writes the finals.
template <int KIND, class SrcT, class ChalT>
__global__ void __launch_bounds__(SC_TAIL_THREADS) sc_tail_kernel(ScTables tb, size_t size, u32 round, u32 num_vars,
                                                                  int pending, ScIO io) {
    constexpr int NT = ScTraits<KIND>::NT, NACC = ScTraits<KIND>::NACC;
    constexpr int WC = Width<ChalT>::W, WS = Width<SrcT>::W;
    __shared__ u32 red[32 * 16];
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ u32 r_sh[4];

    ZKB_STAMP_BEGIN
    if (io.dyn_nv) { num_vars = io.dyn_nv[0]; size = size_t(1) << num_vars; }
    Tr tr;
    if (threadIdx.x == 0) tr_load(tr, io.tr, trbuf);
    ChalT r = zero_of<ChalT>();
    if (pending) from_words(r, io.chal + (size_t)(round - 1) * WC);
    bool in_src = true;           // tables still in their input buffers / input type
    ScTables cur = tb;

    // Split sumcheck: phase 0 runs the local rounds (sums exchanged), then the per-GPU remainders
    // are gathered into `world`-element tables in shared memory and phase 1 runs the last rounds.
    __shared__ __align__(16) u32 gathered[3][XCH_MAX_WORLD * 4];
    const bool split = io.xch != nullptr && io.xch->world > 1;
    u32 stop = split ? io.xch_local_vars : num_vars;
    for (int phase = 0; phase < 2; phase++) {
    for (; round < stop; round++) {
        u32 w[16];
        if (in_src) {
            if (!pending) {
                SrcT acc[NACC];
#pragma unroll
                for (int k = 0; k < NACC; k++) acc[k] = zero_of<SrcT>();
                sc_pass<KIND, SrcT, ChalT, false>(cur, size / 2, r, threadIdx.x, blockDim.x, acc);
#pragma unroll
                for (int k = 0; k < NACC; k++) {
                    ChalT e; widen_to(acc[k], e); to_words(e, w + k * WC);
                }
            } else {
                ChalT acc[NACC];
#pragma unroll
                for (int k = 0; k < NACC; k++) acc[k] = zero_of<ChalT>();
                sc_pass<KIND, SrcT, ChalT, true>(cur, size / 4, r, threadIdx.x, blockDim.x, acc);
#pragma unroll
                for (int k = 0; k < NACC; k++) to_words(acc[k], w + k * WC);
                size /= 2;
                in_src = false;
#pragma unroll
                for (int t = 0; t < NT; t++) cur.src[t] = cur.dst[t];
            }
        } else {
            ChalT acc[NACC];
#pragma unroll
            for (int k = 0; k < NACC; k++) acc[k] = zero_of<ChalT>();
            if (pending) {
                sc_pass<KIND, ChalT, ChalT, true>(cur, size / 4, r, threadIdx.x, blockDim.x, acc);
                size /= 2;
            } else {
                sc_pass<KIND, ChalT, ChalT, false>(cur, size / 2, r, threadIdx.x, blockDim.x, acc);
            }
#pragma unroll
            for (int k = 0; k < NACC; k++) to_words(acc[k], w + k * WC);
        }
        block_sum_words<NACC * WC>(w, red);
        if (io.xch && phase == 0 && threadIdx.x < 32) xch_allreduce_warp<NACC * WC>(*io.xch, io.xch->seq + round, w);
        if (threadIdx.x == 0) {
            ChalT rn = sc_finish_round<KIND, ChalT, ChalT>(w, io, round, tr);
            to_words(rn, r_sh);
        }
        __syncthreads();
        from_words(r, r_sh);
        pending = 1;
        __syncthreads();
    }
    if (!split || phase == 1) break;
    // size == 2: fold the last local challenge in, gather everybody's remainder (ordered by rank =
    // the low index bits), and continue on the gathered tables with nothing pending.
    if (threadIdx.x < 32) {
        u32 mine[NT * WC];
#pragma unroll
        for (int k = 0; k < NT * WC; k++) mine[k] = 0;
        if (threadIdx.x == 0) {
#pragma unroll
            for (int t = 0; t < NT; t++) {
                ChalT v;
                if (in_src) v = lerp(ld_el<SrcT>(cur.src[t], 0), ld_el<SrcT>(cur.src[t], 1), r);
                else {
                    ChalT a = ld_el<ChalT>(cur.src[t], 0), b = ld_el<ChalT>(cur.src[t], 1);
                    v = a + r * (b - a);
                }
                to_words(v, mine + t * WC);
            }
        }
        u32 got[NT * WC];
        const bool ok = xch_exchange_warp<NT * WC>(*io.xch, io.xch->seq + io.xch_local_vars, mine, got);
        const u32 sdr = threadIdx.x;                  // lane s holds rank s's remainder
        if (sdr < io.xch->world) {
#pragma unroll
            for (int t = 0; t < NT; t++)
#pragma unroll
                for (int k = 0; k < WC; k++) gathered[t][sdr * WC + k] = ok ? got[t * WC + k] : 0u;
        }
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < NT; t++) { cur.src[t] = gathered[t]; cur.dst[t] = gathered[t]; }
    in_src = false;
    pending = 0;
    size = io.xch->world;
    stop = num_vars;
    }

    if (threadIdx.x == 0) {
        for (u32 q = 0; q < io.post_squeezes; q++) {
            u32 v = tr_squeeze(tr);
            if (io.post_out) io.post_out[q] = v;
        }
        tr_store(tr, io.tr);
        // size == 2 here: fold the last challenge in.
#pragma unroll
        for (int t = 0; t < NT; t++) {
            ChalT v;
            if (in_src) v = lerp(ld_el<SrcT>(cur.src[t], 0), ld_el<SrcT>(cur.src[t], 1), r);
            else {
                ChalT a = ld_el<ChalT>(cur.src[t], 0), b = ld_el<ChalT>(cur.src[t], 1);
                v = a + r * (b - a);
            }
            to_words(v, io.fin + t * WC);
        }
    }
    (void)WS;
    ZKB_STAMP_END(io.tr, 2);
}

}  // namespace zkb
