// Single-CTA tail of the product sumcheck over EF tables with the table work taken off the
// critical path (rust/zk_ml_prover/src/proving/sumcheck.rs:1262-1315 computes the same messages).
//
// In the plain tail every round is: pass over the tables (fold with the last challenge, sum the
// round polynomial), block reduction, then one thread hashes (about five SHA-256 compressions)
// while a thousand threads wait.  Here warp 0 only hashes.  While it hashes round k, the other warps
// fold the tables with r_(k-1) and compute the NEXT round's sums as polynomials in the still
// unknown r_k: with lo(r) = a + r (b - a), hi(r) = c + r (d - c) over the four quarters a, b, c,
// d of a table, each of s0 = sum lo_f lo_g, s1 = sum hi_f hi_g, s2 = sum (2hi - lo)_f (2hi - lo)_g
// is a quadratic in r with nine EF coefficient sums in all.  When r_k arrives the hashing thread
// evaluates the three quadratics and goes on hashing; the table work overlaps the hash chain
// instead of alternating with it.  All values are canonical field elements, so the messages are
// bit-identical to the plain tail's.
#pragma once
#include "sumcheck.cuh"

namespace zkb {

constexpr int PIPE_THREADS = 512;                                 // at most; 128 registers per thread (the worker pass keeps 36 sums)
constexpr int PIPE_MAX_WORKER_WARPS = PIPE_THREADS / 32 - 1;      // 15
constexpr int PIPE_NW = 36;                                       // nine EF coefficient sums

// Roles.  Warp 0 hashes.  Warps 4, 8, 12 would share warp 0's scheduler (warp w issues on sub-
// partition w mod 4), its instruction cache and its issue slots; they only join the CTA barriers,
// so the hash chain has a sub-partition to itself.  The other warps are the workers, numbered
// 0, 1, 2, ... in warp order.
__device__ __forceinline__ bool pipe_is_worker(int warp) { return (warp & 3) != 0; }
__device__ __forceinline__ int pipe_worker_index(int warp) { return warp - 1 - (warp >> 2); }
__device__ __forceinline__ int pipe_worker_warps() { const int last = (int)(blockDim.x >> 5) - 1; return last - (last >> 2); }
// Barrier 1 among the worker warps only; blockDim.x is a multiple of 32.
__device__ __forceinline__ void pipe_worker_barrier() { asm volatile("bar.sync 1, %0;" ::"r"(pipe_worker_warps() * 32) : "memory"); }

// Coefficient sums of the next round over one pair index: quarters (a, b, c, d) of f and g.
__device__ __forceinline__ void pipe_accum(Fe* C, Fe fa, Fe fb, Fe fc, Fe fd, Fe ga, Fe gb, Fe gc, Fe gd) {
    const Fe ef = fb - fa, eg = gb - ga, hf = fd - fc, hg = gd - gc;       // lo = a + r e, hi = c + r h
    C[0] = C[0] + fa * ga;  C[1] = C[1] + fa * eg + ga * ef;  C[2] = C[2] + ef * eg;
    C[3] = C[3] + fc * gc;  C[4] = C[4] + fc * hg + gc * hf;  C[5] = C[5] + hf * hg;
    const Fe pf = dbl_minus(fc, fa), pg = dbl_minus(gc, ga);               // 2 hi - lo at r = 0
    const Fe qf = dbl_minus(hf, ef), qg = dbl_minus(hg, eg);               // its slope in r
    C[6] = C[6] + pf * pg;  C[7] = C[7] + pf * qg + pg * qf;  C[8] = C[8] + qf * qg;
}

// Workers only (see pipe_is_worker; at least two worker warps, so that 36 threads can add the rows).  Tables of size n at (rf, rg); if `fold`, they are first
// folded with r into size n / 2 at (wf, wg) (in place allowed) and the sums are taken over the
// folded tables.  Leaves the 36 summed words in out[] (shared memory) when the result size is >= 4.
__device__ __forceinline__ void pipe_worker_pass(const Fe* rf, const Fe* rg, Fe* wf, Fe* wg, size_t n, bool fold, Fe r,
                                                 u32 (*cw)[PIPE_NW], u32* out) {
    const int worker_warps = pipe_worker_warps();
    const int wid = pipe_worker_index(threadIdx.x >> 5) * 32 + (threadIdx.x & 31);
    const size_t workers = (size_t)worker_warps * 32;
    const size_t m = fold ? n / 2 : n;              // size of the tables the sums run over
    Fe C[9];
#pragma unroll
    for (int i = 0; i < 9; i++) C[i] = fe_zero();
    if (m >= 4) {
        const size_t q = m / 4;                     // pair indices of the next round
        for (size_t j = wid; j < q; j += workers) {
            Fe fa, fb, fc, fd, ga, gb, gc, gd;
            if (fold) {
                // folded element x is lerp(T[x], T[x + n/2], r); this thread owns x = j, j+q, j+2q, j+3q
                const size_t h = n / 2;
                fa = lerp(ld_fe(rf + j), ld_fe(rf + j + h), r);                 ga = lerp(ld_fe(rg + j), ld_fe(rg + j + h), r);
                fc = lerp(ld_fe(rf + j + q), ld_fe(rf + j + q + h), r);         gc = lerp(ld_fe(rg + j + q), ld_fe(rg + j + q + h), r);
                fb = lerp(ld_fe(rf + j + 2 * q), ld_fe(rf + j + 2 * q + h), r); gb = lerp(ld_fe(rg + j + 2 * q), ld_fe(rg + j + 2 * q + h), r);
                fd = lerp(ld_fe(rf + j + 3 * q), ld_fe(rf + j + 3 * q + h), r); gd = lerp(ld_fe(rg + j + 3 * q), ld_fe(rg + j + 3 * q + h), r);
                st_fe(wf + j, fa); st_fe(wf + j + q, fc); st_fe(wf + j + 2 * q, fb); st_fe(wf + j + 3 * q, fd);
                st_fe(wg + j, ga); st_fe(wg + j + q, gc); st_fe(wg + j + 2 * q, gb); st_fe(wg + j + 3 * q, gd);
            } else {
                fa = ld_fe(rf + j); fc = ld_fe(rf + j + q); fb = ld_fe(rf + j + 2 * q); fd = ld_fe(rf + j + 3 * q);
                ga = ld_fe(rg + j); gc = ld_fe(rg + j + q); gb = ld_fe(rg + j + 2 * q); gd = ld_fe(rg + j + 3 * q);
            }
            pipe_accum(C, fa, fb, fc, fd, ga, gb, gc, gd);
        }
    } else if (fold) {
        // two elements remain after this fold: nothing to sum, just fold (one thread)
        if (wid == 0) {
            const size_t h = n / 2;
            for (size_t x = 0; x < h; x++) {
                Fe a = lerp(ld_fe(rf + x), ld_fe(rf + x + h), r), b = lerp(ld_fe(rg + x), ld_fe(rg + x + h), r);
                st_fe(wf + x, a); st_fe(wg + x, b);
            }
        }
    }
    if (m >= 4) {
        u32 w[PIPE_NW];
#pragma unroll
        for (int i = 0; i < 9; i++) to_words(C[i], w + 4 * i);
        const int lane = threadIdx.x & 31, warp = pipe_worker_index(threadIdx.x >> 5);
#pragma unroll
        for (int k = 0; k < PIPE_NW; k++) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) w[k] = add31(w[k], __shfl_down_sync(0xffffffffu, w[k], off));
        }
        if (lane == 0) {
#pragma unroll
            for (int k = 0; k < PIPE_NW; k++) cw[warp][k] = w[k];
        }
        pipe_worker_barrier();
        if (wid < PIPE_NW) {
            u32 v = 0;
            for (int rw = 0; rw < worker_warps; rw++) v = add31(v, cw[rw][wid]);
            out[wid] = v;
        }
    }
}

__global__ void __launch_bounds__(PIPE_THREADS) sc_tail_product_pipe_kernel(ScTables tb, size_t size, u32 round, u32 num_vars,
                                                                               int pending, ScIO io) {
    __shared__ u32 red[32 * 16];
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ u32 r_sh[2][4];                       // indexed by round parity: round k+1's challenge never overwrites r_k while a slow warp still reads it
    __shared__ u32 cw[PIPE_MAX_WORKER_WARPS][PIPE_NW];
    __shared__ u32 csum[2][PIPE_NW];
    __shared__ u32 w_sh[12];

    ZKB_STAMP_BEGIN
    Tr tr;
    if (threadIdx.x == 0) tr_load(tr, io.tr, trbuf);
    Fe r = fe_zero();
    if (pending) from_words(r, io.chal + (size_t)(round - 1) * 4);

    // ---- prologue: the message of `round`, computed directly by the whole CTA
    const Fe* rf = reinterpret_cast<const Fe*>(tb.src[0]);
    const Fe* rg = reinterpret_cast<const Fe*>(tb.src[1]);
    Fe* wf = reinterpret_cast<Fe*>(tb.dst[0]);
    Fe* wg = reinterpret_cast<Fe*>(tb.dst[1]);
    size_t n = size;                                 // size of the tables the current round sums over
    u32 w[16];
    {
        Fe acc[3] = {fe_zero(), fe_zero(), fe_zero()};
        if (pending) {
            sc_pass<SC_PRODUCT, Fe, Fe, true>(tb, n / 4, r, threadIdx.x, blockDim.x, acc);
            n /= 2;
            rf = wf; rg = wg;                        // folded tables live in dst from now on
        } else {
            sc_pass<SC_PRODUCT, Fe, Fe, false>(tb, n / 2, r, threadIdx.x, blockDim.x, acc);
        }
#pragma unroll
        for (int k = 0; k < 3; k++) to_words(acc[k], w + 4 * k);
        block_sum_words<12>(w, red);                 // ends with a CTA barrier: folded tables visible
    }

    bool first = true;
    u32 k = round;
    for (;;) {
        // thread 0 hashes round k; the workers prepare round k + 1 as polynomials in r_k
        if (threadIdx.x == 0) {
            Fe rn = sc_finish_round<SC_PRODUCT, Fe, Fe>(w, io, k, tr);
            to_words(rn, r_sh[k & 1]);
        } else if (pipe_is_worker(threadIdx.x >> 5)) {
            if (first) pipe_worker_pass(rf, rg, wf, wg, n, false, r, cw, csum[k & 1]);
            else       pipe_worker_pass(rf, rg, wf, wg, 2 * n, true, r, cw, csum[k & 1]);
        }
        __syncthreads();
        if (!first) { rf = wf; rg = wg; }            // the fold above wrote dst
        first = false;
        from_words(r, r_sh[k & 1]);                  // r_k
        if (n == 2) break;                           // round k was the last one
        if (threadIdx.x < 32) {                      // three lanes evaluate the three quadratics, lane 0 collects
            if (threadIdx.x < 3) {
                const u32* c = csum[k & 1] + 12 * threadIdx.x;
                Fe c0, c1, c2;
                from_words(c0, c); from_words(c1, c + 4); from_words(c2, c + 8);
                to_words(c0 + r * (c1 + r * c2), w_sh + 4 * threadIdx.x);
            }
            __syncwarp();
            if (threadIdx.x == 0) {
#pragma unroll
                for (int i = 0; i < 12; i++) w[i] = w_sh[i];
            }
        }
        k++;
        n /= 2;
    }
    (void)num_vars;

    if (threadIdx.x == 0) {
        for (u32 q = 0; q < io.post_squeezes; q++) {
            u32 v = tr_squeeze(tr);
            if (io.post_out) io.post_out[q] = v;
        }
        tr_store(tr, io.tr);
        // two elements per table remain (folded through r_(k-1)): fold the last challenge in
        Fe fv = lerp(ld_fe(rf), ld_fe(rf + 1), r), gv = lerp(ld_fe(rg), ld_fe(rg + 1), r);
        to_words(fv, io.fin);
        to_words(gv, io.fin + 4);
    }
    ZKB_STAMP_END(io.tr, 1);
}

}  // namespace zkb
