// eq-table construction, the weight-matrix fold (the one pass over the full weights inside a
// matmul proof) and the forward matvec.
//
//   eq_evals / eq_evals_ef   rust/zk_ml_prover/src/field/m31_ops.rs:30-50, 175-191
//   fold_eq_matvec(_ef)      rust/zk_ml_prover/src/proving/matmul.rs:76-128, 743-835
//   matmul_forward           rust/zk_ml_prover/src/transformer/mod.rs:140-163
//
// Both matrix kernels stream W (row-major u32) exactly once with 16-byte loads; products are
// accumulated unreduced in 64 bits (three < 2^62 products fit) and folded every third row.
#pragma once
#include "m31.cuh"

namespace zkb {

// out[idx] = prod_i (bit_i(idx) ? r_i : 1 - r_i), r_0 = most significant bit.  Written
// top-down per element (no in-place butterfly, so no read/write race between threads).
template <class T>
__device__ __forceinline__ T eq_at_index(const T* r, u32 k, size_t idx);
template <>
__device__ __forceinline__ Fp eq_at_index<Fp>(const Fp* r, u32 k, size_t idx) {
    Fp acc = fp_one();
    for (u32 i = 0; i < k; i++) {
        Fp ri = r[i];
        acc = acc * (((idx >> (k - 1 - i)) & 1) ? ri : (fp_one() - ri));
    }
    return acc;
}
template <>
__device__ __forceinline__ Fe eq_at_index<Fe>(const Fe* r, u32 k, size_t idx) {
    Fe acc = fe_one();
    for (u32 i = 0; i < k; i++) {
        Fe ri = ld_fe(r + i);
        acc = acc * (((idx >> (k - 1 - i)) & 1) ? ri : (fe_one() - ri));
    }
    return acc;
}
template <class T>
__global__ void eq_evals_kernel(const T* __restrict__ r, u32 k, T* out) {
    size_t n = size_t(1) << k;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        st_fe(out + i, eq_at_index<T>(r, k, i));
}

// ---- fold_eq_matvec: acc[j] += eq[i] * W[i][j] -----------------------------------------------
// grid.x tiles columns (128 * 4 per CTA), grid.y tiles rows.  A CTA is 2 row groups x 128 column
// threads: group g takes rows g, g+2, ... of the CTA's row range, eight rows per step, so eight
// 16-byte loads per thread are in flight.  Four products of canonical values fit one 64-bit
// sum (4 (p-1)^2 < 2^64); each such sum is folded once (2^31 == 1) and added to a 64-bit
// accumulator that is only reduced at the end.  The two groups' column sums meet in shared
// memory and one group adds them to the global 64-bit accumulators with atomicAdd; integer
// addition is associative, so the result does not depend on the order.  NC = 1 (base eq) or 4
// (EF eq).
constexpr int FOLD_GROUPS = 2;
constexpr int FOLD_UNROLL = 8;
constexpr int FOLD_ROWS_TILE = FOLD_GROUPS * FOLD_UNROLL;   // granularity of the per-CTA row range

__device__ __forceinline__ u64 part_reduce(u64 a) { return (a & ZKB_P) + (a >> 31); }   // keeps a < 2^34

// ATOMIC: column sums are added to 64-bit accumulators acc[n][NC] (zeroed by the caller).
// Otherwise every row tile writes its own canonical sums to part[row tile][n * NC] (u32) and
// fold_finalize_partials_kernel adds the slabs: no atomics (they serialise per address when a
// hundred row-CTAs meet on one column) and nothing to clear.
template <int NC, bool ATOMIC>
__global__ void __launch_bounds__(128 * FOLD_GROUPS, 2) fold_eq_matvec_kernel(const u32* __restrict__ W, size_t m, size_t n,
                                                                             const u32* __restrict__ eq /* [m_pad][NC] */,
                                                                             size_t rows_per_cta, unsigned long long* acc, u32* part) {
    __shared__ u32 sums[FOLD_GROUPS - 1][128][4 * NC];
    const int tx = threadIdx.x & 127, g = threadIdx.x >> 7;
    const bool vec_n = (n % 4 == 0);
    // gridDim.x CTAs walk the (column tile, row tile) pairs; with as many CTAs as tiles this is one tile each
    const size_t col_tiles = (n + 511) / 512, row_tiles = (m + rows_per_cta - 1) / rows_per_cta;
    for (size_t tile = blockIdx.x; tile < col_tiles * row_tiles; tile += gridDim.x) {
    const size_t tile_x = tile % col_tiles, tile_y = tile / col_tiles;
    const size_t j0 = (tile_x * 128 + tx) * 4;
    const size_t r0 = tile_y * rows_per_cta;
    const size_t r1 = r0 + rows_per_cta < m ? r0 + rows_per_cta : m;
    const bool vec = vec_n && (j0 + 4 <= n);
    u64 a[4][NC];                       // grows by less than 2^35 per step: no overflow for any m < 2^28
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
        for (int k = 0; k < NC; k++) a[c][k] = 0;

    if (j0 < n) {
        size_t row = r0 + g;
        for (; row + (FOLD_UNROLL - 1) * FOLD_GROUPS < r1; row += FOLD_UNROLL * FOLD_GROUPS) {
            u32 w[FOLD_UNROLL][4];
#pragma unroll
            for (int q = 0; q < FOLD_UNROLL; q++) {
                const u32* rp = W + (row + (size_t)q * FOLD_GROUPS) * n;
                if (vec) {
                    uint4 t = __ldcs(reinterpret_cast<const uint4*>(rp + j0));     // read once: evict first, keep L2 for the small tables of the other layers' tails
                    w[q][0] = t.x; w[q][1] = t.y; w[q][2] = t.z; w[q][3] = t.w;
                } else {
#pragma unroll
                    for (int c = 0; c < 4; c++) w[q][c] = (j0 + c < n) ? rp[j0 + c] : 0u;
                }
            }
#pragma unroll
            for (int k = 0; k < NC; k++) {
                u32 e[FOLD_UNROLL];
#pragma unroll
                for (int q = 0; q < FOLD_UNROLL; q++) e[q] = __ldg(eq + (row + (size_t)q * FOLD_GROUPS) * NC + k);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    u64 t0 = (u64)e[0] * w[0][c] + (u64)e[1] * w[1][c] + (u64)e[2] * w[2][c] + (u64)e[3] * w[3][c];
                    u64 t1 = (u64)e[4] * w[4][c] + (u64)e[5] * w[5][c] + (u64)e[6] * w[6][c] + (u64)e[7] * w[7][c];
                    a[c][k] += part_reduce(t0) + part_reduce(t1);
                }
            }
        }
        for (; row < r1; row += FOLD_GROUPS) {
            const u32* rp = W + row * n;
            u32 w[4];
#pragma unroll
            for (int c = 0; c < 4; c++) w[c] = (j0 + c < n) ? rp[j0 + c] : 0u;
#pragma unroll
            for (int k = 0; k < NC; k++) {
                const u32 e = __ldg(eq + row * NC + k);
#pragma unroll
                for (int c = 0; c < 4; c++) a[c][k] += part_reduce((u64)e * w[c]);
            }
        }
    }
    if (g > 0) {
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int k = 0; k < NC; k++) sums[g - 1][tx][c * NC + k] = red64(a[c][k]);
    }
    __syncthreads();
    if (g == 0 && j0 < n) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            if (j0 + c < n) {
#pragma unroll
                for (int k = 0; k < NC; k++) {
                    u64 v = red64(a[c][k]);
#pragma unroll
                    for (int q = 0; q < FOLD_GROUPS - 1; q++) v += sums[q][tx][c * NC + k];
                    if (ATOMIC) atomicAdd(acc + (j0 + c) * NC + k, (unsigned long long)v);
                    else part[tile_y * n * NC + (j0 + c) * NC + k] = red64(v);
                }
            }
        }
    }
    __syncthreads();                    // sums[] is reused by the next tile
    }
}
// Tiling: 512 columns per tile; rows split so that about four tiles per SM exist.  Returns
// (column tiles, row tiles); the launch uses column tiles * row tiles CTAs, or fewer CTAs that
// walk the tiles (fold_grid).
inline dim3 fold_launch_dims(int sm_count, size_t m, size_t n, size_t* rows_per_out) {
    const unsigned col_ctas = (unsigned)((n + 511) / 512);
    unsigned want_rows = (unsigned)((sm_count * 4 + col_ctas - 1) / col_ctas);
    if (want_rows > m / 32 + 1) want_rows = (unsigned)(m / 32 + 1);      // at least two steps per CTA
    if (want_rows < 1) want_rows = 1;
    size_t rows_per = (m + want_rows - 1) / want_rows;
    rows_per = (rows_per + FOLD_ROWS_TILE - 1) / FOLD_ROWS_TILE * FOLD_ROWS_TILE;
    *rows_per_out = rows_per;
    return dim3(col_ctas, (unsigned)((m + rows_per - 1) / rows_per));
}
constexpr int FOLD_THREADS = 128 * FOLD_GROUPS;
// CTAs of the launch: all tiles at once, or one CTA per SM when the GPU is shared with other contexts
// (the kernel needs 128 registers x 256 threads = half of an SM's register file).
inline unsigned fold_grid(dim3 tiles, int sm_count, bool polite) {
    unsigned t = tiles.x * tiles.y;
    return polite && t > (unsigned)sm_count ? (unsigned)sm_count : t;
}

// Sum of the row-CTAs' slabs -> canonical u32 (interleaved EF coordinates when NC = 4), zero beyond n.
template <int NC>
__global__ void fold_finalize_partials_kernel(const u32* __restrict__ part, u32 slabs, size_t n, size_t n_pad, u32* out) {
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_pad * NC; t += (size_t)gridDim.x * blockDim.x) {
        u64 v = 0;
        if (t < n * NC) {
#pragma unroll 8
            for (u32 r = 0; r < slabs; r++) v += part[(size_t)r * n * NC + t];
        }
        out[t] = red64(v);
    }
}
// acc -> canonical u32 (interleaved EF coordinates when NC = 4), zero beyond n up to n_pad.
template <int NC>
__global__ void fold_finalize_kernel(unsigned long long* acc, size_t n, size_t n_pad, u32* out) {
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_pad * NC; t += (size_t)gridDim.x * blockDim.x) {
        u32 v = 0;
        if (t < n * NC) { v = red64(acc[t]); acc[t] = 0; }
        out[t] = v;
    }
}

// ---- forward matvec: y[i] = sum_j W[i][j] x[j] (+ nothing; the Qwen path has no bias) ---------
// WPR warps share a row (each a contiguous quarter / half / ... of it), so that short matrices
// still put enough warps on every SM; every lane keeps four 16-byte loads in flight.  x is read
// through the read-only cache (it is small and reused by every row).  CTA = 8 warps = 8 / WPR rows.
// Up to four matrices that share the input vector and the column count are handled by one launch
// (the q / k / v / gate projections of a layer, or gate / up of its MLP): row i of the launch is
// row i - first[t] of matrix t.
struct MatvecBatch {
    const u32* W[4];
    u32* y[4];
    u32 first[5];        // first[t] = rows before matrix t; first[count] = total rows
    u32 count;
};

template <int WPR>
__device__ __forceinline__ u64 matvec_row_part(const u32* __restrict__ row, const u32* __restrict__ x, size_t n, int sub, int lane) {
    u64 acc = 0;
    if (n % 4 == 0) {
        // this warp's span of 16-byte groups
        const size_t groups = n / 4, per = (groups + WPR - 1) / WPR;
        const size_t g0 = (size_t)sub * per, g1 = g0 + per < groups ? g0 + per : groups;
        const uint4* rw = reinterpret_cast<const uint4*>(row);
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        size_t gidx = g0 + lane;
        for (; gidx + 96 < g1; gidx += 128) {
            uint4 w0 = __ldcs(rw + gidx), w1 = __ldcs(rw + gidx + 32), w2 = __ldcs(rw + gidx + 64), w3 = __ldcs(rw + gidx + 96);
            uint4 v0 = __ldg(xv + gidx), v1 = __ldg(xv + gidx + 32), v2 = __ldg(xv + gidx + 64), v3 = __ldg(xv + gidx + 96);
            acc += part_reduce((u64)w0.x * v0.x + (u64)w0.y * v0.y) + part_reduce((u64)w0.z * v0.z + (u64)w0.w * v0.w);
            acc += part_reduce((u64)w1.x * v1.x + (u64)w1.y * v1.y) + part_reduce((u64)w1.z * v1.z + (u64)w1.w * v1.w);
            acc += part_reduce((u64)w2.x * v2.x + (u64)w2.y * v2.y) + part_reduce((u64)w2.z * v2.z + (u64)w2.w * v2.w);
            acc += part_reduce((u64)w3.x * v3.x + (u64)w3.y * v3.y) + part_reduce((u64)w3.z * v3.z + (u64)w3.w * v3.w);
            acc = part_reduce(acc);             // 8 terms below 2^33 each: stays far below 2^64
        }
        for (; gidx < g1; gidx += 32) {
            uint4 w0 = rw[gidx];
            uint4 v0 = __ldg(xv + gidx);
            acc = part_reduce(acc + part_reduce((u64)w0.x * v0.x + (u64)w0.y * v0.y) + part_reduce((u64)w0.z * v0.z + (u64)w0.w * v0.w));
        }
    } else {
        const size_t per = (n + WPR - 1) / WPR;
        const size_t c0 = (size_t)sub * per, c1 = c0 + per < n ? c0 + per : n;
        for (size_t j = c0 + lane; j < c1; j += 32) acc = part_reduce(acc + part_reduce((u64)row[j] * __ldg(x + j)));
    }
    return acc;
}

template <int WPR>
__global__ void __launch_bounds__(256) matvec_forward_kernel(MatvecBatch mb, const u32* __restrict__ x, size_t n, int pf_rows) {
    __shared__ u32 part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = warp % WPR;                         // which part of the row
    constexpr int RPC = 8 / WPR;                        // rows per CTA
    const size_t m = mb.first[mb.count];
    // Launched as a programmatic dependent: the weights do not depend on the kernel before this one
    // (only x does), so while that kernel is still running every CTA pulls the rows of its first
    // pass into L2; then it waits for x.
    pdl_launch_dependents();
    {
        const size_t i0 = (size_t)blockIdx.x * RPC;
        const size_t lines_per_row = (n * 4 + 127) / 128;
        const size_t pf = (size_t)(pf_rows < RPC ? pf_rows : RPC);
        for (size_t q = threadIdx.x; q < pf * lines_per_row; q += blockDim.x) {
            const size_t i = i0 + q / lines_per_row;
            if (i < m) {
                u32 t = 0;
                while (t + 1 < mb.count && i >= mb.first[t + 1]) t++;
                prefetch_l2(reinterpret_cast<const char*>(mb.W[t] + (i - mb.first[t]) * n) + (q % lines_per_row) * 128);
            }
        }
    }
    pdl_wait();
    for (size_t i0 = (size_t)blockIdx.x * RPC; i0 < m; i0 += (size_t)gridDim.x * RPC) {
        const size_t i = i0 + warp / WPR;
        u64 acc = 0;
        u32 t = 0;
        if (i < m) {
            while (t + 1 < mb.count && i >= mb.first[t + 1]) t++;
            acc = matvec_row_part<WPR>(mb.W[t] + (i - mb.first[t]) * n, x, n, sub, lane);
        }
        u32 r = red64(acc);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) r = add31(r, __shfl_down_sync(0xffffffffu, r, off));
        if (WPR == 1) {
            if (lane == 0 && i < m) mb.y[t][i - mb.first[t]] = r;
        } else {
            if (lane == 0) part[warp] = r;
            __syncthreads();
            if (lane == 0 && sub == 0 && i < m) {
                u32 v = r;
#pragma unroll
                for (int q = 1; q < WPR; q++) v = add31(v, part[warp + q]);
                mb.y[t][i - mb.first[t]] = v;
            }
            __syncthreads();
        }
    }
}

// ---- forward matvec through a shared-memory ring filled by bulk asynchronous copies ---------------------
// One persistent CTA per SM: warp MVB_CONSUMER_WARPS issues one bulk copy (cp.async.bulk, global ->
// this CTA's shared memory, completion counted on an mbarrier) per tile of R whole rows into a ring of
// S stages; the other warps multiply tiles out of shared memory against x, which also sits there.
// The bytes in flight per SM are the ring (up to ~160 KB), not what fits the registers of the
// resident warps, which is what bounds the register-staged kernel above.  Rows of one tile are
// split over MVB_CONSUMER_WARPS / R warps; the last of them to finish adds the partial sums (an
// arrival counter per row in shared memory, no CTA-wide barrier).  The copies of the first tiles are
// issued before the wait on the previous kernel (the weights do not depend on it, only x does).
// Every wait on an mbarrier is bounded; when one runs out the kernel records ST_COPY_TIMEOUT and the
// issuing thread still waits (bounded again) for its copies in flight before it returns.
constexpr int MVB_CONSUMER_WARPS = 16;
constexpr int MVB_THREADS = (MVB_CONSUMER_WARPS + 1) * 32;
constexpr unsigned long long MVB_WAIT_LIMIT_NS = 2000000000ull;
constexpr u32 ST_COPY_TIMEOUT = 10;

__device__ __forceinline__ u32 smem_addr(const void* p) { return (u32)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* b, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* b, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(b)) : "memory");
}
// Bounded by wall time (two seconds on the global timer, looked at every 256 tries), not by a try count:
// how long one try_wait may suspend the thread is up to the hardware.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* b, u32 parity) {
    unsigned long long t0 = 0;
    for (u32 it = 0;; it++) {
        u32 ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(smem_addr(b)), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 255) == 255) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > MVB_WAIT_LIMIT_NS) return false;
        }
    }
}
// global -> shared memory of this CTA, `bytes` a multiple of 16, both addresses 16-byte aligned
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, u32 bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

struct MvbShape { u32 n, R, S, n_al; };     // columns, rows per tile, stages, x length rounded up to 32 words
__host__ __device__ inline size_t mvb_smem_bytes(const MvbShape& sh) {
    return (size_t)sh.n_al * 4 + (size_t)sh.S * sh.R * sh.n * 4 + (size_t)sh.S * 16 + (size_t)sh.S * (MVB_CONSUMER_WARPS + 8) * 4 + 64;
}
// tile g of the batch: matrix t, first row r0, rows in it
__device__ __forceinline__ void mvb_locate(const MatvecBatch& mb, u32 R, u32 g, u32& t, u32& r0, u32& rows) {
    t = 0;
    for (;;) {
        const u32 m_t = mb.first[t + 1] - mb.first[t];
        const u32 tiles_t = (m_t + R - 1) / R;
        if (g < tiles_t || t + 1 >= mb.count) { r0 = g * R; rows = m_t - r0 < R ? m_t - r0 : R; return; }
        g -= tiles_t;
        t++;
    }
}
__global__ void __launch_bounds__(MVB_THREADS, 1) matvec_forward_bulk_kernel(MatvecBatch mb, const u32* __restrict__ x, MvbShape sh, u32 n_tiles, u32* status) {
    extern __shared__ __align__(128) unsigned char mvb_smem[];
    u32* xs = reinterpret_cast<u32*>(mvb_smem);
    u32* ring = xs + sh.n_al;
    const u32 stage_words = sh.R * sh.n;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(ring + (size_t)sh.S * stage_words);
    unsigned long long* empty = full + sh.S;
    u32* part = reinterpret_cast<u32*>(empty + sh.S);            // [S][MVB_CONSUMER_WARPS]
    u32* cnt = part + sh.S * MVB_CONSUMER_WARPS;                 // [S][8]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (u32 s = 0; s < sh.S; s++) { mbar_init(full + s, 1); mbar_init(empty + s, MVB_CONSUMER_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (u32 i = threadIdx.x; i < sh.S * 8; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    pdl_launch_dependents();
    if (warp == MVB_CONSUMER_WARPS) {
        if (lane == 0) {
            u32 k = 0;
            bool ok = true;
            for (u32 g = blockIdx.x; g < n_tiles; g += gridDim.x, k++) {
                const u32 s = k % sh.S, ph = (k / sh.S) & 1;
                if (!mbar_wait_bounded(empty + s, ph ^ 1)) { atomicExch(status, ST_COPY_TIMEOUT); ok = false; break; }
                u32 t, r0, rows;
                mvb_locate(mb, sh.R, g, t, r0, rows);
                const u32 bytes = rows * sh.n * 4;
                mbar_arrive_expect_tx(full + s, bytes);
                bulk_copy_g2s(ring + (size_t)s * stage_words, mb.W[t] + (size_t)r0 * sh.n, bytes, full + s);
            }
            // no copy of this thread may still be in flight when it leaves: wait for the last use of every stage
            for (u32 j = 0; j < sh.S && j < k; j++) {
                const u32 kk = k - 1 - j, s = kk % sh.S, ph = (kk / sh.S) & 1;
                if (!mbar_wait_bounded(full + s, ph) && ok) { atomicExch(status, ST_COPY_TIMEOUT); ok = false; }
            }
        }
        return;
    }
    pdl_wait();                                   // x comes from the kernel before this one
    {
        const uint4* xg = reinterpret_cast<const uint4*>(x);
        uint4* xv = reinterpret_cast<uint4*>(xs);
        for (u32 i = threadIdx.x; i < sh.n / 4; i += MVB_CONSUMER_WARPS * 32) xv[i] = __ldg(xg + i);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(MVB_CONSUMER_WARPS * 32) : "memory");
    const u32 wpr = MVB_CONSUMER_WARPS / sh.R;    // warps per row
    const u32 row_in_tile = warp / wpr, sub = warp % wpr;
    const u32 groups = sh.n / 4, per = (groups + wpr - 1) / wpr;
    const u32 g0 = sub * per, g1 = g0 + per < groups ? g0 + per : groups;
    u32 k = 0;
    for (u32 g = blockIdx.x; g < n_tiles; g += gridDim.x, k++) {
        const u32 s = k % sh.S, ph = (k / sh.S) & 1;
        if (!mbar_wait_bounded(full + s, ph)) { if (lane == 0) atomicExch(status, ST_COPY_TIMEOUT); break; }
        u32 t, r0, rows;
        mvb_locate(mb, sh.R, g, t, r0, rows);
        if (row_in_tile < rows) {
            const uint4* rw = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_words + (size_t)row_in_tile * sh.n);
            const uint4* xv = reinterpret_cast<const uint4*>(xs);
            u64 acc = 0;
            u32 gi = g0 + lane;
            for (; gi + 96 < g1; gi += 128) {
                const uint4 w0 = rw[gi], w1 = rw[gi + 32], w2 = rw[gi + 64], w3 = rw[gi + 96];
                const uint4 v0 = xv[gi], v1 = xv[gi + 32], v2 = xv[gi + 64], v3 = xv[gi + 96];
                acc += part_reduce((u64)w0.x * v0.x + (u64)w0.y * v0.y) + part_reduce((u64)w0.z * v0.z + (u64)w0.w * v0.w);
                acc += part_reduce((u64)w1.x * v1.x + (u64)w1.y * v1.y) + part_reduce((u64)w1.z * v1.z + (u64)w1.w * v1.w);
                acc += part_reduce((u64)w2.x * v2.x + (u64)w2.y * v2.y) + part_reduce((u64)w2.z * v2.z + (u64)w2.w * v2.w);
                acc += part_reduce((u64)w3.x * v3.x + (u64)w3.y * v3.y) + part_reduce((u64)w3.z * v3.z + (u64)w3.w * v3.w);
                acc = part_reduce(acc);
            }
            for (; gi < g1; gi += 32) {
                const uint4 w0 = rw[gi], v0 = xv[gi];
                acc = part_reduce(acc + part_reduce((u64)w0.x * v0.x + (u64)w0.y * v0.y) + part_reduce((u64)w0.z * v0.z + (u64)w0.w * v0.w));
            }
            u32 r = red64(acc);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) r = add31(r, __shfl_down_sync(0xffffffffu, r, off));
            if (lane == 0) {
                if (wpr == 1) {
                    mb.y[t][r0 + row_in_tile] = r;
                } else {
                    volatile u32* pv = part + s * MVB_CONSUMER_WARPS;
                    pv[warp] = r;
                    __threadfence_block();
                    if (atomicAdd(cnt + s * 8 + row_in_tile, 1u) == wpr - 1) {
                        __threadfence_block();
                        u32 v = 0;
                        for (u32 q = 0; q < wpr; q++) v = add31(v, pv[row_in_tile * wpr + q]);
                        mb.y[t][r0 + row_in_tile] = v;
                        cnt[s * 8 + row_in_tile] = 0;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);    // this warp has read everything it needs from the stage
    }
}

}  // namespace zkb
