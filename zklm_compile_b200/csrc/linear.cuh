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
// grid.x tiles columns (blockDim.x * 4 per CTA), grid.y tiles rows.  Each CTA adds its partial
// column sums (canonical, < 2^31) to 64-bit accumulators with atomicAdd; integer addition is
// associative, so the result does not depend on the order.  NC = 1 (base eq) or 4 (EF eq).
constexpr int FOLD_ROWS_TILE = 64;

__device__ __forceinline__ u64 part_reduce(u64 a) { return (a & ZKB_P) + (a >> 31); }   // keeps a < 2^34

template <int NC>
__global__ void __launch_bounds__(128) fold_eq_matvec_kernel(const u32* __restrict__ W, size_t m, size_t n,
                                                            const u32* __restrict__ eq /* [m_pad][NC] */,
                                                            size_t rows_per_cta, unsigned long long* acc /* [n][NC] */) {
    __shared__ u32 eq_s[FOLD_ROWS_TILE * NC];
    const size_t j0 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const size_t r0 = (size_t)blockIdx.y * rows_per_cta;
    const size_t r1 = r0 + rows_per_cta < m ? r0 + rows_per_cta : m;
    const bool vec = (n % 4 == 0) && (j0 + 4 <= n);
    u64 a[4][NC];
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
        for (int k = 0; k < NC; k++) a[c][k] = 0;

    for (size_t rb = r0; rb < r1; rb += FOLD_ROWS_TILE) {
        const int rows = (int)(r1 - rb < FOLD_ROWS_TILE ? r1 - rb : FOLD_ROWS_TILE);
        __syncthreads();
        for (int t = threadIdx.x; t < rows * NC; t += blockDim.x) eq_s[t] = eq[rb * NC + t];
        __syncthreads();
        if (j0 < n) {
            // three rows per step: their 16-byte loads are issued together (more bytes in flight per
            // thread), their products (< 2^62 each) are summed unreduced and folded once
            int rr = 0;
            for (; rr + 3 <= rows; rr += 3) {
                u32 w[3][4];
#pragma unroll
                for (int q = 0; q < 3; q++) {
                    const u32* row = W + (rb + rr + q) * n;
                    if (vec) {
                        uint4 t = *reinterpret_cast<const uint4*>(row + j0);
                        w[q][0] = t.x; w[q][1] = t.y; w[q][2] = t.z; w[q][3] = t.w;
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; c++) w[q][c] = (j0 + c < n) ? row[j0 + c] : 0u;
                    }
                }
#pragma unroll
                for (int k = 0; k < NC; k++) {
                    const u32 e0 = eq_s[rr * NC + k], e1 = eq_s[(rr + 1) * NC + k], e2 = eq_s[(rr + 2) * NC + k];
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        a[c][k] = part_reduce(a[c][k] + (u64)e0 * w[0][c] + (u64)e1 * w[1][c] + (u64)e2 * w[2][c]);
                }
            }
            for (; rr < rows; rr++) {
                const u32* row = W + (rb + rr) * n;
                u32 w[4];
#pragma unroll
                for (int c = 0; c < 4; c++) w[c] = (j0 + c < n) ? row[j0 + c] : 0u;
#pragma unroll
                for (int k = 0; k < NC; k++) {
                    const u32 e = eq_s[rr * NC + k];
#pragma unroll
                    for (int c = 0; c < 4; c++) a[c][k] = part_reduce(a[c][k] + (u64)e * w[c]);
                }
            }
        }
    }
    if (j0 < n) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            if (j0 + c < n) {
#pragma unroll
                for (int k = 0; k < NC; k++) atomicAdd(acc + (j0 + c) * NC + k, (unsigned long long)red64(a[c][k]));
            }
        }
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
// One warp per row; x is read through the read-only cache (it is small and reused by every row).
__global__ void __launch_bounds__(256) matvec_forward_kernel(const u32* __restrict__ W, const u32* __restrict__ x,
                                                             size_t m, size_t n, u32* y) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t i = warp; i < m; i += nwarps) {
        const u32* row = W + i * n;
        u64 acc = 0;
        if (n % 4 == 0) {
            int since = 0;
            for (size_t j = (size_t)lane * 4; j < n; j += 128) {
                uint4 w = *reinterpret_cast<const uint4*>(row + j);
                uint4 v = __ldg(reinterpret_cast<const uint4*>(x + j));
                u64 t = (u64)w.x * v.x + (u64)w.y * v.y;      // two products < 2^63
                u64 u = (u64)w.z * v.z + (u64)w.w * v.w;
                acc += part_reduce(t) + part_reduce(u);
                if (++since == (1 << 20)) { since = 0; acc = part_reduce(acc); }
            }
        } else {
            for (size_t j = lane; j < n; j += 32) acc += part_reduce((u64)row[j] * __ldg(x + j));
        }
        u32 r = red64(acc);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) r = add31(r, __shfl_down_sync(0xffffffffu, r, off));
        if (lane == 0) y[i] = r;
    }
}

}  // namespace zkb
