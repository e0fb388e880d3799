// LogUp lookup argument, device side (rust/zk_ml_prover/src/proving/lookup.rs:643-762, EF;
// :432-604 base field).  Table entry `raw` has input i16_to_field(raw as i16); the output
// column is built on the host (f64 math) and uploaded once.
//
//   multiplicities      histogram of the lookup inputs over the table     (lookup.rs:396-411)
//   active subtable     entries with m > 0, in ascending table index       (lookup.rs:675-699)
//   h                   h[i] = 1/(alpha - f_i), h[n+k] = -m_k/(alpha - T_k) (lookup.rs:706-729)
// Inverses are computed per element (each thread inverts its own denominators after a
// Montgomery batch of LOGUP_BATCH); field inverses are unique, so the values equal the
// reference's serial Montgomery pass.
#pragma once
#include "m31.cuh"
#include "sumcheck.cuh"

namespace zkb {

enum : u32 { ST_OK = 0, ST_LOGUP_IDENTITY = 3, ST_ALPHA_COLLISION = 4, ST_NOT_QR = 5, ST_LOOKUP_KEY = 8 };

// lookup.rs:377-390
__device__ __forceinline__ u32 field_to_table_index(u32 v, u32 n_table) {
    u32 half = n_table / 2;
    if (v < half) return v;
    if (v >= ZKB_P - half) return v + n_table - ZKB_P;
    return 0xffffffffu;
}
__device__ __forceinline__ u32 table_input_at(u32 raw, u32 n_table) {
    // i16_to_field(raw as i16) (or i8 for 256-entry tables)
    u32 half = n_table / 2;
    return raw < half ? raw : ZKB_P - (n_table - raw);
}

__global__ void logup_hist_kernel(const u32* __restrict__ inputs, u32 n, u32 n_table, u32* mult) {
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        u32 idx = field_to_table_index(inputs[i], n_table);
        if (idx < n_table) atomicAdd(mult + idx, 1u);
    }
}

// Single CTA: stable compaction of the nonzero multiplicities.
//   act_idx[k], act_mult[k], act_entry[k] = table_in + table_out (one F per entry, lookup.rs:690-699)
//   dyn[0] = n_active, dyn[1] = num_vars = log2_ceil(n + n_active), dyn[2] = n
__global__ void __launch_bounds__(1024) logup_compact_kernel(const u32* __restrict__ mult, const u32* __restrict__ table_out, u32 n_table,
                                                             u32 n_lookups, u32* act_idx, u32* act_mult, u32* act_entry, u32* dyn) {
    __shared__ u32 counts[1024];
    const u32 per = (n_table + blockDim.x - 1) / blockDim.x;
    const u32 lo = threadIdx.x * per, hi = lo + per < n_table ? lo + per : n_table;
    u32 c = 0;
    for (u32 j = lo; j < hi; j++) c += mult[j] != 0;
    counts[threadIdx.x] = c;
    __syncthreads();
    // inclusive scan (Hillis-Steele)
    for (u32 off = 1; off < blockDim.x; off <<= 1) {
        u32 v = threadIdx.x >= off ? counts[threadIdx.x - off] : 0u;
        __syncthreads();
        counts[threadIdx.x] += v;
        __syncthreads();
    }
    u32 pos = counts[threadIdx.x] - c;
    for (u32 j = lo; j < hi; j++) {
        u32 mj = mult[j];
        if (mj) {
            act_idx[pos] = j;
            act_mult[pos] = mj;
            act_entry[pos] = add31(table_input_at(j, n_table), table_out[j]);
            pos++;
        }
    }
    if (threadIdx.x == blockDim.x - 1) {
        u32 n_active = counts[threadIdx.x];
        u32 total = n_lookups + n_active, nv = 1;
        while ((1u << nv) < total) nv++;
        dyn[0] = n_active; dyn[1] = nv; dyn[2] = n_lookups;
    }
}

// Base-field path: the committed active subtable is inp + beta * out (lookup.rs:466-481).
__global__ void logup_encode_active_kernel(const u32* __restrict__ act_idx, const u32* __restrict__ dyn, const u32* __restrict__ table_out,
                                           u32 n_table, const u32* __restrict__ beta, u32* out) {
    const u32 n_active = dyn[0], b = beta[0];
    for (u32 k = blockIdx.x * blockDim.x + threadIdx.x; k < n_active; k += gridDim.x * blockDim.x) {
        u32 j = act_idx[k];
        out[k] = add31(table_input_at(j, n_table), mul31(b, table_out[j]));
    }
}

constexpr int LOGUP_BATCH = 4;

template <class ChalT> struct LogupEnc;
template <> struct LogupEnc<Fe> {
    static __device__ __forceinline__ Fe enc(u32 a, u32 b, Fe beta) { Fe t = beta * Fp{b}; t.x = add31(t.x, a); return t; }
    static __device__ __forceinline__ bool is_zero(Fe v) { return (v.x | v.y | v.z | v.w) == 0; }
    static __device__ __forceinline__ Fe inv(Fe v) { return fe_inv(v); }
    static __device__ __forceinline__ Fe neg_scaled(Fe v, u32 m) { return fe_zero() - v * Fp{m}; }
};
template <> struct LogupEnc<Fp> {
    static __device__ __forceinline__ Fp enc(u32 a, u32 b, Fp beta) { return Fp{add31(a, mul31(beta.v, b))}; }
    static __device__ __forceinline__ bool is_zero(Fp v) { return v.v == 0; }
    static __device__ __forceinline__ Fp inv(Fp v) { return Fp{inv31(v.v)}; }
    static __device__ __forceinline__ Fp neg_scaled(Fp v, u32 m) { return fp_zero() - v * Fp{m}; }
};

// h over the combined domain, zero-filled up to `cap` elements.  chal[0] = beta, chal[1] = alpha.
template <class ChalT>
__global__ void logup_h_kernel(const u32* __restrict__ inputs, const u32* __restrict__ outputs, const u32* __restrict__ table_out,
                               u32 n_table, const u32* __restrict__ act_idx, const u32* __restrict__ act_mult,
                               const u32* __restrict__ dyn, const ChalT* __restrict__ chal, ChalT* h, u32 cap, u32* status) {
    const u32 n = dyn[2], n_active = dyn[0], total = n + n_active;
    const ChalT beta = ld_fe(chal), alpha = ld_fe(chal + 1);
    const u32 stride = gridDim.x * blockDim.x * LOGUP_BATCH;
    for (u32 base = (blockIdx.x * blockDim.x + threadIdx.x) * LOGUP_BATCH; base < cap; base += stride) {
        ChalT d[LOGUP_BATCH], pre[LOGUP_BATCH];
        u32 mk[LOGUP_BATCH];
        int cnt = 0;
#pragma unroll
        for (int t = 0; t < LOGUP_BATCH; t++) {
            u32 i = base + t;
            if (i < total) {
                ChalT enc;
                if (i < n) { enc = LogupEnc<ChalT>::enc(inputs[i], outputs[i], beta); mk[t] = 0; }
                else {
                    u32 j = act_idx[i - n];
                    enc = LogupEnc<ChalT>::enc(table_input_at(j, n_table), table_out[j], beta);
                    mk[t] = act_mult[i - n];
                }
                d[t] = alpha - enc;
                if (LogupEnc<ChalT>::is_zero(d[t])) atomicExch(status, (u32)ST_ALPHA_COLLISION);
                cnt = t + 1;
            }
        }
        // Montgomery batch over this thread's denominators: one inversion per LOGUP_BATCH
        bool any_zero = false;
        for (int t = 0; t < cnt; t++) any_zero |= LogupEnc<ChalT>::is_zero(d[t]);
        if (cnt > 0 && !any_zero) {
            pre[0] = d[0];
            for (int t = 1; t < cnt; t++) pre[t] = pre[t - 1] * d[t];
            ChalT inv = LogupEnc<ChalT>::inv(pre[cnt - 1]);
            for (int t = cnt - 1; t >= 0; t--) {
                ChalT it = t ? inv * pre[t - 1] : inv;
                if (t) inv = inv * d[t];
                u32 i = base + t;
                st_fe(h + i, i < n ? it : LogupEnc<ChalT>::neg_scaled(it, mk[t]));
            }
        } else {
            for (int t = 0; t < cnt; t++) st_fe(h + base + t, zero_of<ChalT>());
        }
#pragma unroll
        for (int t = 0; t < LOGUP_BATCH; t++)
            if (base + t >= total && base + t < cap) st_fe(h + base + t, zero_of<ChalT>());
    }
}

// words = [inputs (n) | n as u64 LE (2 words) | outputs (n)] for the external-data digest
// blake3("lookup-external-data-v1" || n u64 || inputs || n u64 || outputs) (lookup.rs:609-621).
__global__ void logup_digest_concat_kernel(const u32* __restrict__ inputs, const u32* __restrict__ outputs, u32 n, u32* dst) {
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < 2 * n + 2; i += gridDim.x * blockDim.x) {
        u32 v;
        if (i < n) v = inputs[i];
        else if (i == n) v = n;
        else if (i == n + 1) v = 0;
        else v = outputs[i - n - 2];
        dst[i] = v;
    }
}

}  // namespace zkb
