// Forward-pass helpers of a Qwen-style layer at seq_len = 1 (the matvecs are in linear.cuh).
//
//   rmsnorm_forward            rust/zk_ml_prover/src/transformer/mod.rs:245-288
//   requantize_to_i16_field    rust/zk_ml_prover/src/transformer/mod.rs:293-324
//   lookup + gating            rust/zk_ml_prover/src/transformer/qwen.rs:286-316
#pragma once
#include "logup.cuh"

namespace zkb {

// a^((p-1)/2) == 1 (0 counts as a residue), common.rs:44-53
__device__ __forceinline__ bool is_qr31(u32 a) {
    if (a == 0) return true;
    u32 r = a;
    for (int i = 0; i < 30; i++) r = mul31(r, r);
    return mul31(r, inv31(a)) == 1;
}
// a^(2^29), common.rs:34-40
__device__ __forceinline__ u32 sqrt31(u32 a) {
    u32 r = a;
    for (int i = 0; i < 29; i++) r = mul31(r, r);
    return r;
}

// Single CTA.  out[i] = gamma[i] * x'[i] * r with r = sqrt(d / sum x'^2); x' = x except that
// x'[0] = x[0] + delta for the first delta in 0, +1, -1, +2, -2, ... that makes d / sum_sq a
// quadratic residue.  scalars[0] = delta (two's complement), scalars[1] = sum_sq of x'.
// Vectors are written zero-padded to n_pad.  With `addend`, the input is x + addend (the residual
// add in front of the second norm), which is also written, zero-padded, to sum_out; every thread
// reads back only elements it wrote itself.
__global__ void __launch_bounds__(1024) rmsnorm_forward_kernel(const u32* __restrict__ x, const u32* __restrict__ gamma, u32 d, u32 n_pad,
                                                               u32* out, u32* x_used, u32* scalars, u32* status,
                                                               const u32* __restrict__ addend = nullptr, u32* sum_out = nullptr) {
    __shared__ u32 red[32];
    __shared__ u32 sh[3];   // r, x0', ok
    pdl_small_prologue();
    u32 acc = 0;
    if (addend) {
        for (u32 i = threadIdx.x; i < n_pad; i += blockDim.x) {
            const u32 v = i < d ? add31(x[i], addend[i]) : 0u;
            sum_out[i] = v;
            acc = add31(acc, mul31(v, v));
        }
    } else {
        for (u32 i = threadIdx.x; i < d; i += blockDim.x) acc = add31(acc, mul31(x[i], x[i]));
    }
    u32 w[1] = {acc};
    block_sum_words<1>(w, red);
    const u32* xin = addend ? sum_out : x;     // plain pointer: sum_out was written above, by the same threads that read it
    if (threadIdx.x == 0) {
        const u32 sum_sq = w[0], x0 = xin[0];
        u32 ok = 0, r = 0, nx0 = x0, ssq = sum_sq;
        int delta = 0;
        if (sum_sq != 0) {
            u32 target = mul31(d, inv31(sum_sq));
            if (is_qr31(target)) { ok = 1; r = sqrt31(target); }
        }
        for (int dl = 1; dl < 100 && !ok; dl++) {
            for (int s = 0; s < 2 && !ok; s++) {
                int pert = s == 0 ? dl : -dl;
                u32 adj = pert > 0 ? (u32)pert : ZKB_P - (u32)(-pert);
                u32 cand = add31(x0, adj);
                u32 cs = add31(sub31(sum_sq, mul31(x0, x0)), mul31(cand, cand));
                if (cs == 0) continue;
                u32 target = mul31(d, inv31(cs));
                if (is_qr31(target)) { ok = 1; r = sqrt31(target); nx0 = cand; delta = pert; ssq = cs; }
            }
        }
        if (!ok) atomicExch(status, (u32)ST_NOT_QR);
        sh[0] = r; sh[1] = nx0; sh[2] = ok;
        scalars[0] = (u32)delta;
        scalars[1] = ssq;
    }
    __syncthreads();
    const u32 r = sh[0], nx0 = sh[1];
    for (u32 i = threadIdx.x; i < n_pad; i += blockDim.x) {
        u32 xi = i < d ? (i == 0 ? nx0 : xin[i]) : 0u;
        x_used[i] = xi;
        out[i] = i < d ? mul31(mul31(gamma[i], xi), r) : 0u;
    }
}

__device__ __forceinline__ long long centered(u32 v) { return v > ZKB_P / 2 ? (long long)v - (long long)ZKB_P : (long long)v; }
__device__ __forceinline__ u32 to_field_i64(long long x) { return x >= 0 ? (u32)((unsigned long long)x % ZKB_P) : sub31(0u, (u32)((unsigned long long)(-x) % ZKB_P)); }

// q = requantize(raw); t = table[q]; prod = other . t  (all zero-padded to n_pad).
// Every CTA first finds the largest magnitude of the whole vector by itself (n is a few thousand
// words, read from L2), so no separate single-CTA launch sits in the forward chain; CTA 0 records it.
__global__ void __launch_bounds__(256) requant_lookup_mul_apply_kernel(const u32* __restrict__ raw, u32 n, u32 n_pad, unsigned long long* max_abs_out,
                                                const u32* __restrict__ table_out, u32 n_table, const u32* __restrict__ other,
                                                u32* q_out, u32* t_out, u32* prod_out, u32* status) {
    __shared__ unsigned long long mx_s[8];
    pdl_small_prologue();
    unsigned long long mx = 1;
    for (u32 i = threadIdx.x; i < n; i += blockDim.x) {
        long long s = centered(raw[i]);
        unsigned long long a = (unsigned long long)(s < 0 ? -s : s);
        mx = a > mx ? a : mx;
    }
    for (int off = 16; off > 0; off >>= 1) {
        unsigned long long o = __shfl_down_sync(0xffffffffu, mx, off);
        mx = o > mx ? o : mx;
    }
    if ((threadIdx.x & 31) == 0) mx_s[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = 1;
    for (u32 wv = 0; wv < (blockDim.x + 31) / 32; wv++) mx = mx_s[wv] > mx ? mx_s[wv] : mx;
    if (blockIdx.x == 0 && threadIdx.x == 0) *max_abs_out = mx;
    const long long max_abs = (long long)mx;
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += gridDim.x * blockDim.x) {
        u32 q = 0, t = 0, pr = 0;
        if (i < n) {
            long long v = centered(raw[i]), scaled;
            if (max_abs <= 32767) scaled = v;
            else {
                long long half = max_abs / 2;
                scaled = v >= 0 ? (v * 32767 + half) / max_abs : (v * 32767 - half) / max_abs;
            }
            scaled = scaled < -32768 ? -32768 : (scaled > 32767 ? 32767 : scaled);
            q = to_field_i64(scaled);
            u32 idx = field_to_table_index(q, n_table);
            if (idx >= n_table) { atomicExch(status, (u32)ST_LOOKUP_KEY); idx = 0; }
            t = table_out[idx];
            pr = mul31(other[i], t);
        }
        q_out[i] = q; t_out[i] = t; prod_out[i] = pr;
    }
}

// out = a + b (n valid, zero-padded to n_pad)
__global__ void add_vec_kernel(const u32* __restrict__ a, const u32* __restrict__ b, u32 n, u32 n_pad, u32* out) {
    pdl_small_prologue();
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += gridDim.x * blockDim.x)
        out[i] = i < n ? add31(a[i], b[i]) : 0u;
}
// GQA head replication at seq_len = 1 (qwen.rs:272-284): out[h*d_head + d] = v[(h / group) * d_head + d]
__global__ void replicate_heads_kernel(const u32* __restrict__ v, u32 num_q_heads, u32 group, u32 d_head, u32 n_pad, u32* out) {
    pdl_small_prologue();
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += gridDim.x * blockDim.x) {
        u32 h = i / d_head, d = i % d_head;
        out[i] = h < num_q_heads ? v[(h / group) * d_head + d] : 0u;
    }
}

}  // namespace zkb
