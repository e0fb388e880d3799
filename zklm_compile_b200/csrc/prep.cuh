// Small "glue" kernels between sumchecks: table preparation for MLE-eval / hadamard / add /
// RMSNorm proofs and the seq_len = 1 attention consistency check.  Vectors handled here are
// at most a few 10^4 elements (one model dimension), so these are latency-, not bandwidth-bound;
// the point of fusing them is fewer launches on the critical path.
#pragma once
#include "linear.cuh"
#include "sumcheck.cuh"

namespace zkb {

// Up to three base-field vectors widened to EF plus (optionally) the eq table at an EF point,
// all of length 2^k.  src[i] may be shorter than 2^k (`len[i]` valid entries, rest zero).
struct WidenEqArgs {
    const u32* src[3];
    Fe* dst[3];
    u32 len[3];
    u32 nsrc;
    const Fe* point;   // nullptr: no eq table
    Fe* eq_out;
    u32 k;
};
__global__ void widen_eq_kernel(WidenEqArgs a) {
    const size_t n = size_t(1) << a.k;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        for (u32 t = 0; t < a.nsrc; t++) {
            u32 v = i < a.len[t] ? a.src[t][i] : 0u;
            st_fe(a.dst[t] + i, Fe{v, 0, 0, 0});
        }
        if (a.point) st_fe(a.eq_out + i, eq_at_index<Fe>(a.point, a.k, i));
    }
}
// out[i] = a[i] * b[i] (i < n), zero up to n_pad; optionally also sum_i x[i]^2 into *sumsq
// (single CTA; rmsnorm.rs:532-540: g = gamma . x and sum_sq).
__global__ void __launch_bounds__(1024) rmsnorm_prep_kernel(const u32* __restrict__ x, const u32* __restrict__ gamma, u32 d, u32 n_pad,
                                                            u32* g_out, u32* sumsq_out) {
    __shared__ u32 red[32];
    u32 acc = 0;
    for (u32 i = threadIdx.x; i < n_pad; i += blockDim.x) {
        u32 xi = i < d ? x[i] : 0u;
        g_out[i] = i < d ? mul31(gamma[i], xi) : 0u;
        acc = add31(acc, mul31(xi, xi));
    }
    u32 w[1] = {acc};
    block_sum_words<1>(w, red);
    if (threadIdx.x == 0) *sumsq_out = w[0];
}

// One CTA per message: root[blockIdx.x] = blake3(prefix || words_i).
struct B3Multi {
    const u32* words[4];
    u32 n_words[4];
    u32* root[4];
    u32* cvs[4];
};
__global__ void __launch_bounds__(256) b3_commit_multi_kernel(B3Prefix pre, B3Multi m) {
    const int b = blockIdx.x;
    b3_hash_block(pre, m.words[b], m.n_words[b], m.cvs[b]);
    if (threadIdx.x == 0)
        for (int i = 0; i < 8; i++) m.root[b][i] = m.cvs[b][i];
}

// seq_len = 1 attention consistency (rust/zk_ml_prover/src/transformer/qwen.rs:838-876):
// squeeze log_attn base challenges r, evaluate the MLE of attn_out at r and of v at r (GDN) or at
// [r[..log_kv] || r[len-log_d..]] (GQA), absorb both values, record them.
__global__ void __launch_bounds__(1024) seq1_consistency_kernel(TrState* st, const u32* __restrict__ attn_out, u32 attn_len, u32 log_attn,
                                                                const u32* __restrict__ v, u32 v_len, u32 log_v, u32 is_gqa, u32 log_kv,
                                                                u32 log_d, u32* out2) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ Fp r_s[32], rv_s[32];
    __shared__ u32 red[64];
    Tr tr;
    if (threadIdx.x == 0) {
        tr_load(tr, st, trbuf);
        for (u32 i = 0; i < log_attn; i++) r_s[i].v = tr_squeeze(tr);
        if (!is_gqa) for (u32 i = 0; i < log_v; i++) rv_s[i] = r_s[i];
        else {
            for (u32 i = 0; i < log_kv; i++) rv_s[i] = r_s[i];
            for (u32 i = 0; i < log_d; i++) rv_s[log_kv + i] = r_s[log_attn - log_d + i];
        }
    }
    __syncthreads();
    u32 acc[2] = {0, 0};
    for (u32 i = threadIdx.x; i < attn_len; i += blockDim.x)
        acc[0] = add31(acc[0], mul31(eq_at_index<Fp>(r_s, log_attn, i).v, attn_out[i]));
    for (u32 i = threadIdx.x; i < v_len; i += blockDim.x)
        acc[1] = add31(acc[1], mul31(eq_at_index<Fp>(rv_s, log_v, i).v, v[i]));
    block_sum_words<2>(acc, red);
    if (threadIdx.x == 0) {
        tr_absorb_u32(tr, acc[0]);
        tr_absorb_u32(tr, acc[1]);
        tr_store(tr, st);
        out2[0] = acc[0];
        out2[1] = acc[1];
    }
}

// dst[i] = src[i] for i < n, 0 for n <= i < n_pad.
__global__ void pad_copy_kernel(const u32* __restrict__ src, size_t n, size_t n_pad, u32* dst) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = i < n ? src[i] : 0u;
}

}  // namespace zkb
