// The reference's op-list mode on the device: MLP / GPT-2 shaped models as a list of ops proved in
// reverse order on one transcript "structured-ml-proof" with base-field challenges.
//
//   forward pass of the ops          rust/zk_ml_prover/src/pipeline/forward.rs:24-520
//   sequential prover                rust/zk_ml_prover/src/pipeline/prove.rs:36, 191-648
//   squared LayerNorm                rust/zk_ml_prover/src/proving/layernorm.rs:445-695
//   layernorm_forward_simple         rust/zk_ml_prover/src/transformer/gpt2.rs:912-953
//   SerializedLayerProof variants    rust/zk_ml_prover/src/protocol.rs:653-694
//
// Weights are resident and their blake3 commitments are computed when an op is added (the
// reference hashes them inside its prove loop; the bytes are the same).  Activations stay on the
// device from the input vector to the last proof; the host only orders the launches and, at the
// end, serialises the record into bincode(Vec<SerializedLayerProof>).
#pragma once
#include "protocols2.cuh"
#include <memory>
#include <string>

namespace zkb {

// ---- forward kernels -----------------------------------------------------------------------------
// y[i] += b[i]
__global__ void bias_add_kernel(u32* y, const u32* __restrict__ b, u32 m) {
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < m; i += gridDim.x * blockDim.x) y[i] = add31(y[i], b[i]);
}
// relu on centred values (forward.rs:126-131): out = v if from_field(v) >= 0 else 0; zero-padded
__global__ void relu_forward_kernel(const u32* __restrict__ z, u32 n, u32 n_pad, u32* out) {
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += gridDim.x * blockDim.x)
        out[i] = (i < n && z[i] <= ZKB_P / 2) ? z[i] : 0u;
}
// a = relu(z), b = [z >= 0], 1 - b over the padded domain (prove.rs:243-261; padding entries are 0 >= 0, so b = 1 there)
__global__ void relu_prep_kernel(const u32* __restrict__ z, u32 n, u32 n_pad, u32* a, u32* b, u32* omb) {
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += gridDim.x * blockDim.x) {
        const u32 v = i < n ? z[i] : 0u;
        const bool pos = v <= ZKB_P / 2;
        a[i] = pos ? v : 0u; b[i] = pos ? 1u : 0u; omb[i] = pos ? 0u : 1u;
    }
}
__global__ void fill_kernel(u32* dst, u32 n, u32 v) {
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = v;
}
// q = requantize_to_i16_field(raw) (transformer/mod.rs:293-324), optionally t = table[q]; zero-padded.
// Every CTA finds the largest magnitude by itself (a few thousand words from L2).
__global__ void __launch_bounds__(256) requant_lookup_kernel(const u32* __restrict__ raw, u32 n, u32 n_pad, const u32* __restrict__ table_out,
                                                             u32 n_table, u32* q_out, u32* t_out, u32* status) {
    __shared__ unsigned long long mx_s[8];
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
    const long long max_abs = (long long)mx;
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += gridDim.x * blockDim.x) {
        u32 q = 0, t = 0;
        if (i < n) {
            long long v = centered(raw[i]), scaled;
            if (max_abs <= 32767) scaled = v;
            else {
                long long half = max_abs / 2;
                scaled = v >= 0 ? (v * 32767 + half) / max_abs : (v * 32767 - half) / max_abs;
            }
            scaled = scaled < -32768 ? -32768 : (scaled > 32767 ? 32767 : scaled);
            q = to_field_i64(scaled);
            if (table_out) {
                u32 idx = field_to_table_index(q, n_table);
                if (idx >= n_table) { atomicExch(status, (u32)ST_LOOKUP_KEY); idx = 0; }
                t = table_out[idx];
            }
        }
        q_out[i] = q;
        if (t_out) t_out[i] = t;
    }
}
// layernorm_forward_simple (gpt2.rs:912-953), single CTA.  With S1 = sum x and S2 = sum x^2 of the
// (perturbed) input, mu = S1 / d and sum (x - mu)^2 = S2 - S1 mu, so every candidate perturbation of
// x[0] costs a handful of multiplications.  Writes x' (perturbed input), xc = x' - mu, y = gamma xc r
// + beta, all zero-padded to n_pad, and scalars {perturbation, mu, sum_sq, r}.
__global__ void __launch_bounds__(1024) layernorm_forward_kernel(const u32* __restrict__ x, const u32* __restrict__ gamma, const u32* __restrict__ beta,
                                                                 u32 d, u32 n_pad, u32* x_used, u32* xc, u32* y, u32* scalars, u32* status) {
    __shared__ u32 red[32 * 2];
    __shared__ u32 sh[4];
    u32 w[2] = {0, 0};
    for (u32 i = threadIdx.x; i < d; i += blockDim.x) { w[0] = add31(w[0], x[i]); w[1] = add31(w[1], mul31(x[i], x[i])); }
    block_sum_words<2>(w, red);
    if (threadIdx.x == 0) {
        const u32 S1 = w[0], S2 = w[1], x0 = x[0], d_inv = inv31(d);
        u32 ok = 0, mu = 0, r = 0, ssq = 0, nx0 = x0;
        int pert = 0;
        for (int delta = 0; delta < 100 && !ok; delta++) {
            for (int s = 0; s < 2 && !ok; s++) {
                const int p = delta == 0 ? 0 : (s == 0 ? delta : -delta);
                const u32 adj = p >= 0 ? (u32)p : ZKB_P - (u32)(-p);
                const u32 c0 = add31(x0, adj);
                const u32 s1 = add31(S1, adj), s2 = add31(sub31(S2, mul31(x0, x0)), mul31(c0, c0));
                const u32 m = mul31(s1, d_inv);
                const u32 q = sub31(s2, mul31(s1, m));
                if (q != 0) {
                    const u32 target = mul31(d, inv31(q));
                    if (is_qr31(target)) { ok = 1; mu = m; r = sqrt31(target); ssq = q; nx0 = c0; pert = p; }
                }
                if (delta == 0) break;
            }
        }
        if (!ok) atomicExch(status, (u32)ST_NOT_QR);
        sh[0] = mu; sh[1] = r; sh[2] = nx0;
        scalars[0] = (u32)pert; scalars[1] = mu; scalars[2] = ssq; scalars[3] = r;
    }
    __syncthreads();
    const u32 mu = sh[0], r = sh[1], nx0 = sh[2];
    for (u32 i = threadIdx.x; i < n_pad; i += blockDim.x) {
        const u32 xi = i < d ? (i == 0 ? nx0 : x[i]) : 0u;
        const u32 c = i < d ? sub31(xi, mu) : 0u;
        x_used[i] = xi; xc[i] = c;
        y[i] = i < d ? add31(mul31(mul31(gamma[i], c), r), beta[i]) : 0u;
    }
}
// g = gamma * xc, h = y - beta over the padded domain (layernorm.rs:543-560)
__global__ void layernorm_prep_kernel(const u32* __restrict__ xc, const u32* __restrict__ gamma, const u32* __restrict__ beta,
                                      const u32* __restrict__ y, u32 d, u32 n_pad, u32* g, u32* h, u32* gamma_pad) {
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += gridDim.x * blockDim.x) {
        g[i] = i < d ? mul31(gamma[i], xc[i]) : 0u;
        h[i] = i < d ? sub31(y[i], beta[i]) : 0u;
        gamma_pad[i] = i < d ? gamma[i] : 0u;
    }
}

// SHA-256(len u32 LE || values u32 LE) of a device vector (hash_values, common.rs:78-85) as eight
// little-endian words of the digest bytes.
__global__ void __launch_bounds__(TRSCRIPT_THREADS) hash_values_kernel(const u32* __restrict__ v, u32 n, u32* digest_out) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ u32 tile[2 * 512];
    __shared__ u32 kw[2 * 32 * SHA_KW_STRIDE];
    __shared__ u32 bc[1];
    Tr tr;
    tr.buf = trbuf; tr.buflen = 0; tr.total = 0;
    if (threadIdx.x == 0) { tr_iv(tr.h); tr_absorb_u32(tr, n); }
    tr_absorb_stream_2w(tr, n, [=](u32 g) -> u32 { return v[g]; }, reinterpret_cast<u32*>(trbuf), tile, kw, bc);
    if (threadIdx.x == 0) {
        u32 d[8];
        tr_finalize_reseed(tr, d);
        for (int i = 0; i < 8; i++) digest_out[i] = bswap32(d[i]);
    }
}

// The same digest for a list of vectors, one CTA each: the content digests of an op list (save,
// set_input, attention, passthrough) depend only on the forward pass, not on the transcript, so they
// are all computed side by side in one launch instead of one after another between the proofs.
struct HashJob { const u32* v; u32 n; u32 _pad; };
__global__ void __launch_bounds__(TRSCRIPT_THREADS) hash_values_multi_kernel(const HashJob* __restrict__ jobs, u32* digests_out) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ u32 tile[2 * 512];
    __shared__ u32 kw[2 * 32 * SHA_KW_STRIDE];
    __shared__ u32 bc[1];
    const u32* v = jobs[blockIdx.x].v;
    const u32 n = jobs[blockIdx.x].n;
    Tr tr;
    tr.buf = trbuf; tr.buflen = 0; tr.total = 0;
    if (threadIdx.x == 0) { tr_iv(tr.h); tr_absorb_u32(tr, n); }
    tr_absorb_stream_2w(tr, n, [=](u32 g) -> u32 { return v[g]; }, reinterpret_cast<u32*>(trbuf), tile, kw, bc);
    if (threadIdx.x == 0) {
        u32 d[8];
        tr_finalize_reseed(tr, d);
        for (int i = 0; i < 8; i++) digests_out[8 * blockIdx.x + i] = bswap32(d[i]);
    }
}

// ---- squared LayerNorm (layernorm.rs:522-695) ----------------------------------------------------------
struct LayerNormRec {
    u32 k = 0;
    size_t scalars = 0;       // {mu, sum_sq}
    size_t roots = 0;         // xc, gamma, g, h
    ScRec mean, var, g_prod, g_triple, h_sq, g_sq;
    EvalRec xc_mean, xc_var, g_prod_eval, xc_triple, gamma_triple, h_sq_eval, g_sq_eval;
};
// xc, y: zero-padded to 2^k on the device; gamma, beta: d entries; fwd_scalars: {perturbation, mu, sum_sq, r}.
inline LayerNormRec prove_layernorm_sqr(zkb_ctx* c, TrState* tr, const u32* xc, const u32* gamma, const u32* beta, const u32* y, u32 d,
                                        const u32* fwd_scalars) {
    LayerNormRec R;
    R.k = log2_ceil_u(d);
    const u32 k = R.k;
    const size_t n = size_t(1) << k;
    u32* g = (u32*)c->scratch(n * 4 + 16);
    u32* h = (u32*)c->scratch(n * 4 + 16);
    u32* gamma_pad = (u32*)c->scratch(n * 4 + 16);
    u32* ones = (u32*)c->scratch(n * 4 + 16);
    R.scalars = c->rec_alloc(2);
    R.roots = c->rec_alloc(32);
    layernorm_prep_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(xc, gamma, beta, y, d, (u32)n, g, h, gamma_pad);
    ZKB_LAUNCHED(c);
    fill_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(ones, (u32)n, 1u);
    ZKB_LAUNCHED(c);
    ZKB_CUDA(cudaMemcpyAsync(c->rec_dev + R.scalars, fwd_scalars + 1, 8, cudaMemcpyDeviceToDevice, c->stream));
    B3Multi bm{};
    const u32* vecs[4] = {xc, gamma_pad, g, h};
    for (int i = 0; i < 4; i++) {
        bm.words[i] = vecs[i]; bm.n_words[i] = (u32)n; bm.root[i] = c->rec_dev + R.roots + 8 * i;
        bm.cvs[i] = (u32*)c->scratch((n * 4 + 7 + 1023) / 1024 * 32 + 64);
    }
    b3_commit_multi_kernel<<<4, 256, 0, c->stream>>>(b3_prefix("weights", 7), bm);
    ZKB_LAUNCHED(c);
    u32* discard = (u32*)c->scratch((size_t)k * 4 + 16);
    {
        ScriptBuilder sb;
        sb.words_dev(c->rec_dev + R.roots, 32);
        sb.words_dev(c->rec_dev + R.scalars, 2);      // mu, sum_sq
        sb.squeeze(discard, k);                       // _mean_point
        sb.run(c, tr);
    }
    const u32* root_xc = c->rec_dev + R.roots, *root_gamma = root_xc + 8, *root_g = root_xc + 16, *root_h = root_xc + 24;
    const u32* tm[3] = {ones, xc, nullptr};
    R.mean = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tm, k);
    R.xc_mean = prove_mle_eval_base(c, tr, xc, c->rec_dev + R.mean.chal, k, "lnsqr-xc-mean", root_xc);
    const u32* tv[3] = {xc, xc, nullptr};
    R.var = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tv, k);
    R.xc_var = prove_mle_eval_base(c, tr, xc, c->rec_dev + R.var.chal, k, "lnsqr-xc-var", root_xc);
    u32* gc_point = (u32*)c->scratch((size_t)k * 4 + 16);
    { ScriptBuilder sb; sb.squeeze(gc_point, k); sb.run(c, tr); }
    Fp* eq = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)gc_point, k, eq);
    ZKB_LAUNCHED(c);
    const u32* tgp[3] = {(const u32*)eq, g, nullptr};
    R.g_prod = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tgp, k);
    R.g_prod_eval = prove_mle_eval_base(c, tr, g, c->rec_dev + R.g_prod.chal, k, "lnsqr-g-prod", root_g);
    const u32* tgt[3] = {(const u32*)eq, gamma_pad, xc};
    R.g_triple = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, tgt, k);
    const u32* s_gt = c->rec_dev + R.g_triple.chal;
    R.xc_triple = prove_mle_eval_base(c, tr, xc, s_gt, k, "lnsqr-xc-triple", root_xc);
    R.gamma_triple = prove_mle_eval_base(c, tr, gamma_pad, s_gt, k, "lnsqr-gamma-triple", root_gamma);
    u32* sq_point = (u32*)c->scratch((size_t)k * 4 + 16);
    { ScriptBuilder sb; sb.squeeze(sq_point, k); sb.run(c, tr); }
    Fp* eq2 = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)sq_point, k, eq2);
    ZKB_LAUNCHED(c);
    const u32* ths[3] = {(const u32*)eq2, h, h};
    R.h_sq = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, ths, k);
    R.h_sq_eval = prove_mle_eval_base(c, tr, h, c->rec_dev + R.h_sq.chal, k, "lnsqr-h-sq", root_h);
    const u32* tgs[3] = {(const u32*)eq2, g, g};
    R.g_sq = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, tgs, k);
    R.g_sq_eval = prove_mle_eval_base(c, tr, g, c->rec_dev + R.g_sq.chal, k, "lnsqr-g-sq", root_g);
    return R;
}
// LayerNormSqrProof in serde field order (layernorm.rs:468-519)
inline void put_layernorm_sqr(Ser& s, const LayerNormRec& R) {
    const u64 n = u64(1) << R.k;
    s.u32le(s.rec[R.scalars]);                                       // mu
    s.sumcheck(R.mean, true); s.words(R.mean.fin, 2);
    s.sumcheck(R.var, true); s.words(R.var.fin, 2);
    s.u32le(s.rec[R.scalars + 1]);                                   // sum_sq_value
    s.sumcheck(R.g_prod, true); s.words(R.g_prod.fin, 2);
    s.sumcheck(R.g_triple, true); s.words(R.g_triple.fin, 3);
    put_claimed_sum_base(s, R.g_prod);                               // t_g_claimed
    s.sumcheck(R.h_sq, true); s.words(R.h_sq.fin, 3); put_claimed_sum_base(s, R.h_sq);
    s.sumcheck(R.g_sq, true); s.words(R.g_sq.fin, 3); put_claimed_sum_base(s, R.g_sq);
    for (int i = 0; i < 4; i++) s.commitment(R.roots + 8 * i, n);
    const EvalRec* ev[7] = {&R.xc_mean, &R.xc_var, &R.g_prod_eval, &R.xc_triple, &R.gamma_triple, &R.h_sq_eval, &R.g_sq_eval};
    for (int i = 0; i < 7; i++) { put_eval_base(s, *ev[i]); put_claimed_sum_base(s, ev[i]->sc); }
}

// ---- ReLU op (prove.rs:237-340) ---------------------------------------------------------------------
struct ReluRec {
    u32 k = 0;
    size_t root = 0;
    bool have_chain = false;
    EvalRec chain, a_eval;
    ScRec product, boolean;
};
// z: pre-activation (n valid entries) on the device; chain_point: the previous proof's matmul challenge
// point (k words on the device) or null.
inline ReluRec prove_relu(zkb_ctx* c, TrState* tr, const u32* z, u32 n_valid, const u32* chain_point) {
    ReluRec R;
    R.k = log2_ceil_u(n_valid);
    const u32 k = R.k;
    const size_t n = size_t(1) << k;
    u32* a = (u32*)c->scratch(n * 4 + 16);
    u32* b = (u32*)c->scratch(n * 4 + 16);
    u32* omb = (u32*)c->scratch(n * 4 + 16);
    u32* zp = (u32*)c->scratch(n * 4 + 16);
    relu_prep_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(z, n_valid, (u32)n, a, b, omb);
    ZKB_LAUNCHED(c);
    pad_copy_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(z, n_valid, n, zp);
    ZKB_LAUNCHED(c);
    R.root = commit_small(c, a, (u32)n, nullptr, (u32)n, nullptr);
    const u32* root_dev = c->rec_dev + R.root;
    if (chain_point) {
        R.have_chain = true;
        R.chain = prove_mle_eval_base(c, tr, a, chain_point, k, "relu-chain", root_dev);
    }
    u32* r_point = (u32*)c->scratch((size_t)k * 4 + 16);
    {
        ScriptBuilder sb;
        sb.words_dev(root_dev, 8);
        sb.squeeze(r_point, k);
        sb.run(c, tr);
    }
    R.a_eval = prove_mle_eval_base(c, tr, a, r_point, k, "relu-eval", root_dev);
    Fp* eq = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)r_point, k, eq);
    ZKB_LAUNCHED(c);
    const u32* t1[3] = {(const u32*)eq, b, zp};
    R.product = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, t1, k);
    u32* r2 = (u32*)c->scratch((size_t)k * 4 + 16);
    { ScriptBuilder sb; sb.squeeze(r2, k); sb.run(c, tr); }
    Fp* eq2 = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)r2, k, eq2);
    ZKB_LAUNCHED(c);
    const u32* t2[3] = {(const u32*)eq2, b, omb};
    R.boolean = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, t2, k);
    return R;
}
// SerializedLayerProof::Relu (protocol.rs:655-666)
inline void put_relu(Ser& s, const ReluRec& R) {
    s.commitment(R.root, u64(1) << R.k);
    put_claimed_sum_base(s, R.a_eval.sc);                            // a_at_r = MLE of a at r = sum eq(r) a
    put_eval_base(s, R.a_eval);
    s.u8(R.have_chain ? 1 : 0); if (R.have_chain) put_eval_base(s, R.chain);
    s.u8(R.have_chain ? 1 : 0); if (R.have_chain) put_claimed_sum_base(s, R.chain.sc);
    s.sumcheck(R.product, true); s.words(R.product.fin, 3);
    s.sumcheck(R.boolean, true); s.words(R.boolean.fin, 3);
}

}  // namespace zkb

// ---- the op list object behind the C ABI -------------------------------------------------------------
struct zkb_oplist {
    enum Kind { LINEAR, RELU, LAYERNORM, GELU, ATTENTION, SAVE, ADD_SAVED, SET_INPUT, SET_INPUT_REQUANT, PASSTHROUGH, ATTENTION_ROWS };
    struct Op {
        Kind kind;
        std::string name, aux;
        zkb::u32 m = 0, n = 0;                 // linear
        zkb::u32* w = nullptr; zkb::u32* b = nullptr; zkb::u32 root[8] = {};
        zkb::u32* gamma = nullptr; zkb::u32* beta = nullptr;      // layernorm (d words each)
        const zkb::u32* table = nullptr; zkb::u32 n_table = 0;  // gelu
        zkb::u32* values = nullptr; zkb::u32 n_values = 0;        // set_input
        // trace (device, zero-padded to a power of two; allocated when the op is added)
        zkb::u32 in_len = 0, out_len = 0;
        zkb::u32* out = nullptr;               // activation after the op
        zkb::u32* aux0 = nullptr;              // relu: pre-activation; layernorm: xc; gelu: requantised input
        zkb::u32* aux1 = nullptr;              // layernorm: perturbed x
        zkb::u32 heads = 0, kv_heads = 0, seq = 0, d_head = 0;      // attention at seq_len >= 2, kv_heads != 0: gqa_attention (table = exp table; aux0 / aux1 = K / V when given by the caller)
        zkb::u32* scalars = nullptr;           // layernorm: {perturbation, mu, sum_sq, r}
        int save_of = -1;                      // add_saved: index of the matching save op
    };
    zkb_ctx* ctx = nullptr;
    std::vector<Op> ops;
    zkb::u32 in_len = 0;                       // model input length (set by the first call of prove / forward)
    zkb::u32* x = nullptr;                     // model input on the device
    zkb::u32 x_cap = 0;
    std::vector<void*> owned;                  // device allocations to free
    zkb::u32 cur_len = 0;                      // running activation length while ops are added
    std::vector<zkb::HashJob> hash_jobs;       // distinct (vector, length) pairs whose content digest a proof needs
    zkb::HashJob* hash_jobs_dev = nullptr;
    size_t hash_jobs_nops = 0;                 // number of ops the job list was built for
    size_t hash_base = 0;                      // record offset of the digests of the current proof
    bool len_known = false;
};
