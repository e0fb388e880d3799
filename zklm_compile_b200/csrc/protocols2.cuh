// RMSNorm, LogUp and the lookup-then-hadamard gates (see protocols.cuh for the conventions).
#pragma once
#include "protocols.cuh"

namespace zkb {

// ---- RMSNorm (rmsnorm.rs:512-667) ----------------------------------------------------------------
struct RmsNormRec {
    u32 k = 0;
    size_t scalars = 0;         // {delta, sum_sq} copied from the forward pass
    size_t roots = 0;           // x, gamma, g, h roots (4 x 8 words)
    ScRec var, g_prod, g_triple, h_sq, g_sq;
    EvalRec x_var, g_prod_eval, x_triple, gamma_triple, h_sq_eval, g_sq_eval;
    size_t gc_point = 0, sq_point = 0;
};
// x (the possibly perturbed input), gamma, y: d valid entries; x and y zero-padded to 2^k on device.
// fwd_scalars: device {delta, sum_sq of x} from rmsnorm_forward_kernel.
inline RmsNormRec prove_rmsnorm_ef(zkb_ctx* c, TrState* tr, const u32* x, const u32* gamma, const u32* y, u32 d, const u32* fwd_scalars) {
    RmsNormRec R;
    R.k = log2_ceil_u(d);
    const u32 k = R.k;
    const size_t n = size_t(1) << k;
    u32* g = (u32*)c->scratch(n * 4);
    u32* gamma_pad = (u32*)c->scratch(n * 4);
    R.scalars = c->rec_alloc(2);
    R.roots = c->rec_alloc(32);
    u32* sc_dev = c->rec_dev + R.scalars;
    pad_copy_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(gamma, d, n, gamma_pad);
    ZKB_LAUNCHED(c);
    rmsnorm_prep_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(x, gamma, d, (u32)n, g, sc_dev + 1);
    ZKB_LAUNCHED(c);
    ZKB_CUDA(cudaMemcpyAsync(sc_dev, fwd_scalars, 4, cudaMemcpyDeviceToDevice, c->stream));   // delta
    B3Multi bm{};
    const u32* vecs[4] = {x, gamma_pad, g, y};
    for (int i = 0; i < 4; i++) {
        bm.words[i] = vecs[i]; bm.n_words[i] = (u32)n; bm.root[i] = c->rec_dev + R.roots + 8 * i;
        bm.cvs[i] = (u32*)c->scratch((n * 4 + 7 + 1023) / 1024 * 32 + 64);
    }
    b3_commit_multi_kernel<<<4, 256, 0, c->stream>>>(b3_prefix("weights", 7), bm);
    ZKB_LAUNCHED(c);
    {
        ScriptBuilder sb;
        sb.str("rmsnorm-pert-v1");
        sb.words_dev(sc_dev, 1);                                  // delta as u32
        sb.words_dev(c->rec_dev + R.roots, 32);                   // four roots
        sb.words_dev(sc_dev + 1, 1);                              // sum_sq
        sb.run(c, tr);
    }
    const u32* root_x = c->rec_dev + R.roots, *root_gamma = root_x + 8, *root_g = root_x + 16, *root_h = root_x + 24;
    // step 1: sum x^2
    const u32* tv[3] = {x, x, nullptr};
    R.var = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_EF, tv, k);
    R.x_var = prove_mle_eval_ef_base(c, tr, x, (u32)n, (const Fe*)(c->rec_dev + R.var.chal), k, "rmsnorm-x-var", root_x);
    // step 2: g = gamma . x
    R.gc_point = c->rec_alloc(4 * (size_t)k);
    { ScriptBuilder sb; sb.squeeze(c->rec_dev + R.gc_point, 4 * k); sb.run(c, tr); }
    const Fe* gc = (const Fe*)(c->rec_dev + R.gc_point);
    Fe* eq = (Fe*)c->scratch(n * 16);
    Fe* g_ef = (Fe*)c->scratch(n * 16);
    Fe* gamma_ef = (Fe*)c->scratch(n * 16);
    Fe* x_ef = (Fe*)c->scratch(n * 16);
    {
        WidenEqArgs w{};
        w.src[0] = g; w.dst[0] = g_ef; w.len[0] = (u32)n; w.src[1] = gamma_pad; w.dst[1] = gamma_ef; w.len[1] = (u32)n;
        w.src[2] = x; w.dst[2] = x_ef; w.len[2] = (u32)n; w.nsrc = 3; w.point = gc; w.eq_out = eq; w.k = k;
        widen_eq_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(w);
        ZKB_LAUNCHED(c);
    }
    const u32* tgp[3] = {(const u32*)eq, (const u32*)g_ef, nullptr};
    R.g_prod = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_EF_FULL, tgp, k);          // eq and g_ef are reused below
    R.g_prod_eval = prove_mle_eval_ef_base(c, tr, g, (u32)n, (const Fe*)(c->rec_dev + R.g_prod.chal), k, "rmsnorm-g-prod", root_g);
    const u32* tgt[3] = {(const u32*)eq, (const u32*)gamma_ef, (const u32*)x_ef};
    ScOpts ogt;
    ogt.clobber[0] = ogt.clobber[1] = ogt.clobber[2] = true;
    R.g_triple = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE_EF_FULL, tgt, k, ogt);
    const Fe* s_gt = (const Fe*)(c->rec_dev + R.g_triple.chal);
    R.x_triple = prove_mle_eval_ef_base(c, tr, x, (u32)n, s_gt, k, "rmsnorm-x-triple", root_x);
    R.gamma_triple = prove_mle_eval_ef_base(c, tr, gamma_pad, (u32)n, s_gt, k, "rmsnorm-gamma-triple", root_gamma);
    // step 3: squared checks
    R.sq_point = c->rec_alloc(4 * (size_t)k);
    { ScriptBuilder sb; sb.squeeze(c->rec_dev + R.sq_point, 4 * k); sb.run(c, tr); }
    Fe* eq2 = eq;                         // the first eq table has been consumed
    Fe* h_ef = gamma_ef;                  // so have gamma_ef / x_ef
    {
        WidenEqArgs w{};
        w.src[0] = y; w.dst[0] = h_ef; w.len[0] = (u32)n; w.nsrc = 1;
        w.point = (const Fe*)(c->rec_dev + R.sq_point); w.eq_out = eq2; w.k = k;
        widen_eq_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(w);
        ZKB_LAUNCHED(c);
    }
    const u32* ths[3] = {(const u32*)eq2, (const u32*)h_ef, (const u32*)h_ef};
    R.h_sq = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE_EF_FULL, ths, k);             // eq2 is reused by the g^2 check
    R.h_sq_eval = prove_mle_eval_ef_base(c, tr, y, (u32)n, (const Fe*)(c->rec_dev + R.h_sq.chal), k, "rmsnorm-h-sq", root_h);
    const u32* tgs[3] = {(const u32*)eq2, (const u32*)g_ef, (const u32*)g_ef};
    R.g_sq = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE_EF_FULL, tgs, k);
    R.g_sq_eval = prove_mle_eval_ef_base(c, tr, g, (u32)n, (const Fe*)(c->rec_dev + R.g_sq.chal), k, "rmsnorm-g-sq", root_g);
    return R;
}
// RmsNormProofEF in serde field order (rmsnorm.rs:457-503)
inline void put_rmsnorm(Ser& s, const RmsNormRec& R, bool stripped) {
    const bool ch = !stripped;
    const u64 n = u64(1) << R.k;
    s.u32le(s.rec[R.scalars]);                                   // perturbation_delta (i32)
    s.sumcheck(R.var, ch); s.ef(R.var.fin); s.ef(R.var.fin + 4);
    s.u32le(s.rec[R.scalars + 1]);                               // sum_sq_value
    s.sumcheck(R.h_sq, ch); s.ef(R.h_sq.fin); s.ef(R.h_sq.fin + 4); s.ef(R.h_sq.fin + 8);
    s.claimed_sum_ef(R.h_sq);                                    // s_h
    s.sumcheck(R.g_sq, ch); s.ef(R.g_sq.fin); s.ef(R.g_sq.fin + 4); s.ef(R.g_sq.fin + 8);
    s.claimed_sum_ef(R.g_sq);                                    // s_g
    s.sumcheck(R.g_prod, ch); s.ef(R.g_prod.fin); s.ef(R.g_prod.fin + 4);
    s.sumcheck(R.g_triple, ch); s.ef(R.g_triple.fin); s.ef(R.g_triple.fin + 4); s.ef(R.g_triple.fin + 8);
    s.claimed_sum_ef(R.g_prod);                                  // t_g_claimed
    for (int i = 0; i < 4; i++) s.commitment(R.roots + 8 * i, n);
    const EvalRec* ev[6] = {&R.x_var, &R.g_prod_eval, &R.x_triple, &R.gamma_triple, &R.h_sq_eval, &R.g_sq_eval};
    for (int i = 0; i < 6; i++) { put_eval(s, *ev[i], ch); s.claimed_sum_ef(ev[i]->sc); }
}

// Base-field twin (rmsnorm.rs:96-246): same sequence with challenges in M31; the tables stay
// base-field vectors, so nothing is widened.
inline RmsNormRec prove_rmsnorm_base(zkb_ctx* c, TrState* tr, const u32* x, const u32* gamma, const u32* y, u32 d, const u32* fwd_scalars) {
    RmsNormRec R;
    R.k = log2_ceil_u(d);
    const u32 k = R.k;
    const size_t n = size_t(1) << k;
    u32* g = (u32*)c->scratch(n * 4);
    u32* gamma_pad = (u32*)c->scratch(n * 4);
    R.scalars = c->rec_alloc(2);
    R.roots = c->rec_alloc(32);
    u32* sc_dev = c->rec_dev + R.scalars;
    pad_copy_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(gamma, d, n, gamma_pad);
    ZKB_LAUNCHED(c);
    rmsnorm_prep_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(x, gamma, d, (u32)n, g, sc_dev + 1);
    ZKB_LAUNCHED(c);
    ZKB_CUDA(cudaMemcpyAsync(sc_dev, fwd_scalars, 4, cudaMemcpyDeviceToDevice, c->stream));
    B3Multi bm{};
    const u32* vecs[4] = {x, gamma_pad, g, y};
    for (int i = 0; i < 4; i++) {
        bm.words[i] = vecs[i]; bm.n_words[i] = (u32)n; bm.root[i] = c->rec_dev + R.roots + 8 * i;
        bm.cvs[i] = (u32*)c->scratch((n * 4 + 7 + 1023) / 1024 * 32 + 64);
    }
    b3_commit_multi_kernel<<<4, 256, 0, c->stream>>>(b3_prefix("weights", 7), bm);
    ZKB_LAUNCHED(c);
    {
        ScriptBuilder sb;
        sb.str("rmsnorm-pert-v1");
        sb.words_dev(sc_dev, 1);
        sb.words_dev(c->rec_dev + R.roots, 32);
        sb.words_dev(sc_dev + 1, 1);
        sb.run(c, tr);
    }
    const u32* root_x = c->rec_dev + R.roots, *root_gamma = root_x + 8, *root_g = root_x + 16, *root_h = root_x + 24;
    const u32* tv[3] = {x, x, nullptr};
    R.var = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tv, k);
    R.x_var = prove_mle_eval_base(c, tr, x, c->rec_dev + R.var.chal, k, "rmsnorm-x-var", root_x);
    R.gc_point = c->rec_alloc(k);
    { ScriptBuilder sb; sb.squeeze(c->rec_dev + R.gc_point, k); sb.run(c, tr); }
    Fp* eq = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)(c->rec_dev + R.gc_point), k, eq);
    ZKB_LAUNCHED(c);
    const u32* tgp[3] = {(const u32*)eq, g, nullptr};
    R.g_prod = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tgp, k);
    R.g_prod_eval = prove_mle_eval_base(c, tr, g, c->rec_dev + R.g_prod.chal, k, "rmsnorm-g-prod", root_g);
    const u32* tgt[3] = {(const u32*)eq, gamma_pad, x};
    R.g_triple = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, tgt, k);
    const u32* s_gt = c->rec_dev + R.g_triple.chal;
    R.x_triple = prove_mle_eval_base(c, tr, x, s_gt, k, "rmsnorm-x-triple", root_x);
    R.gamma_triple = prove_mle_eval_base(c, tr, gamma_pad, s_gt, k, "rmsnorm-gamma-triple", root_gamma);
    R.sq_point = c->rec_alloc(k);
    { ScriptBuilder sb; sb.squeeze(c->rec_dev + R.sq_point, k); sb.run(c, tr); }
    Fp* eq2 = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)(c->rec_dev + R.sq_point), k, eq2);
    ZKB_LAUNCHED(c);
    const u32* ths[3] = {(const u32*)eq2, y, y};
    R.h_sq = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, ths, k);
    R.h_sq_eval = prove_mle_eval_base(c, tr, y, c->rec_dev + R.h_sq.chal, k, "rmsnorm-h-sq", root_h);
    const u32* tgs[3] = {(const u32*)eq2, g, g};
    R.g_sq = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, tgs, k);
    R.g_sq_eval = prove_mle_eval_base(c, tr, g, c->rec_dev + R.g_sq.chal, k, "rmsnorm-g-sq", root_g);
    return R;
}
// RmsNormProof in serde field order (rmsnorm.rs:36-85)
inline void put_rmsnorm_base(Ser& s, const RmsNormRec& R) {
    const u64 n = u64(1) << R.k;
    s.u32le(s.rec[R.scalars]);
    s.sumcheck(R.var, true); s.words(R.var.fin, 2);
    s.u32le(s.rec[R.scalars + 1]);
    s.sumcheck(R.h_sq, true); s.words(R.h_sq.fin, 3); put_claimed_sum_base(s, R.h_sq);
    s.sumcheck(R.g_sq, true); s.words(R.g_sq.fin, 3); put_claimed_sum_base(s, R.g_sq);
    s.sumcheck(R.g_prod, true); s.words(R.g_prod.fin, 2);
    s.sumcheck(R.g_triple, true); s.words(R.g_triple.fin, 3);
    put_claimed_sum_base(s, R.g_prod);                           // t_g_claimed
    for (int i = 0; i < 4; i++) s.commitment(R.roots + 8 * i, n);
    const EvalRec* ev[6] = {&R.x_var, &R.g_prod_eval, &R.x_triple, &R.gamma_triple, &R.h_sq_eval, &R.g_sq_eval};
    for (int i = 0; i < 6; i++) { put_eval_base(s, *ev[i]); put_claimed_sum_base(s, ev[i]->sc); }
}

// ---- LogUp (lookup.rs:643-762) -------------------------------------------------------------------
struct LookupRec {
    u32 n = 0, max_nv = 0;
    size_t dyn = 0;             // {n_active, num_vars, n}
    size_t chal = 0;            // beta, alpha
    size_t root_table = 0, root_mult = 0, digest = 0;
    ScRec sc;
};
// inputs / outputs: n lookups on device; table_out: n_table output column on device.
inline LookupRec prove_lookup_ef(zkb_ctx* c, TrState* tr, const u32* table_out, u32 n_table, const u32* inputs, const u32* outputs, u32 n) {
    LookupRec R;
    R.n = n;
    const u32 max_active = n < n_table ? n : n_table;
    R.max_nv = log2_ceil_u((size_t)n + max_active);
    const size_t cap = size_t(1) << R.max_nv;
    R.chal = c->rec_alloc(8);
    R.dyn = c->rec_alloc(4);
    u32* chal = c->rec_dev + R.chal;
    u32* dyn = c->rec_dev + R.dyn;
    {
        ScriptBuilder sb;
        unsigned char zero[32] = {0};
        sb.bytes(zero, 32);                                      // table.commitment.root placeholder
        sb.word(n);
        sb.pairs_dev(inputs, outputs, n);
        sb.squeeze(chal, 8);                                     // beta then alpha
        sb.run(c, tr);
    }
    u32* mult = (u32*)c->scratch((size_t)n_table * 4);
    u32* act_idx = (u32*)c->scratch((size_t)max_active * 4 + 16);
    u32* act_mult = (u32*)c->scratch((size_t)max_active * 4 + 16);
    u32* act_entry = (u32*)c->scratch((size_t)max_active * 4 + 16);
    ZKB_CUDA(cudaMemsetAsync(mult, 0, (size_t)n_table * 4, c->stream));
    logup_hist_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(inputs, n, n_table, mult);
    ZKB_LAUNCHED(c);
    logup_compact_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(mult, table_out, n_table, n, act_idx, act_mult, act_entry, dyn);
    ZKB_LAUNCHED(c);
    Fe* h = (Fe*)c->scratch(cap * 16);
    logup_h_kernel<Fe><<<grid_for(c, cap / LOGUP_BATCH + 1), 256, 0, c->stream>>>(inputs, outputs, table_out, n_table, act_idx, act_mult, dyn,
                                                                                   (const Fe*)chal, h, (u32)cap, c->status);
    ZKB_LAUNCHED(c);
    R.root_table = commit_small(c, act_entry, 0, dyn, max_active, tr);
    R.root_mult = commit_small(c, act_mult, 0, dyn, max_active, tr);
    const u32* tabs[3] = {(const u32*)h, nullptr, nullptr};
    ScOpts o;
    o.clobber[0] = true;
    o.dyn_nv = dyn + 1;
    o.dyn_off = (long)R.dyn;
    o.check_zero_sum = true;
    R.sc = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_ONES_EF_FULL, tabs, R.max_nv, o);
    // external-data digest (not absorbed; lookup.rs:609-621)
    u32* cat = (u32*)c->scratch(((size_t)2 * n + 2) * 4);
    logup_digest_concat_kernel<<<grid_for(c, 2 * (size_t)n + 2), 256, 0, c->stream>>>(inputs, outputs, n, cat);
    ZKB_LAUNCHED(c);
    R.digest = c->rec_alloc(8);
    {
        unsigned char pre[31];
        memcpy(pre, "lookup-external-data-v1", 23);
        u64 n64 = n;
        memcpy(pre + 23, &n64, 8);
        size_t max_chunks = ((size_t)(2 * n + 2) * 4 + 31 + 1023) / 1024 + 1;
        u32* cvs = (u32*)c->scratch(max_chunks * 32);
        b3_commit_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(b3_prefix(pre, 31), cat, 2 * n + 2, nullptr, cvs, c->rec_dev + R.digest, nullptr);
        ZKB_LAUNCHED(c);
    }
    return R;
}
// LookupProofEF (lookup.rs:89-115) with inputs/outputs stripped as the layer prover does
// (qwen.rs:895-900) when strip_io is set; `in`/`out` host copies are needed otherwise.
inline void put_lookup(Ser& s, const LookupRec& R, bool stripped, const u32* in_host, const u32* out_host) {
    const u32 n_active = s.rec[R.dyn], nv = s.rec[R.dyn + 1];
    s.commitment(R.root_table, n_active);
    s.commitment(R.root_mult, n_active);
    s.sumcheck(R.sc, !stripped, nv);
    s.ef(R.sc.fin);                          // h_at_s (the ONES tail writes g(s) to slot 0)
    s.u8(0); s.u8(0);                        // alpha, beta: None
    if (in_host) { s.u64le(R.n); for (u32 i = 0; i < R.n; i++) s.u32le(in_host[i]); s.u64le(R.n); for (u32 i = 0; i < R.n; i++) s.u32le(out_host[i]); }
    else { s.u64le(0); s.u64le(0); }
    s.u64le(0);                              // multiplicities: empty
    s.root(R.digest);
}

// Base-field twin (lookup.rs:432-604): challenges in M31, active subtable committed as
// inp + beta * out, all-ones product sumcheck over base-field h.
inline LookupRec prove_lookup_base(zkb_ctx* c, TrState* tr, const u32* table_out, u32 n_table, const u32* inputs, const u32* outputs, u32 n) {
    LookupRec R;
    R.n = n;
    const u32 max_active = n < n_table ? n : n_table;
    R.max_nv = log2_ceil_u((size_t)n + max_active);
    const size_t cap = size_t(1) << R.max_nv;
    R.chal = c->rec_alloc(2);
    R.dyn = c->rec_alloc(4);
    u32* chal = c->rec_dev + R.chal;
    u32* dyn = c->rec_dev + R.dyn;
    {
        ScriptBuilder sb;
        unsigned char zero[32] = {0};
        sb.bytes(zero, 32);
        sb.word(n);
        sb.pairs_dev(inputs, outputs, n);
        sb.squeeze(chal, 2);                                     // beta then alpha
        sb.run(c, tr);
    }
    u32* mult = (u32*)c->scratch((size_t)n_table * 4);
    u32* act_idx = (u32*)c->scratch((size_t)max_active * 4 + 16);
    u32* act_mult = (u32*)c->scratch((size_t)max_active * 4 + 16);
    u32* act_entry = (u32*)c->scratch((size_t)max_active * 4 + 16);
    u32* act_enc = (u32*)c->scratch((size_t)max_active * 4 + 16);
    ZKB_CUDA(cudaMemsetAsync(mult, 0, (size_t)n_table * 4, c->stream));
    logup_hist_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(inputs, n, n_table, mult);
    ZKB_LAUNCHED(c);
    logup_compact_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(mult, table_out, n_table, n, act_idx, act_mult, act_entry, dyn);
    ZKB_LAUNCHED(c);
    logup_encode_active_kernel<<<grid_for(c, max_active), 256, 0, c->stream>>>(act_idx, dyn, table_out, n_table, chal, act_enc);
    ZKB_LAUNCHED(c);
    Fp* h = (Fp*)c->scratch(cap * 4 + 16);
    logup_h_kernel<Fp><<<grid_for(c, cap / LOGUP_BATCH + 1), 256, 0, c->stream>>>(inputs, outputs, table_out, n_table, act_idx, act_mult, dyn,
                                                                                   (const Fp*)chal, h, (u32)cap, c->status);
    ZKB_LAUNCHED(c);
    R.root_table = commit_small(c, act_enc, 0, dyn, max_active, tr);
    R.root_mult = commit_small(c, act_mult, 0, dyn, max_active, tr);
    const u32* tabs[3] = {(const u32*)h, nullptr, nullptr};
    ScOpts o;
    o.dyn_nv = dyn + 1;
    o.dyn_off = (long)R.dyn;
    o.check_zero_sum = true;
    R.sc = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_ONES, tabs, R.max_nv, o);
    u32* cat = (u32*)c->scratch(((size_t)2 * n + 2) * 4);
    logup_digest_concat_kernel<<<grid_for(c, 2 * (size_t)n + 2), 256, 0, c->stream>>>(inputs, outputs, n, cat);
    ZKB_LAUNCHED(c);
    R.digest = c->rec_alloc(8);
    {
        unsigned char pre[31];
        memcpy(pre, "lookup-external-data-v1", 23);
        u64 n64 = n;
        memcpy(pre + 23, &n64, 8);
        size_t max_chunks = ((size_t)(2 * n + 2) * 4 + 31 + 1023) / 1024 + 1;
        u32* cvs = (u32*)c->scratch(max_chunks * 32);
        b3_commit_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(b3_prefix(pre, 31), cat, 2 * n + 2, nullptr, cvs, c->rec_dev + R.digest, nullptr);
        ZKB_LAUNCHED(c);
    }
    return R;
}
// LookupProof (lookup.rs:39-85)
inline void put_lookup_base(Ser& s, const LookupRec& R, const u32* in_host, const u32* out_host) {
    const u32 n_active = s.rec[R.dyn], nv = s.rec[R.dyn + 1];
    s.commitment(R.root_table, n_active);
    s.commitment(R.root_mult, n_active);
    s.sumcheck(R.sc, true, nv);
    s.u32le(1);                              // ones_at_s
    s.words(R.sc.fin, 1);                    // h_at_s
    s.u32le(s.rec[R.chal + 1]);              // alpha
    s.u32le(s.rec[R.chal]);                  // beta
    s.u64le(R.n); for (u32 i = 0; i < R.n; i++) s.u32le(in_host[i]);
    s.u64le(R.n); for (u32 i = 0; i < R.n; i++) s.u32le(out_host[i]);
    s.u64le(0);                              // multiplicities: empty
    s.root(R.digest);
}

// ---- lookup, squeeze the hadamard point, hadamard (sigmoid_gate.rs:90-114, swiglu.rs:99-118) ------
struct GateRec { LookupRec lk; HadamardRec had; size_t point = 0; };
inline GateRec prove_gate_ef(zkb_ctx* c, TrState* tr, const u32* table_out, u32 n_table, const u32* lk_in, const u32* lk_out,
                             const u32* had_a, const u32* had_b, const u32* out, u32 len) {
    GateRec R;
    R.lk = prove_lookup_ef(c, tr, table_out, n_table, lk_in, lk_out, len);
    u32 k = log2_ceil_u(len);
    R.point = c->rec_alloc(4 * (size_t)k);
    { ScriptBuilder sb; sb.squeeze(c->rec_dev + R.point, 4 * k); sb.run(c, tr); }
    R.had = prove_hadamard_ef(c, tr, had_a, had_b, out, len, (const Fe*)(c->rec_dev + R.point), k);
    return R;
}
inline void put_gate(Ser& s, const GateRec& R, bool stripped) {
    put_lookup(s, R.lk, stripped, nullptr, nullptr);
    put_hadamard(s, R.had, stripped);
}

}  // namespace zkb
