// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Matmul sub-protocol (y = W x), restating rust/zk_ml_prover/src/proving/matmul.rs for the
// default build (no `pcs` feature: weights are bound by blake3 + an MLE-eval sumcheck), plus
// the forward matvec of rust/zk_ml_prover/src/transformer/mod.rs:140-163.
#pragma once
#include "basefold.hpp"

namespace zko {

// Products of canonical values are below 2^62; folding once (2^31 == 1 mod p) leaves a term below
// 2^32, so a 64-bit accumulator takes 2^31 of them before it has to be reduced.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define ZKO_CLONES __attribute__((target_clones("avx2", "default")))
#else
#define ZKO_CLONES
#endif
ZKO_CLONES static uint64_t dot_fold(const uint32_t* w, const uint32_t* x, size_t n) {
    uint64_t acc = 0;
    for (size_t j = 0; j < n; j++) {
        uint64_t p = uint64_t(w[j]) * x[j];
        acc += (p & P31) + (p >> 31);
    }
    return acc;
}
ZKO_CLONES static void macc_row(uint64_t* a, const uint32_t* w, size_t n, uint32_t e) {
    for (size_t j = 0; j < n; j++) {
        uint64_t p = uint64_t(e) * w[j];
        a[j] += (p & P31) + (p >> 31);
    }
}
ZKO_CLONES static void macc_row4(uint64_t* a0, uint64_t* a1, uint64_t* a2, uint64_t* a3, const uint32_t* w, size_t n, uint32_t e0,
                                 uint32_t e1, uint32_t e2, uint32_t e3) {
    for (size_t j = 0; j < n; j++) {
        const uint64_t x = w[j];
        uint64_t p0 = e0 * x, p1 = e1 * x, p2 = e2 * x, p3 = e3 * x;
        a0[j] += (p0 & P31) + (p0 >> 31);
        a1[j] += (p1 & P31) + (p1 >> 31);
        a2[j] += (p2 & P31) + (p2 >> 31);
        a3[j] += (p3 & P31) + (p3 >> 31);
    }
}
static_assert(sizeof(F) == 4, "F is a bare u32: vectors of F are read as u32 arrays");

// transformer/mod.rs:140-163 — y[i] = sum_j W[i,j] x[j] (+ bias), exact mod p.
inline VF matmul_forward(const VF& w, const VF& x, size_t m, size_t n, const VF* bias = nullptr) {
    VF y(m);
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(w.data());
    const uint32_t* xp = reinterpret_cast<const uint32_t*>(x.data());
    par_rows(m, [&](size_t lo, size_t hi, int) {
        for (size_t i = lo; i < hi; i++) {
            F v = F(reduce64(dot_fold(wp + i * n, xp, n)));
            if (bias) v += (*bias)[i];
            y[i] = v;
        }
    });
    return y;
}

// matmul.rs:76-128 — w_partial[j] = sum_i eq_r[i] W[i,j], zero-padded to n_pad; per-worker partial
// vectors merged at the end, as the reference does.
inline VF fold_eq_matvec(const VF& w, size_t m, size_t n, size_t n_pad, const VF& r_point) {
    size_t m_pad = size_t(1) << r_point.size();
    VF eq = eq_evals(r_point);
    size_t rows = m < m_pad ? m : m_pad;
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(w.data());
    const int T = matrix_threads() > 1 ? matrix_threads() : 1;
    std::vector<std::vector<uint64_t>> part(T);
    par_rows(rows, [&](size_t lo, size_t hi, int t) {
        part[t].assign(n, 0);
        for (size_t i = lo; i < hi; i++) macc_row(part[t].data(), wp + i * n, n, eq[i].v);
    });
    VF out(n_pad, F::zero());
    for (auto& pt : part)
        for (size_t j = 0; j < pt.size(); j++) out[j] += F(reduce64(pt[j]));
    return out;
}
// matmul.rs:743-835 — EF weights eq_r[i], base-field W; four independent base accumulators.
inline VEF fold_eq_matvec_ef(const VF& w, size_t m, size_t n, size_t n_pad, const VEF& r_point) {
    size_t m_pad = size_t(1) << r_point.size();
    VEF eq = eq_evals_ef(r_point);
    size_t rows = m < m_pad ? m : m_pad;
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(w.data());
    const int T = matrix_threads() > 1 ? matrix_threads() : 1;
    std::vector<std::vector<uint64_t>> part(T);
    par_rows(rows, [&](size_t lo, size_t hi, int t) {
        part[t].assign(4 * n, 0);
        uint64_t* a = part[t].data();
        for (size_t i = lo; i < hi; i++) {
            auto e = eq[i].arr();
            macc_row4(a, a + n, a + 2 * n, a + 3 * n, wp + i * n, n, e[0], e[1], e[2], e[3]);
        }
    });
    VEF out(n_pad, EF::zero());
    for (auto& pt : part) {
        if (pt.empty()) continue;
        for (size_t j = 0; j < n; j++)
            out[j] += EF(C(F(reduce64(pt[j])), F(reduce64(pt[n + j]))), C(F(reduce64(pt[2 * n + j])), F(reduce64(pt[3 * n + j]))));
    }
    return out;
}

// matmul.rs:24-31
struct MatmulProof {
    SumcheckProof sumcheck_proof;
    uint32_t w_at_rs = 0, x_at_s = 0;
    std::vector<uint32_t> r_point, s_point;
};
// matmul.rs:458-474
struct SuccinctMatmulProof {
    MatmulProof matmul_proof;
    MleEvalProof w_eval_proof;
    uint32_t w_claimed_value = 0;
    WeightCommitment w_partial_commitment;
    bool bound = false;
    // basefold_proof: Option = None in the default build
};

// matmul.rs:134-180
inline MatmulProof prove_matmul(const VF& w, const VF& x, const VF& y, size_t m, size_t n, Transcript& tr, VF* w_partial_out) {
    size_t log_m = log2_ceil(m), log_n = log2_ceil(n), m_pad = size_t(1) << log_m, n_pad = size_t(1) << log_n;
    VF y_pad = padded(y, m_pad), x_pad = padded(x, n_pad);
    tr.absorb_many(y_pad);
    VF r = tr.squeeze_many(log_m);
    VF w_partial = fold_eq_matvec(w, m, n, n_pad, r);
    Prod sc = prove_product(w_partial, x_pad, log_n, tr);
    MatmulProof p;
    p.sumcheck_proof = sc.proof;
    p.w_at_rs = sc.f_at_s.v; p.x_at_s = sc.g_at_s.v;
    for (F v : r) p.r_point.push_back(v.v);
    p.s_point = sc.proof.challenges;
    if (w_partial_out) *w_partial_out = w_partial;
    return p;
}
// matmul.rs:482-511 with bind_weights' default branch (:346-355)
inline SuccinctMatmulProof prove_matmul_succinct(const VF& w, const VF& x, const VF& y, size_t m, size_t n, Transcript& tr) {
    VF w_partial;
    SuccinctMatmulProof p;
    p.matmul_proof = prove_matmul(w, x, y, m, n, tr, &w_partial);
    VF s;
    for (uint32_t v : p.matmul_proof.s_point) s.push_back(F(v));
    p.w_partial_commitment = commit_weights_fast(w_partial);
    tr.absorb_bytes(p.w_partial_commitment.root);
    p.w_eval_proof = prove_mle_eval_no_merkle(w_partial, s, tr);
    return p;
}
struct MatmulVerify { bool valid = false; VF x_claim_point; F x_claim_value; };
// matmul.rs:604-707 (default branch)
inline MatmulVerify verify_matmul_succinct(const SuccinctMatmulProof& p, const VF& y, size_t m, size_t n, Transcript& tr) {
    MatmulVerify out;
    size_t log_m = log2_ceil(m), m_pad = size_t(1) << log_m;
    (void)n;
    VF y_pad = padded(y, m_pad);
    tr.absorb_many(y_pad);
    VF r = tr.squeeze_many(log_m);
    std::vector<uint32_t> r_raw;
    for (F v : r) r_raw.push_back(v.v);
    if (r_raw != p.matmul_proof.r_point) return out;
    F claim = mle_evaluate(y_pad, r);
    F w_at_rs(p.matmul_proof.w_at_rs), x_at_s(p.matmul_proof.x_at_s);
    if (!verify_product_with_challenges(claim, p.matmul_proof.sumcheck_proof, w_at_rs, x_at_s, tr)) return out;
    VF s;
    for (uint32_t v : p.matmul_proof.s_point) s.push_back(F(v));
    tr.absorb_bytes(p.w_partial_commitment.root);
    if (!verify_mle_eval(w_at_rs, s, p.w_eval_proof, tr)) return out;
    out.valid = true; out.x_claim_point = s; out.x_claim_value = x_at_s;
    return out;
}

// matmul.rs:717-726
struct MatmulProofEF {
    SumcheckProofEF sumcheck_proof;
    EFElement w_at_rs{}, x_at_s{};
    std::vector<EFElement> r_point, s_point;
};
// matmul.rs:947-960
struct SuccinctMatmulProofEF {
    MatmulProofEF matmul_proof;
    MleEvalProofEF w_eval_proof;
    EFElement w_claimed_value{};
    WeightCommitment w_partial_commitment;
    bool bound = false;
    bool has_basefold = false;                 // basefold_proof: Option<BasefoldOpeningProof> (matmul.rs:958-959)
    BasefoldOpeningProof basefold_proof;
};

// The reference picks its weight binding at compile time (cargo features, matmul.rs:360-453):
//   BIND_BLAKE3    default build: blake3 of w_partial, no Basefold            matmul.rs:441-443
//   BIND_PCS       feature pcs: Basefold of w_partial (4 n_pad base words)     matmul.rs:422-438
//   BIND_PCS_FULL  feature pcs-full: Basefold of the row-padded matrix W       matmul.rs:372-403
// and its Merkle node hash by target architecture (pcs.rs:87-135).  The oracle keeps both as
// a process-wide setting, the analogue of "which binary was built".
enum BindMode : int { BIND_BLAKE3 = 0, BIND_PCS = 1, BIND_PCS_FULL = 2 };
struct Features { int bind_mode = BIND_BLAKE3; int node_kind = NODE_BLAKE3; };
inline Features& features() { static Features f; return f; }

// matmul.rs:838-885
inline MatmulProofEF prove_matmul_ef(const VF& w, const VF& x, const VF& y, size_t m, size_t n, Transcript& tr, VEF* w_partial_out) {
    size_t log_m = log2_ceil(m), log_n = log2_ceil(n), m_pad = size_t(1) << log_m, n_pad = size_t(1) << log_n;
    VF y_pad = padded(y, m_pad), x_pad = padded(x, n_pad);
    tr.absorb_many(y_pad);
    VEF r = tr.squeeze_ef_many(log_m);
    VEF w_partial = fold_eq_matvec_ef(w, m, n, n_pad, r);
    ProdEF sc = prove_product_ef_mixed(w_partial, x_pad, log_n, tr);
    MatmulProofEF p;
    p.sumcheck_proof = sc.proof;
    p.w_at_rs = sc.f_at_s.arr(); p.x_at_s = sc.g_at_s.arr();
    for (EF v : r) p.r_point.push_back(v.arr());
    p.s_point = sc.proof.challenges;
    if (w_partial_out) *w_partial_out = w_partial;
    return p;
}
// matmul.rs:963-997 with bind_weights_ef (matmul.rs:360-453).  In the PCS modes the evaluation
// point is squeezed from the transcript (one base-field value per variable) and the 16-byte
// Merkle root is stored zero-padded in the 32-byte commitment.
inline SuccinctMatmulProofEF prove_matmul_succinct_ef(const VF& w, const VF& x, const VF& y, size_t m, size_t n, Transcript& tr) {
    VEF w_partial;
    SuccinctMatmulProofEF p;
    p.matmul_proof = prove_matmul_ef(w, x, y, m, n, tr, &w_partial);
    VF base;
    for (EF v : w_partial) { auto a = v.arr(); for (int k = 0; k < 4; k++) base.push_back(F(a[k])); }
    VEF s;
    for (auto& e : p.matmul_proof.s_point) s.push_back(ef_of(e));
    const int mode = features().bind_mode;
    if (mode == BIND_BLAKE3) {
        p.w_partial_commitment = commit_weights_fast(base);
    } else {
        VF coeffs;
        size_t num_coeffs;
        if (mode == BIND_PCS_FULL) {
            size_t m_pad = size_t(1) << log2_ceil(m), n_pad = size_t(1) << log2_ceil(n);
            coeffs.assign(m_pad * n_pad, F::zero());
            for (size_t i = 0; i < m; i++) for (size_t j = 0; j < n; j++) coeffs[i * n_pad + j] = w[i * n + j];
            num_coeffs = w.size();       // commit_and_prove_vec records the caller's count (matmul.rs:392)
        } else {
            coeffs = base;
            num_coeffs = base.size();
        }
        VF bf_point = tr.squeeze_many(log2_ceil(coeffs.size()));
        auto r = basefold_commit_and_prove(coeffs, bf_point, tr, features().node_kind);
        memcpy(p.w_partial_commitment.root.data(), r.first.root.data(), 16);
        p.w_partial_commitment.num_weights = num_coeffs;
        p.w_partial_commitment.log_height = r.first.log_n;
        p.w_partial_commitment.kind = 0;
        p.has_basefold = true;
        p.basefold_proof = std::move(r.second);
    }
    tr.absorb_bytes(p.w_partial_commitment.root);
    p.w_eval_proof = prove_mle_eval_ef_with_claim_no_merkle(w_partial, s, tr);
    return p;
}
struct MatmulVerifyEF { bool valid = false; VEF x_claim_point; EF x_claim_value; };
// matmul.rs:1000-1117 (Basefold branch :1061-1093, default branch :1094-1104)
inline MatmulVerifyEF verify_matmul_succinct_ef(const SuccinctMatmulProofEF& p, const VF& y, size_t m, size_t n, Transcript& tr) {
    MatmulVerifyEF out;
    size_t log_m = log2_ceil(m), m_pad = size_t(1) << log_m;
    (void)n;
    VF y_pad = padded(y, m_pad);
    tr.absorb_many(y_pad);
    VEF r = tr.squeeze_ef_many(log_m);
    if (!p.matmul_proof.r_point.empty()) {
        std::vector<EFElement> rr;
        for (EF v : r) rr.push_back(v.arr());
        if (rr != p.matmul_proof.r_point) return out;
    }
    EF claim = mle_evaluate_ef(y_pad, r);
    EF w_at_rs = ef_of(p.matmul_proof.w_at_rs), x_at_s = ef_of(p.matmul_proof.x_at_s);
    VEF derived;
    if (!verify_product_ef_with_challenges(claim, p.matmul_proof.sumcheck_proof, w_at_rs, x_at_s, tr, &derived)) return out;
    VEF s;
    if (p.matmul_proof.s_point.empty()) s = derived;
    else for (auto& e : p.matmul_proof.s_point) s.push_back(ef_of(e));
    if (p.has_basefold) {
        BasefoldCommitment c;
        memcpy(c.root.data(), p.w_partial_commitment.root.data(), 16);
        c.num_coeffs = p.w_partial_commitment.num_weights;
        c.log_n = p.w_partial_commitment.log_height;
        if (c.log_n > 40) return out;
        VF bf_point = tr.squeeze_many(c.log_n);
        tr.absorb_bytes(c.root);
        if (!basefold_verify_opening(c, F(p.basefold_proof.final_value), bf_point, p.basefold_proof, tr, features().node_kind)) return out;
    }
    tr.absorb_bytes(p.w_partial_commitment.root);
    if (!verify_mle_eval_ef(w_at_rs, s, p.w_eval_proof, tr)) return out;
    out.valid = true; out.x_claim_point = s; out.x_claim_value = x_at_s;
    return out;
}

}  // namespace zko
