// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Extension-field sub-protocols of a Qwen-style layer, restating
//   rust/zk_ml_prover/src/proving/elementwise.rs:429-642  (hadamard / add, EF)
//   rust/zk_ml_prover/src/proving/rmsnorm.rs:457-900       (RMSNorm, EF)
//   rust/zk_ml_prover/src/proving/lookup.rs:322-411, 609-762, 940-976 (LogUp, EF)
//   rust/zk_ml_prover/src/proving/sigmoid_gate.rs:90-114, swiglu.rs:99-118
#pragma once
#include "commit.hpp"
#include "matmul.hpp"
#include <stdexcept>

namespace zko {

// ------------------------------------------------------------------ hadamard (elementwise.rs:415-480)
struct HadamardProofEF {
    SumcheckProofEF product_sumcheck;
    EFElement fin_eq{}, fin_a{}, fin_b{};
    EFElement c_eval{};
    MleEvalProofEF c_eval_proof;
    WeightCommitment c_commitment;
};
inline HadamardProofEF prove_hadamard_ef(const VF& a, const VF& b, const VF& c, const VEF& point, Transcript& tr) {
    size_t log_n = point.size(), n_pad = size_t(1) << log_n;
    VF a_pad = padded(a, n_pad), b_pad = padded(b, n_pad), c_pad = padded(c, n_pad);
    HadamardProofEF p;
    p.c_commitment = commit_weights_fast(c_pad);
    tr.absorb_bytes(p.c_commitment.root);
    VEF eq = eq_evals_ef(point);
    TripEF t = prove_triple_ef_full(eq, widen(a_pad), widen(b_pad), log_n, tr);
    p.product_sumcheck = t.proof;
    p.fin_eq = t.f_at_s.arr(); p.fin_a = t.g_at_s.arr(); p.fin_b = t.h_at_s.arr();
    p.c_eval = mle_evaluate_ef(c_pad, point).arr();
    p.c_eval_proof = prove_mle_eval_ef_base_bound(c_pad, point, "hadamard-c-eval-ef", p.c_commitment, tr);
    return p;
}
// elementwise.rs:483-523
inline bool verify_hadamard_ef(const HadamardProofEF& p, const VEF& point, Transcript& tr) {
    tr.absorb_bytes(p.c_commitment.root);
    EF c_eval = ef_of(p.c_eval);
    VEF s;
    if (!verify_triple_ef_with_challenges(c_eval, p.product_sumcheck, ef_of(p.fin_eq), ef_of(p.fin_a), ef_of(p.fin_b), tr, &s)) return false;
    if (compute_eq_at_point_ef(point, s) != ef_of(p.fin_eq)) return false;
    return verify_mle_eval_ef_bound(p.c_commitment, c_eval, point, p.c_eval_proof, "hadamard-c-eval-ef", tr);
}

// ------------------------------------------------------------------ add (elementwise.rs:527-595)
struct AddProofEF {
    SumcheckProofEF a_sumcheck;
    EFElement a_fin_eq{}, a_fin{};
    SumcheckProofEF b_sumcheck;
    EFElement b_fin_eq{}, b_fin{};
    EFElement c_eval{};
    MleEvalProofEF c_eval_proof;
    WeightCommitment c_commitment;
};
inline AddProofEF prove_add_ef(const VF& a, const VF& b, const VF& c, const VEF& point, Transcript& tr) {
    size_t log_n = point.size(), n_pad = size_t(1) << log_n;
    VF a_pad = padded(a, n_pad), b_pad = padded(b, n_pad), c_pad = padded(c, n_pad);
    AddProofEF p;
    p.c_commitment = commit_weights_fast(c_pad);
    tr.absorb_bytes(p.c_commitment.root);
    VEF eq = eq_evals_ef(point);
    ProdEF ra = prove_product_ef_full(eq, widen(a_pad), log_n, tr);
    ProdEF rb = prove_product_ef_full(eq, widen(b_pad), log_n, tr);
    p.a_sumcheck = ra.proof; p.a_fin_eq = ra.f_at_s.arr(); p.a_fin = ra.g_at_s.arr();
    p.b_sumcheck = rb.proof; p.b_fin_eq = rb.f_at_s.arr(); p.b_fin = rb.g_at_s.arr();
    p.c_eval = mle_evaluate_ef(c_pad, point).arr();
    p.c_eval_proof = prove_mle_eval_ef_base_bound(c_pad, point, "add-c-eval-ef", p.c_commitment, tr);
    return p;
}
// elementwise.rs:598-642
inline bool verify_add_ef(const AddProofEF& p, const VEF& point, Transcript& tr) {
    tr.absorb_bytes(p.c_commitment.root);
    if (p.a_sumcheck.round_polys.empty() || p.a_sumcheck.round_polys[0].size() < 2 || p.b_sumcheck.round_polys.empty() ||
        p.b_sumcheck.round_polys[0].size() < 2) return false;          // the reference indexes out of bounds and panics
    EF a_eval = ef_of(p.a_sumcheck.round_polys[0][0]) + ef_of(p.a_sumcheck.round_polys[0][1]);
    VEF sa, sb;
    if (!verify_product_ef_with_challenges(a_eval, p.a_sumcheck, ef_of(p.a_fin_eq), ef_of(p.a_fin), tr, &sa)) return false;
    if (compute_eq_at_point_ef(point, sa) != ef_of(p.a_fin_eq)) return false;
    EF b_eval = ef_of(p.b_sumcheck.round_polys[0][0]) + ef_of(p.b_sumcheck.round_polys[0][1]);
    if (!verify_product_ef_with_challenges(b_eval, p.b_sumcheck, ef_of(p.b_fin_eq), ef_of(p.b_fin), tr, &sb)) return false;
    if (compute_eq_at_point_ef(point, sb) != ef_of(p.b_fin_eq)) return false;
    EF c_eval = ef_of(p.c_eval);
    if (a_eval + b_eval != c_eval) return false;
    return verify_mle_eval_ef_bound(p.c_commitment, c_eval, point, p.c_eval_proof, "add-c-eval-ef", tr);
}

// ------------------------------------------------------------------ RMSNorm (rmsnorm.rs:457-667)
struct RmsNormProofEF {
    int32_t perturbation_delta = 0;
    SumcheckProofEF var_proof;
    EFElement var_fin_a{}, var_fin_b{};
    uint32_t sum_sq_value = 0;
    SumcheckProofEF h_sq_proof;
    EFElement h_sq_fin[3]{};
    EFElement s_h{};
    SumcheckProofEF g_sq_proof;
    EFElement g_sq_fin[3]{};
    EFElement s_g{};
    SumcheckProofEF g_prod_proof;
    EFElement g_prod_fin[2]{};
    SumcheckProofEF g_triple_proof;
    EFElement g_triple_fin[3]{};
    EFElement t_g_claimed{};
    WeightCommitment x_commitment, gamma_commitment, g_commitment, h_commitment;
    MleEvalProofEF x_var_eval_proof;      EFElement x_at_var_s{};
    MleEvalProofEF g_prod_eval_proof;     EFElement g_at_prod_s{};
    MleEvalProofEF x_triple_eval_proof;   EFElement x_at_triple_s{};
    MleEvalProofEF gamma_triple_eval_proof; EFElement gamma_at_triple_s{};
    MleEvalProofEF h_sq_eval_proof;       EFElement h_at_sq_s{};
    MleEvalProofEF g_sq_eval_proof;       EFElement g_at_gsq_s{};
};
inline VEF points_of(const std::vector<EFElement>& c) { VEF o; for (auto& e : c) o.push_back(ef_of(e)); return o; }

inline RmsNormProofEF prove_rmsnorm_ef(const VF& x, const VF& gamma, const VF& y, int32_t delta, Transcript& tr) {
    size_t d = x.size(), log_n = log2_ceil(d), n_pad = size_t(1) << log_n;
    VF x_pad = padded(x, n_pad), gamma_pad = padded(gamma, n_pad), h_pad = padded(y, n_pad);
    VF g_pad(n_pad, F::zero());
    for (size_t i = 0; i < d; i++) g_pad[i] = gamma_pad[i] * x_pad[i];
    F sum_sq;
    for (F v : x_pad) sum_sq += v * v;
    RmsNormProofEF p;
    p.perturbation_delta = delta;
    p.sum_sq_value = sum_sq.v;
    p.x_commitment = commit_weights_fast(x_pad);
    p.gamma_commitment = commit_weights_fast(gamma_pad);
    p.g_commitment = commit_weights_fast(g_pad);
    p.h_commitment = commit_weights_fast(h_pad);
    tr.absorb_bytes("rmsnorm-pert-v1");
    tr.absorb(uint32_t(delta));
    tr.absorb_bytes(p.x_commitment.root); tr.absorb_bytes(p.gamma_commitment.root);
    tr.absorb_bytes(p.g_commitment.root); tr.absorb_bytes(p.h_commitment.root);
    tr.absorb(sum_sq.v);
    // step 1: variance
    ProdEF var = prove_product_ef(x_pad, x_pad, log_n, tr);
    p.var_proof = var.proof; p.var_fin_a = var.f_at_s.arr(); p.var_fin_b = var.g_at_s.arr();
    VEF s_var = points_of(var.proof.challenges);
    p.x_at_var_s = mle_evaluate_ef(x_pad, s_var).arr();
    p.x_var_eval_proof = prove_mle_eval_ef_base_bound(x_pad, s_var, "rmsnorm-x-var", p.x_commitment, tr);
    // step 2: g consistency
    VEF gc_point = tr.squeeze_ef_many(log_n);
    VEF eq_gc = eq_evals_ef(gc_point);
    EF t_g;
    for (size_t i = 0; i < n_pad; i++) t_g += eq_gc[i] * EF::from_f(g_pad[i]);
    VEF g_ef = widen(g_pad);
    ProdEF gp = prove_product_ef_full(eq_gc, g_ef, log_n, tr);
    p.g_prod_proof = gp.proof; p.g_prod_fin[0] = gp.f_at_s.arr(); p.g_prod_fin[1] = gp.g_at_s.arr();
    VEF s_gp = points_of(gp.proof.challenges);
    p.g_at_prod_s = mle_evaluate_ef(g_pad, s_gp).arr();
    p.g_prod_eval_proof = prove_mle_eval_ef_base_bound(g_pad, s_gp, "rmsnorm-g-prod", p.g_commitment, tr);
    TripEF gt = prove_triple_ef_full(eq_gc, widen(gamma_pad), widen(x_pad), log_n, tr);
    p.g_triple_proof = gt.proof;
    p.g_triple_fin[0] = gt.f_at_s.arr(); p.g_triple_fin[1] = gt.g_at_s.arr(); p.g_triple_fin[2] = gt.h_at_s.arr();
    p.t_g_claimed = t_g.arr();
    VEF s_gt = points_of(gt.proof.challenges);
    p.x_at_triple_s = mle_evaluate_ef(x_pad, s_gt).arr();
    p.x_triple_eval_proof = prove_mle_eval_ef_base_bound(x_pad, s_gt, "rmsnorm-x-triple", p.x_commitment, tr);
    p.gamma_at_triple_s = mle_evaluate_ef(gamma_pad, s_gt).arr();
    p.gamma_triple_eval_proof = prove_mle_eval_ef_base_bound(gamma_pad, s_gt, "rmsnorm-gamma-triple", p.gamma_commitment, tr);
    // step 3: squared checks
    VEF sq_point = tr.squeeze_ef_many(log_n);
    VEF eq_sq = eq_evals_ef(sq_point);
    EF s_h, s_g;
    for (size_t i = 0; i < n_pad; i++) s_h += eq_sq[i] * EF::from_f(h_pad[i]) * EF::from_f(h_pad[i]);
    VEF h_ef = widen(h_pad);
    TripEF hs = prove_triple_ef_full(eq_sq, h_ef, h_ef, log_n, tr);
    p.h_sq_proof = hs.proof;
    p.h_sq_fin[0] = hs.f_at_s.arr(); p.h_sq_fin[1] = hs.g_at_s.arr(); p.h_sq_fin[2] = hs.h_at_s.arr();
    p.s_h = s_h.arr();
    VEF s_hs = points_of(hs.proof.challenges);
    p.h_at_sq_s = mle_evaluate_ef(h_pad, s_hs).arr();
    p.h_sq_eval_proof = prove_mle_eval_ef_base_bound(h_pad, s_hs, "rmsnorm-h-sq", p.h_commitment, tr);
    for (size_t i = 0; i < n_pad; i++) s_g += eq_sq[i] * EF::from_f(g_pad[i]) * EF::from_f(g_pad[i]);
    TripEF gs = prove_triple_ef_full(eq_sq, g_ef, g_ef, log_n, tr);
    p.g_sq_proof = gs.proof;
    p.g_sq_fin[0] = gs.f_at_s.arr(); p.g_sq_fin[1] = gs.g_at_s.arr(); p.g_sq_fin[2] = gs.h_at_s.arr();
    p.s_g = s_g.arr();
    VEF s_gs = points_of(gs.proof.challenges);
    p.g_at_gsq_s = mle_evaluate_ef(g_pad, s_gs).arr();
    p.g_sq_eval_proof = prove_mle_eval_ef_base_bound(g_pad, s_gs, "rmsnorm-g-sq", p.g_commitment, tr);
    return p;
}

}  // namespace zko
