// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Base-field twins of the element-wise sub-protocols (challenges in M31; the mode of the
// reference's MLP / GPT-2 op lists), restating rust/zk_ml_prover/src/proving/elementwise.rs:
//   HadamardProof, prove_hadamard, verify_hadamard   :31-44, 50-98, 106-157
//   AddProof, prove_add, verify_add                  :165-181, 189-235, 244-301
#pragma once
#include "layers.hpp"

namespace zko {

struct HadamardProof {
    SumcheckProof product_sumcheck;
    uint32_t fin_eq = 0, fin_a = 0, fin_b = 0;
    uint32_t c_eval = 0;
    MleEvalProof c_eval_proof;
    WeightCommitment c_commitment;
};
inline HadamardProof prove_hadamard(const VF& a, const VF& b, const VF& c, const VF& point, Transcript& tr) {
    size_t log_n = point.size(), n_pad = size_t(1) << log_n;
    VF a_pad = padded(a, n_pad), b_pad = padded(b, n_pad), c_pad = padded(c, n_pad);
    HadamardProof p;
    p.c_commitment = commit_weights_fast(c_pad);
    tr.absorb_bytes(p.c_commitment.root);
    VF eq = eq_evals(point);
    Trip t = prove_triple(eq, a_pad, b_pad, log_n, tr);
    p.product_sumcheck = t.proof;
    p.fin_eq = t.f_at_s.v; p.fin_a = t.g_at_s.v; p.fin_b = t.h_at_s.v;
    p.c_eval = mle_evaluate(c_pad, point).v;
    p.c_eval_proof = prove_mle_eval_bound(c_pad, point, "hadamard-c-eval", p.c_commitment, tr);
    return p;
}
inline bool verify_hadamard(const HadamardProof& p, const VF& point, Transcript& tr) {
    tr.absorb_bytes(p.c_commitment.root);
    VF s;
    if (p.product_sumcheck.round_polys.size() != point.size()) return false;
    if (!verify_triple_with_challenges(F(p.c_eval), p.product_sumcheck, F(p.fin_eq), F(p.fin_a), F(p.fin_b), tr, &s)) return false;
    if (compute_eq_at_point(point, s) != F(p.fin_eq)) return false;
    return verify_mle_eval_bound(p.c_commitment, F(p.c_eval), point, p.c_eval_proof, "hadamard-c-eval", tr);
}

struct AddProof {
    SumcheckProof a_sumcheck;
    uint32_t a_fin_eq = 0, a_fin = 0;
    SumcheckProof b_sumcheck;
    uint32_t b_fin_eq = 0, b_fin = 0;
    uint32_t c_eval = 0;
    MleEvalProof c_eval_proof;
    WeightCommitment c_commitment;
};
inline AddProof prove_add(const VF& a, const VF& b, const VF& c, const VF& point, Transcript& tr) {
    size_t log_n = point.size(), n_pad = size_t(1) << log_n;
    VF a_pad = padded(a, n_pad), b_pad = padded(b, n_pad), c_pad = padded(c, n_pad);
    AddProof p;
    p.c_commitment = commit_weights_fast(c_pad);
    tr.absorb_bytes(p.c_commitment.root);
    VF eq = eq_evals(point);
    Prod ra = prove_product(eq, a_pad, log_n, tr);
    Prod rb = prove_product(eq, b_pad, log_n, tr);
    p.a_sumcheck = ra.proof; p.a_fin_eq = ra.f_at_s.v; p.a_fin = ra.g_at_s.v;
    p.b_sumcheck = rb.proof; p.b_fin_eq = rb.f_at_s.v; p.b_fin = rb.g_at_s.v;
    p.c_eval = mle_evaluate(c_pad, point).v;
    p.c_eval_proof = prove_mle_eval_bound(c_pad, point, "add-c-eval", p.c_commitment, tr);
    return p;
}
inline bool verify_add(const AddProof& p, const VF& point, Transcript& tr) {
    tr.absorb_bytes(p.c_commitment.root);
    if (p.a_sumcheck.round_polys.empty() || p.b_sumcheck.round_polys.empty()) return false;
    if (p.a_sumcheck.round_polys[0].size() < 2 || p.b_sumcheck.round_polys[0].size() < 2) return false;
    F a_eval = F(p.a_sumcheck.round_polys[0][0]) + F(p.a_sumcheck.round_polys[0][1]);
    VF sa, sb;
    if (!verify_product_with_challenges(a_eval, p.a_sumcheck, F(p.a_fin_eq), F(p.a_fin), tr, &sa)) return false;
    if (compute_eq_at_point(point, sa) != F(p.a_fin_eq)) return false;
    F b_eval = F(p.b_sumcheck.round_polys[0][0]) + F(p.b_sumcheck.round_polys[0][1]);
    if (!verify_product_with_challenges(b_eval, p.b_sumcheck, F(p.b_fin_eq), F(p.b_fin), tr, &sb)) return false;
    if (compute_eq_at_point(point, sb) != F(p.b_fin_eq)) return false;
    if (a_eval + b_eval != F(p.c_eval)) return false;
    return verify_mle_eval_bound(p.c_commitment, F(p.c_eval), point, p.c_eval_proof, "add-c-eval", tr);
}

}  // namespace zko

namespace zko {

// ------------------------------------------------------------------ LogUp lookup, base field
// lookup.rs:39-85 (LookupProof), :322-345 (batch_inverse), :432-604 (prove_lookup),
// :803-874 (verify_lookup_with_data).  Unlike the EF variant, the active subtable is committed
// as inp + beta * out, the challenges alpha and beta are part of the proof, and the sumcheck is
// the base-field all-ones product sumcheck.
struct LookupProof {
    WeightCommitment table_commitment, multiplicity_commitment;
    SumcheckProof sumcheck_proof;
    uint32_t fin_ones = 0, fin_h = 0;
    uint32_t alpha = 0, beta = 0;
    std::vector<uint32_t> inputs, outputs, multiplicities;
    std::array<uint8_t, 32> external_data_digest{};
};
inline VF batch_inverse(const VF& v) {
    size_t n = v.size();
    if (!n) return {};
    VF prefix(n), res(n);
    prefix[0] = v[0];
    for (size_t i = 1; i < n; i++) prefix[i] = prefix[i - 1] * v[i];
    F inv = inverse(prefix[n - 1]);
    for (size_t i = n - 1; i >= 1; i--) { res[i] = inv * prefix[i - 1]; inv = inv * v[i]; }
    res[0] = inv;
    return res;
}
inline LookupProof prove_lookup(const LookupTable& table, const VF& inputs, const VF& outputs, Transcript& tr) {
    size_t n_lookups = inputs.size(), n_table = table.inputs.size();
    uint8_t zero_root[32] = {0};
    tr.absorb_bytes(zero_root, 32);
    tr.absorb(uint32_t(n_lookups));
    for (size_t i = 0; i < n_lookups; i++) { tr.absorb(inputs[i]); tr.absorb(outputs[i]); }
    F beta = tr.squeeze(), alpha = tr.squeeze();
    std::vector<uint32_t> mult(n_table, 0);
    for (F a : inputs) { size_t idx = field_to_table_index(a.v, n_table); if (idx < n_table) mult[idx]++; }
    VF active_t, active_mult;
    for (size_t j = 0; j < n_table; j++) if (mult[j] > 0) {
        active_t.push_back(F(table.inputs[j]) + beta * F(table.outputs[j]));
        active_mult.push_back(F(mult[j]));
    }
    size_t n_active = active_t.size();
    LookupProof p;
    p.table_commitment = commit_weights_fast(active_t);
    p.multiplicity_commitment = commit_weights_fast(active_mult);
    size_t log_n = log2_ceil(n_lookups + n_active), n_pad = size_t(1) << log_n;
    VF denoms;
    for (size_t i = 0; i < n_lookups; i++) {
        F d = alpha - (inputs[i] + beta * outputs[i]);
        if (d == F::zero()) throw LookupFailure("alpha collision with lookup encoding");
        denoms.push_back(d);
    }
    for (size_t k = 0; k < n_active; k++) {
        F d = alpha - active_t[k];
        if (d == F::zero()) throw LookupFailure("alpha collision with table encoding");
        denoms.push_back(d);
    }
    VF inv = batch_inverse(denoms);
    VF h(n_pad, F::zero());
    for (size_t i = 0; i < n_lookups; i++) h[i] = inv[i];
    for (size_t k = 0; k < n_active; k++) h[n_lookups + k] = F::zero() - active_mult[k] * inv[n_lookups + k];
    F sum = F::zero();
    for (F v : h) sum += v;
    if (sum != F::zero()) throw LookupFailure("LogUp identity failed — invalid lookups");
    tr.absorb_bytes(p.table_commitment.root);
    tr.absorb_bytes(p.multiplicity_commitment.root);
    Prod sc = prove_product_ones(h, log_n, tr);
    p.sumcheck_proof = sc.proof;
    p.fin_ones = sc.f_at_s.v; p.fin_h = sc.g_at_s.v;
    p.alpha = alpha.v; p.beta = beta.v;
    for (F v : inputs) p.inputs.push_back(v.v);
    for (F v : outputs) p.outputs.push_back(v.v);
    p.external_data_digest = compute_lookup_external_digest(inputs, outputs);
    return p;
}
inline bool verify_lookup(const LookupProof& p, size_t num_lookups, Transcript& tr) {
    VF inputs, outputs;
    for (uint32_t v : p.inputs) inputs.push_back(F(v));
    for (uint32_t v : p.outputs) outputs.push_back(F(v));
    std::array<uint8_t, 32> zero{};
    if (p.external_data_digest != zero && compute_lookup_external_digest(inputs, outputs) != p.external_data_digest) return false;
    tr.absorb_bytes(zero);
    tr.absorb(uint32_t(num_lookups));
    for (size_t i = 0; i < inputs.size() && i < outputs.size(); i++) { tr.absorb(inputs[i]); tr.absorb(outputs[i]); }
    F beta = tr.squeeze(), alpha = tr.squeeze();
    if (alpha.v != p.alpha || beta.v != p.beta) return false;
    size_t log_n = log2_ceil(num_lookups + p.table_commitment.num_weights);
    tr.absorb_bytes(p.table_commitment.root);
    tr.absorb_bytes(p.multiplicity_commitment.root);
    if (p.sumcheck_proof.round_polys.size() != log_n) return false;
    // sumcheck.rs verify_product with the ones-sumcheck's two stored evaluations [s0, s2]
    if (!verify_product(F::zero(), p.sumcheck_proof, F(p.fin_ones), F(p.fin_h), tr)) return false;   // lookup.rs:857
    return F(p.fin_ones) == F::one();
}

}  // namespace zko

namespace zko {

// ------------------------------------------------------------------ RMSNorm, base field
// rmsnorm.rs:36-85 (RmsNormProof), :96-246 (prove_rmsnorm), :256-447 (verify_rmsnorm).
struct RmsNormProof {
    int32_t perturbation_delta = 0;
    SumcheckProof var_proof;      uint32_t var_fin[2]{};
    uint32_t sum_sq_value = 0;
    SumcheckProof h_sq_proof;     uint32_t h_sq_fin[3]{};   uint32_t s_h = 0;
    SumcheckProof g_sq_proof;     uint32_t g_sq_fin[3]{};   uint32_t s_g = 0;
    SumcheckProof g_prod_proof;   uint32_t g_prod_fin[2]{};
    SumcheckProof g_triple_proof; uint32_t g_triple_fin[3]{};
    uint32_t t_g_claimed = 0;
    WeightCommitment x_commitment, gamma_commitment, g_commitment, h_commitment;
    MleEvalProof x_var_eval_proof;        uint32_t x_at_var_s = 0;
    MleEvalProof g_prod_eval_proof;       uint32_t g_at_prod_s = 0;
    MleEvalProof x_triple_eval_proof;     uint32_t x_at_triple_s = 0;
    MleEvalProof gamma_triple_eval_proof; uint32_t gamma_at_triple_s = 0;
    MleEvalProof h_sq_eval_proof;         uint32_t h_at_sq_s = 0;
    MleEvalProof g_sq_eval_proof;         uint32_t g_at_gsq_s = 0;
};
inline VF base_points_of(const std::vector<uint32_t>& c) { VF o; for (uint32_t v : c) o.push_back(F(v)); return o; }

inline RmsNormProof prove_rmsnorm(const VF& x, const VF& gamma, const VF& y, int32_t delta, Transcript& tr) {
    size_t d = x.size(), log_n = log2_ceil(d), n_pad = size_t(1) << log_n;
    VF x_pad = padded(x, n_pad), gamma_pad = padded(gamma, n_pad), h_pad = padded(y, n_pad);
    VF g_pad(n_pad, F::zero());
    for (size_t i = 0; i < d; i++) g_pad[i] = gamma_pad[i] * x_pad[i];
    F sum_sq;
    for (F v : x_pad) sum_sq += v * v;
    RmsNormProof p;
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
    Prod var = prove_product(x_pad, x_pad, log_n, tr);
    p.var_proof = var.proof; p.var_fin[0] = var.f_at_s.v; p.var_fin[1] = var.g_at_s.v;
    VF s_var = base_points_of(var.proof.challenges);
    p.x_at_var_s = mle_evaluate(x_pad, s_var).v;
    p.x_var_eval_proof = prove_mle_eval_bound(x_pad, s_var, "rmsnorm-x-var", p.x_commitment, tr);
    VF gc_point = tr.squeeze_many(log_n);
    VF eq_gc = eq_evals(gc_point);
    F t_g;
    for (size_t i = 0; i < n_pad; i++) t_g += eq_gc[i] * g_pad[i];
    Prod gp = prove_product(eq_gc, g_pad, log_n, tr);
    p.g_prod_proof = gp.proof; p.g_prod_fin[0] = gp.f_at_s.v; p.g_prod_fin[1] = gp.g_at_s.v;
    VF s_gp = base_points_of(gp.proof.challenges);
    p.g_at_prod_s = mle_evaluate(g_pad, s_gp).v;
    p.g_prod_eval_proof = prove_mle_eval_bound(g_pad, s_gp, "rmsnorm-g-prod", p.g_commitment, tr);
    Trip gt = prove_triple(eq_gc, gamma_pad, x_pad, log_n, tr);
    p.g_triple_proof = gt.proof;
    p.g_triple_fin[0] = gt.f_at_s.v; p.g_triple_fin[1] = gt.g_at_s.v; p.g_triple_fin[2] = gt.h_at_s.v;
    p.t_g_claimed = t_g.v;
    VF s_gt = base_points_of(gt.proof.challenges);
    p.x_at_triple_s = mle_evaluate(x_pad, s_gt).v;
    p.x_triple_eval_proof = prove_mle_eval_bound(x_pad, s_gt, "rmsnorm-x-triple", p.x_commitment, tr);
    p.gamma_at_triple_s = mle_evaluate(gamma_pad, s_gt).v;
    p.gamma_triple_eval_proof = prove_mle_eval_bound(gamma_pad, s_gt, "rmsnorm-gamma-triple", p.gamma_commitment, tr);
    VF sq_point = tr.squeeze_many(log_n);
    VF eq_sq = eq_evals(sq_point);
    F s_h, s_g;
    for (size_t i = 0; i < n_pad; i++) s_h += eq_sq[i] * h_pad[i] * h_pad[i];
    Trip hs = prove_triple(eq_sq, h_pad, h_pad, log_n, tr);
    p.h_sq_proof = hs.proof;
    p.h_sq_fin[0] = hs.f_at_s.v; p.h_sq_fin[1] = hs.g_at_s.v; p.h_sq_fin[2] = hs.h_at_s.v;
    p.s_h = s_h.v;
    VF s_hs = base_points_of(hs.proof.challenges);
    p.h_at_sq_s = mle_evaluate(h_pad, s_hs).v;
    p.h_sq_eval_proof = prove_mle_eval_bound(h_pad, s_hs, "rmsnorm-h-sq", p.h_commitment, tr);
    for (size_t i = 0; i < n_pad; i++) s_g += eq_sq[i] * g_pad[i] * g_pad[i];
    Trip gs = prove_triple(eq_sq, g_pad, g_pad, log_n, tr);
    p.g_sq_proof = gs.proof;
    p.g_sq_fin[0] = gs.f_at_s.v; p.g_sq_fin[1] = gs.g_at_s.v; p.g_sq_fin[2] = gs.h_at_s.v;
    p.s_g = s_g.v;
    VF s_gs = base_points_of(gs.proof.challenges);
    p.g_at_gsq_s = mle_evaluate(g_pad, s_gs).v;
    p.g_sq_eval_proof = prove_mle_eval_bound(g_pad, s_gs, "rmsnorm-g-sq", p.g_commitment, tr);
    return p;
}

inline bool verify_rmsnorm(const RmsNormProof& p, const VF& y, size_t d, Transcript& tr) {
    size_t log_n = log2_ceil(d), n_pad = size_t(1) << log_n;
    F sum_sq(p.sum_sq_value);
    F d_field = F(uint32_t(d));
    tr.absorb_bytes("rmsnorm-pert-v1");
    tr.absorb(uint32_t(p.perturbation_delta));
    tr.absorb_bytes(p.x_commitment.root); tr.absorb_bytes(p.gamma_commitment.root);
    tr.absorb_bytes(p.g_commitment.root); tr.absorb_bytes(p.h_commitment.root);
    tr.absorb(p.sum_sq_value);
    auto rounds_ok = [&](const SumcheckProof& sp) { return sp.round_polys.size() == log_n && sp.challenges.size() == log_n; };
    if (!rounds_ok(p.var_proof) || !rounds_ok(p.g_prod_proof) || !rounds_ok(p.g_triple_proof) || !rounds_ok(p.h_sq_proof) || !rounds_ok(p.g_sq_proof))
        return false;
    if (!verify_product_with_challenges(sum_sq, p.var_proof, F(p.var_fin[0]), F(p.var_fin[1]), tr)) return false;
    if (p.var_fin[0] != p.var_fin[1] || p.x_at_var_s != p.var_fin[0]) return false;
    VF s_var = base_points_of(p.var_proof.challenges);
    if (!verify_mle_eval_bound(p.x_commitment, F(p.x_at_var_s), s_var, p.x_var_eval_proof, "rmsnorm-x-var", tr)) return false;
    VF gc_point = tr.squeeze_many(log_n);
    F t_g(p.t_g_claimed);
    if (!verify_product_with_challenges(t_g, p.g_prod_proof, F(p.g_prod_fin[0]), F(p.g_prod_fin[1]), tr)) return false;
    VF s_gp = base_points_of(p.g_prod_proof.challenges);
    if (compute_eq_at_point(gc_point, s_gp) != F(p.g_prod_fin[0])) return false;
    if (p.g_at_prod_s != p.g_prod_fin[1]) return false;
    if (!verify_mle_eval_bound(p.g_commitment, F(p.g_at_prod_s), s_gp, p.g_prod_eval_proof, "rmsnorm-g-prod", tr)) return false;
    if (!verify_triple_with_challenges(t_g, p.g_triple_proof, F(p.g_triple_fin[0]), F(p.g_triple_fin[1]), F(p.g_triple_fin[2]), tr)) return false;
    VF s_gt = base_points_of(p.g_triple_proof.challenges);
    if (compute_eq_at_point(gc_point, s_gt) != F(p.g_triple_fin[0])) return false;
    if (p.x_at_triple_s != p.g_triple_fin[2]) return false;
    if (!verify_mle_eval_bound(p.x_commitment, F(p.x_at_triple_s), s_gt, p.x_triple_eval_proof, "rmsnorm-x-triple", tr)) return false;
    if (p.gamma_at_triple_s != p.g_triple_fin[1]) return false;
    if (!verify_mle_eval_bound(p.gamma_commitment, F(p.gamma_at_triple_s), s_gt, p.gamma_triple_eval_proof, "rmsnorm-gamma-triple", tr)) return false;
    VF sq_point = tr.squeeze_many(log_n);
    F s_h(p.s_h), s_g(p.s_g);
    if (!verify_triple_with_challenges(s_h, p.h_sq_proof, F(p.h_sq_fin[0]), F(p.h_sq_fin[1]), F(p.h_sq_fin[2]), tr)) return false;
    VF s_hs = base_points_of(p.h_sq_proof.challenges);
    if (compute_eq_at_point(sq_point, s_hs) != F(p.h_sq_fin[0])) return false;
    if (p.h_sq_fin[1] != p.h_sq_fin[2] || p.h_at_sq_s != p.h_sq_fin[1]) return false;
    if (!verify_mle_eval_bound(p.h_commitment, F(p.h_at_sq_s), s_hs, p.h_sq_eval_proof, "rmsnorm-h-sq", tr)) return false;
    if (commit_weights_fast(padded(y, n_pad)).root != p.h_commitment.root) return false;
    if (!verify_triple_with_challenges(s_g, p.g_sq_proof, F(p.g_sq_fin[0]), F(p.g_sq_fin[1]), F(p.g_sq_fin[2]), tr)) return false;
    VF s_gs = base_points_of(p.g_sq_proof.challenges);
    if (compute_eq_at_point(sq_point, s_gs) != F(p.g_sq_fin[0])) return false;
    if (p.g_sq_fin[1] != p.g_sq_fin[2] || p.g_at_gsq_s != p.g_sq_fin[1]) return false;
    if (!verify_mle_eval_bound(p.g_commitment, F(p.g_at_gsq_s), s_gs, p.g_sq_eval_proof, "rmsnorm-g-sq", tr)) return false;
    return sum_sq * s_h == d_field * s_g;
}

}  // namespace zko
