// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// verify_rmsnorm_ef (rust/zk_ml_prover/src/proving/rmsnorm.rs:670-862) and the EF LogUp
// lookup argument with its sigmoid-gate / SwiGLU wrappers
// (rust/zk_ml_prover/src/proving/lookup.rs, sigmoid_gate.rs, swiglu.rs).
#pragma once
#include "layers.hpp"

namespace zko {

inline bool verify_rmsnorm_ef(const RmsNormProofEF& p, const VF& y, size_t d, Transcript& tr) {
    size_t log_n = log2_ceil(d), n_pad = size_t(1) << log_n;
    EF sum_sq = EF::from_f(F(p.sum_sq_value)), d_ef = EF::from_f(F(uint32_t(d)));
    tr.absorb_bytes("rmsnorm-pert-v1");
    tr.absorb(uint32_t(p.perturbation_delta));
    tr.absorb_bytes(p.x_commitment.root); tr.absorb_bytes(p.gamma_commitment.root);
    tr.absorb_bytes(p.g_commitment.root); tr.absorb_bytes(p.h_commitment.root);
    tr.absorb(p.sum_sq_value);
    // variance
    EF xa = ef_of(p.var_fin_a), xb = ef_of(p.var_fin_b);
    VEF s_var;
    if (!verify_product_ef_with_challenges(sum_sq, p.var_proof, xa, xb, tr, &s_var)) return false;
    if (xa != xb) return false;
    if (ef_of(p.x_at_var_s) != xa) return false;
    if (!verify_mle_eval_ef_bound(p.x_commitment, xa, s_var, p.x_var_eval_proof, "rmsnorm-x-var", tr)) return false;
    // g consistency
    VEF gc_point = tr.squeeze_ef_many(log_n);
    EF t_g = ef_of(p.t_g_claimed);
    VEF s_gp;
    if (!verify_product_ef_with_challenges(t_g, p.g_prod_proof, ef_of(p.g_prod_fin[0]), ef_of(p.g_prod_fin[1]), tr, &s_gp)) return false;
    if (compute_eq_at_point_ef(gc_point, s_gp) != ef_of(p.g_prod_fin[0])) return false;
    if (ef_of(p.g_at_prod_s) != ef_of(p.g_prod_fin[1])) return false;
    if (!verify_mle_eval_ef_bound(p.g_commitment, ef_of(p.g_at_prod_s), s_gp, p.g_prod_eval_proof, "rmsnorm-g-prod", tr)) return false;
    VEF s_gt;
    if (!verify_triple_ef_with_challenges(t_g, p.g_triple_proof, ef_of(p.g_triple_fin[0]), ef_of(p.g_triple_fin[1]),
                                          ef_of(p.g_triple_fin[2]), tr, &s_gt)) return false;
    if (compute_eq_at_point_ef(gc_point, s_gt) != ef_of(p.g_triple_fin[0])) return false;
    if (ef_of(p.x_at_triple_s) != ef_of(p.g_triple_fin[2])) return false;
    if (!verify_mle_eval_ef_bound(p.x_commitment, ef_of(p.x_at_triple_s), s_gt, p.x_triple_eval_proof, "rmsnorm-x-triple", tr)) return false;
    if (ef_of(p.gamma_at_triple_s) != ef_of(p.g_triple_fin[1])) return false;
    if (!verify_mle_eval_ef_bound(p.gamma_commitment, ef_of(p.gamma_at_triple_s), s_gt, p.gamma_triple_eval_proof, "rmsnorm-gamma-triple", tr)) return false;
    // squared checks
    VEF sq_point = tr.squeeze_ef_many(log_n);
    EF s_h = ef_of(p.s_h), s_g = ef_of(p.s_g);
    VEF s_hs;
    if (!verify_triple_ef_with_challenges(s_h, p.h_sq_proof, ef_of(p.h_sq_fin[0]), ef_of(p.h_sq_fin[1]), ef_of(p.h_sq_fin[2]), tr, &s_hs)) return false;
    if (compute_eq_at_point_ef(sq_point, s_hs) != ef_of(p.h_sq_fin[0])) return false;
    if (ef_of(p.h_sq_fin[1]) != ef_of(p.h_sq_fin[2])) return false;
    if (ef_of(p.h_at_sq_s) != ef_of(p.h_sq_fin[1])) return false;
    if (!verify_mle_eval_ef_bound(p.h_commitment, ef_of(p.h_at_sq_s), s_hs, p.h_sq_eval_proof, "rmsnorm-h-sq", tr)) return false;
    if (commit_weights_fast(padded(y, n_pad)).root != p.h_commitment.root) return false;
    VEF s_gs;
    if (!verify_triple_ef_with_challenges(s_g, p.g_sq_proof, ef_of(p.g_sq_fin[0]), ef_of(p.g_sq_fin[1]), ef_of(p.g_sq_fin[2]), tr, &s_gs)) return false;
    if (compute_eq_at_point_ef(sq_point, s_gs) != ef_of(p.g_sq_fin[0])) return false;
    if (ef_of(p.g_sq_fin[1]) != ef_of(p.g_sq_fin[2])) return false;
    if (ef_of(p.g_at_gsq_s) != ef_of(p.g_sq_fin[1])) return false;
    if (!verify_mle_eval_ef_bound(p.g_commitment, ef_of(p.g_at_gsq_s), s_gs, p.g_sq_eval_proof, "rmsnorm-g-sq", tr)) return false;
    return sum_sq * s_h == d_ef * s_g;
}

// ------------------------------------------------------------------ lookup tables
// A 65536-entry (or 256-entry) table: entry `raw` has input i16_to_field(raw as i16) and an
// output column supplied by the host (f64 math stays on the host; lookup.rs:122-285).
struct LookupTable {
    std::vector<uint32_t> inputs, outputs;   // same length, table order
};
inline uint32_t i16_to_field(int32_t x) { return to_field(x).v; }
inline LookupTable table_from_outputs(const std::vector<uint32_t>& outputs) {
    LookupTable t;
    size_t n = outputs.size();
    t.outputs = outputs;
    t.inputs.resize(n);
    for (size_t raw = 0; raw < n; raw++) {
        int32_t s = n == 65536 ? int32_t(int16_t(uint16_t(raw))) : int32_t(int8_t(uint8_t(raw)));
        t.inputs[raw] = i16_to_field(s);
    }
    return t;
}
// lookup.rs:377-390
inline size_t field_to_table_index(uint32_t v, size_t n_table) {
    uint64_t half = n_table / 2;
    if (v < half) return v;
    if (uint64_t(v) >= uint64_t(P31) - half) return size_t(uint64_t(v) + n_table - P31);
    return SIZE_MAX;
}
// lookup.rs:348-368 — Montgomery batch inversion in EF.
inline VEF batch_inverse_ef(const VEF& v) {
    size_t n = v.size();
    if (!n) return {};
    VEF prefix(n), res(n);
    prefix[0] = v[0];
    for (size_t i = 1; i < n; i++) prefix[i] = prefix[i - 1] * v[i];
    EF inv = inverse(prefix[n - 1]);
    for (size_t i = n - 1; i >= 1; i--) { res[i] = inv * prefix[i - 1]; inv = inv * v[i]; }
    res[0] = inv;
    return res;
}
// lookup.rs:609-621
inline std::array<uint8_t, 32> compute_lookup_external_digest(const VF& in, const VF& out) {
    std::vector<uint8_t> b;
    auto push = [&](const void* p, size_t n) { const uint8_t* q = (const uint8_t*)p; b.insert(b.end(), q, q + n); };
    push("lookup-external-data-v1", 23);
    uint64_t n = in.size(); push(&n, 8);
    for (F v : in) push(&v.v, 4);
    n = out.size(); push(&n, 8);
    for (F v : out) push(&v.v, 4);
    return blake3(b);
}

// lookup.rs:89-115
struct LookupProofEF {
    WeightCommitment table_commitment, multiplicity_commitment;
    SumcheckProofEF sumcheck_proof;
    EFElement h_at_s{};
    // alpha: None, beta: None
    std::vector<uint32_t> inputs, outputs, multiplicities;
    std::array<uint8_t, 32> external_data_digest{};
};
struct LookupFailure : std::runtime_error { using std::runtime_error::runtime_error; };

// lookup.rs:643-762
inline LookupProofEF prove_lookup_ef(const LookupTable& table, const VF& inputs, const VF& outputs, Transcript& tr) {
    size_t n_lookups = inputs.size(), n_table = table.inputs.size();
    uint8_t zero_root[32] = {0};
    tr.absorb_bytes(zero_root, 32);
    tr.absorb(uint32_t(n_lookups));
    for (size_t i = 0; i < n_lookups; i++) { tr.absorb(inputs[i]); tr.absorb(outputs[i]); }
    EF beta = tr.squeeze_ef(), alpha = tr.squeeze_ef();
    std::vector<uint32_t> mult(n_table, 0);
    for (F a : inputs) { size_t idx = field_to_table_index(a.v, n_table); if (idx < n_table) mult[idx]++; }
    VEF denoms;
    for (size_t i = 0; i < n_lookups; i++) {
        EF d = alpha - (EF::from_f(inputs[i]) + beta * EF::from_f(outputs[i]));
        if (d == EF::zero()) throw LookupFailure("alpha collision with lookup encoding");
        denoms.push_back(d);
    }
    VF active_entries, active_mult;
    for (size_t j = 0; j < n_table; j++) if (mult[j] > 0) {
        EF t = EF::from_f(F(table.inputs[j])) + beta * EF::from_f(F(table.outputs[j]));
        EF d = alpha - t;
        if (d == EF::zero()) throw LookupFailure("alpha collision with table encoding");
        denoms.push_back(d);
        active_entries.push_back(F(table.inputs[j]) + F(table.outputs[j]));
        active_mult.push_back(F(mult[j]));
    }
    size_t n_active = active_mult.size();
    LookupProofEF p;
    p.table_commitment = commit_weights_fast(active_entries);
    p.multiplicity_commitment = commit_weights_fast(active_mult);
    size_t log_n = log2_ceil(n_lookups + n_active), n_pad = size_t(1) << log_n;
    VEF inv = batch_inverse_ef(denoms);
    VEF h(n_pad, EF::zero());
    for (size_t i = 0; i < n_lookups; i++) h[i] = inv[i];
    for (size_t k = 0; k < n_active; k++) h[n_lookups + k] = EF::zero() - EF::from_f(active_mult[k]) * inv[n_lookups + k];
    EF sum;
    for (EF v : h) sum += v;
    if (sum != EF::zero()) throw LookupFailure("LogUp identity failed — invalid lookups");
    tr.absorb_bytes(p.table_commitment.root);
    tr.absorb_bytes(p.multiplicity_commitment.root);
    ProdEF sc = prove_product_ones_ef_full(h, log_n, tr);
    p.sumcheck_proof = sc.proof;
    p.h_at_s = sc.g_at_s.arr();
    for (F v : inputs) p.inputs.push_back(v.v);
    for (F v : outputs) p.outputs.push_back(v.v);
    p.external_data_digest = compute_lookup_external_digest(inputs, outputs);
    return p;
}
// lookup.rs:912-976 (external data supplied by the caller, as the layer verifier does)
inline bool verify_lookup_ef_with_data(const LookupProofEF& p, size_t num_lookups, const VF& inputs, const VF& outputs, Transcript& tr) {
    std::array<uint8_t, 32> zero{};
    if (p.external_data_digest != zero && compute_lookup_external_digest(inputs, outputs) != p.external_data_digest) return false;
    tr.absorb_bytes(zero);
    tr.absorb(uint32_t(num_lookups));
    for (size_t i = 0; i < inputs.size() && i < outputs.size(); i++) { tr.absorb(inputs[i]); tr.absorb(outputs[i]); }
    tr.squeeze_ef(); tr.squeeze_ef();
    tr.absorb_bytes(p.table_commitment.root);
    tr.absorb_bytes(p.multiplicity_commitment.root);
    return verify_product_ef_with_challenges(EF::zero(), p.sumcheck_proof, EF::one(), ef_of(p.h_at_s), tr);
}

// sigmoid_gate.rs:75-114 / swiglu.rs:84-118: lookup, squeeze the hadamard point, hadamard.
struct GateProofEF { LookupProofEF lookup_proof; HadamardProofEF hadamard_proof; };
inline GateProofEF prove_lookup_then_hadamard_ef(const VF& lk_in, const VF& lk_out, const VF& had_a, const VF& had_b,
                                                 const VF& out, const LookupTable& table, Transcript& tr) {
    GateProofEF p;
    size_t log_n = log2_ceil(out.size());
    p.lookup_proof = prove_lookup_ef(table, lk_in, lk_out, tr);
    VEF point = tr.squeeze_ef_many(log_n);
    p.hadamard_proof = prove_hadamard_ef(had_a, had_b, out, point, tr);
    return p;
}
// prove_sigmoid_gate_ef(gate, gate_sigmoid, input, output): hadamard(input, gate_sigmoid) = output
inline GateProofEF prove_sigmoid_gate_ef(const VF& gate, const VF& gate_sigmoid, const VF& input, const VF& output,
                                         const LookupTable& t, Transcript& tr) {
    return prove_lookup_then_hadamard_ef(gate, gate_sigmoid, input, gate_sigmoid, output, t, tr);
}
// prove_swiglu_ef(gate, gate_silu, up, output): hadamard(gate_silu, up) = output
inline GateProofEF prove_swiglu_ef(const VF& gate, const VF& gate_silu, const VF& up, const VF& output,
                                   const LookupTable& t, Transcript& tr) {
    return prove_lookup_then_hadamard_ef(gate, gate_silu, gate_silu, up, output, t, tr);
}
inline bool verify_gate_ef_with_data(const GateProofEF& p, size_t num_elements, const VF& lk_in, const VF& lk_out, Transcript& tr) {
    size_t log_n = log2_ceil(num_elements);
    if (!verify_lookup_ef_with_data(p.lookup_proof, num_elements, lk_in, lk_out, tr)) return false;
    VEF point = tr.squeeze_ef_many(log_n);
    return verify_hadamard_ef(p.hadamard_proof, point, tr);
}

}  // namespace zko
