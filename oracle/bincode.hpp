// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// bincode 1.3 (default options: fixed-width little-endian integers, u64 lengths, u32 enum
// tags, one-byte Option tags, fixed arrays without a length) for the proof structs, with the
// field order of the reference's serde derives.  The reference measures proof size with this
// encoding (rust/zk_ml_prover/src/pipeline/mod.rs:270-283); here it is the byte string the
// parity tests compare.
#pragma once
#include "layers2.hpp"
#include "layers_base.hpp"

namespace zko {

struct Bin {
    std::vector<uint8_t> b;
    void u8(uint8_t v) { b.push_back(v); }
    void u32(uint32_t v) { for (int i = 0; i < 4; i++) b.push_back(uint8_t(v >> (8 * i))); }
    void u64(uint64_t v) { for (int i = 0; i < 8; i++) b.push_back(uint8_t(v >> (8 * i))); }
    void i32(int32_t v) { u32(uint32_t(v)); }
    void ef(const EFElement& e) { for (uint32_t v : e) u32(v); }
    void vec_u32(const std::vector<uint32_t>& v) { u64(v.size()); for (uint32_t x : v) u32(x); }
    void vec_ef(const std::vector<EFElement>& v) { u64(v.size()); for (auto& e : v) ef(e); }
    template <size_t N> void bytes(const std::array<uint8_t, N>& a) { b.insert(b.end(), a.begin(), a.end()); }
    void str(const std::string& t) { u64(t.size()); b.insert(b.end(), t.begin(), t.end()); }

    void put(const SumcheckProof& p) {                      // sumcheck.rs:57-65
        u64(p.round_polys.size());
        for (auto& r : p.round_polys) vec_u32(r);
        vec_u32(p.challenges);
    }
    void put(const SumcheckProofEF& p) {                    // sumcheck.rs:99-107
        u64(p.round_polys.size());
        for (auto& r : p.round_polys) vec_ef(r);
        vec_ef(p.challenges);
    }
    void put(const WeightCommitment& c) {                   // weight_commitment.rs:54-61
        bytes(c.root); u64(c.num_weights); u64(c.log_height); u32(c.kind);
    }
    void put(const MleEvalProof& p) {                       // weight_commitment.rs:65-73
        put(p.eval_sumcheck); u32(p.eq_at_s); u32(p.w_at_s); u8(0);
    }
    void put(const MleEvalProofEF& p) {                     // weight_commitment.rs:340-345
        put(p.eval_sumcheck); ef(p.eq_at_s); ef(p.w_at_s);
    }
    void put(const MatmulProof& p) {                        // matmul.rs:24-31
        put(p.sumcheck_proof); u32(p.w_at_rs); u32(p.x_at_s); vec_u32(p.r_point); vec_u32(p.s_point);
    }
    void put(const SuccinctMatmulProof& p) {                // matmul.rs:458-474
        put(p.matmul_proof); put(p.w_eval_proof); u32(p.w_claimed_value); put(p.w_partial_commitment);
        u8(p.bound ? 1 : 0); u8(0);
    }
    void put(const MatmulProofEF& p) {                      // matmul.rs:717-726
        put(p.sumcheck_proof); ef(p.w_at_rs); ef(p.x_at_s); vec_ef(p.r_point); vec_ef(p.s_point);
    }
    void put(const BatchMerkleProof& p) {                   // pcs.rs:43-53
        vec_u32(p.indices);
        vec_u32(p.values);
        u64(p.auth_nodes.size());
        for (auto& lvl : p.auth_nodes) { u64(lvl.size()); for (auto& d : lvl) bytes(d); }
    }
    void put(const BasefoldCommitment& c) { bytes(c.root); u64(c.num_coeffs); u64(c.log_n); }   // basefold.rs:39-47
    void put(const BasefoldOpeningProof& p) {               // basefold.rs:50-64, 73-81
        u64(p.fold_roots.size());
        for (auto& d : p.fold_roots) bytes(d);
        u64(p.fold_queries.size());
        for (auto& q : p.fold_queries) { put(q.prev_batch_proof); put(q.folded_batch_proof); }
        u32(p.final_value);
        vec_u32(p.final_coeffs);
    }
    void put(const SuccinctMatmulProofEF& p) {              // matmul.rs:947-960
        put(p.matmul_proof); put(p.w_eval_proof); ef(p.w_claimed_value); put(p.w_partial_commitment);
        u8(p.bound ? 1 : 0);
        u8(p.has_basefold ? 1 : 0);
        if (p.has_basefold) put(p.basefold_proof);
    }
    void put(const HadamardProof& p) {                      // elementwise.rs:31-44 (product_finals is a 3-tuple)
        put(p.product_sumcheck); u32(p.fin_eq); u32(p.fin_a); u32(p.fin_b); u32(p.c_eval);
        put(p.c_eval_proof); put(p.c_commitment);
    }
    void put(const AddProof& p) {                           // elementwise.rs:165-181
        put(p.a_sumcheck); u32(p.a_fin_eq); u32(p.a_fin); put(p.b_sumcheck); u32(p.b_fin_eq); u32(p.b_fin); u32(p.c_eval);
        put(p.c_eval_proof); put(p.c_commitment);
    }
    void put(const HadamardProofEF& p) {                    // elementwise.rs:415-426
        put(p.product_sumcheck); ef(p.fin_eq); ef(p.fin_a); ef(p.fin_b); ef(p.c_eval);
        put(p.c_eval_proof); put(p.c_commitment);
    }
    void put(const AddProofEF& p) {                         // elementwise.rs:527-542
        put(p.a_sumcheck); ef(p.a_fin_eq); ef(p.a_fin); put(p.b_sumcheck); ef(p.b_fin_eq); ef(p.b_fin);
        ef(p.c_eval); put(p.c_eval_proof); put(p.c_commitment);
    }
    void put(const RmsNormProof& p) {                       // rmsnorm.rs:36-85
        i32(p.perturbation_delta);
        put(p.var_proof); u32(p.var_fin[0]); u32(p.var_fin[1]); u32(p.sum_sq_value);
        put(p.h_sq_proof); for (uint32_t v : p.h_sq_fin) u32(v); u32(p.s_h);
        put(p.g_sq_proof); for (uint32_t v : p.g_sq_fin) u32(v); u32(p.s_g);
        put(p.g_prod_proof); for (uint32_t v : p.g_prod_fin) u32(v);
        put(p.g_triple_proof); for (uint32_t v : p.g_triple_fin) u32(v); u32(p.t_g_claimed);
        put(p.x_commitment); put(p.gamma_commitment); put(p.g_commitment); put(p.h_commitment);
        put(p.x_var_eval_proof); u32(p.x_at_var_s);
        put(p.g_prod_eval_proof); u32(p.g_at_prod_s);
        put(p.x_triple_eval_proof); u32(p.x_at_triple_s);
        put(p.gamma_triple_eval_proof); u32(p.gamma_at_triple_s);
        put(p.h_sq_eval_proof); u32(p.h_at_sq_s);
        put(p.g_sq_eval_proof); u32(p.g_at_gsq_s);
    }
    void put(const RmsNormProofEF& p) {                     // rmsnorm.rs:457-503
        i32(p.perturbation_delta);
        put(p.var_proof); ef(p.var_fin_a); ef(p.var_fin_b); u32(p.sum_sq_value);
        put(p.h_sq_proof); for (auto& e : p.h_sq_fin) ef(e); ef(p.s_h);
        put(p.g_sq_proof); for (auto& e : p.g_sq_fin) ef(e); ef(p.s_g);
        put(p.g_prod_proof); for (auto& e : p.g_prod_fin) ef(e);
        put(p.g_triple_proof); for (auto& e : p.g_triple_fin) ef(e); ef(p.t_g_claimed);
        put(p.x_commitment); put(p.gamma_commitment); put(p.g_commitment); put(p.h_commitment);
        put(p.x_var_eval_proof); ef(p.x_at_var_s);
        put(p.g_prod_eval_proof); ef(p.g_at_prod_s);
        put(p.x_triple_eval_proof); ef(p.x_at_triple_s);
        put(p.gamma_triple_eval_proof); ef(p.gamma_at_triple_s);
        put(p.h_sq_eval_proof); ef(p.h_at_sq_s);
        put(p.g_sq_eval_proof); ef(p.g_at_gsq_s);
    }
    void put(const LookupProof& p) {                        // lookup.rs:39-85
        put(p.table_commitment); put(p.multiplicity_commitment); put(p.sumcheck_proof); u32(p.fin_ones); u32(p.fin_h);
        u32(p.alpha); u32(p.beta);
        vec_u32(p.inputs); vec_u32(p.outputs); vec_u32(p.multiplicities);
        bytes(p.external_data_digest);
    }
    void put(const LookupProofEF& p) {                      // lookup.rs:89-115
        put(p.table_commitment); put(p.multiplicity_commitment); put(p.sumcheck_proof); ef(p.h_at_s);
        u8(0); u8(0);                                       // alpha: None, beta: None
        vec_u32(p.inputs); vec_u32(p.outputs); vec_u32(p.multiplicities);
        bytes(p.external_data_digest);
    }
    void put(const GateProofEF& p) { put(p.lookup_proof); put(p.hadamard_proof); }  // sigmoid_gate.rs:77-82, swiglu.rs:86-91
};

}  // namespace zko
