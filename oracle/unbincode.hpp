// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// The inverse of bincode.hpp for the extension-field layer proof: QwenLayerProofEF (qwen.rs:711-737)
// and the structs inside it, decoded from the bytes the provers emit, so that the restated verifier
// can be run on byte strings (honest or tampered) and be compared with the GPU verifier.
#pragma once
#include "bincode.hpp"
#include "qwen_verify.hpp"

namespace zko {

struct Rd {
    const uint8_t* p; size_t n, at = 0; bool ok = true;
    uint8_t u8() { if (at + 1 > n) { ok = false; return 0; } return p[at++]; }
    uint32_t u32() { if (at + 4 > n) { ok = false; return 0; } uint32_t v = 0; for (int i = 0; i < 4; i++) v |= uint32_t(p[at + i]) << (8 * i); at += 4; return v; }
    uint64_t u64() { if (at + 8 > n) { ok = false; return 0; } uint64_t v = 0; for (int i = 0; i < 8; i++) v |= uint64_t(p[at + i]) << (8 * i); at += 8; return v; }
    size_t len(size_t elem_bytes) { uint64_t v = u64(); if (!ok || v > (n - at) / (elem_bytes ? elem_bytes : 1) + 1) { ok = false; return 0; } return size_t(v); }
    EFElement ef() { EFElement e; for (auto& v : e) v = u32(); return e; }
    template <size_t N> void bytes(std::array<uint8_t, N>& a) { for (auto& b : a) b = u8(); }
    void vec_u32(std::vector<uint32_t>& v) { size_t k = len(4); v.clear(); for (size_t i = 0; i < k && ok; i++) v.push_back(u32()); }
    void vec_ef(std::vector<EFElement>& v) { size_t k = len(16); v.clear(); for (size_t i = 0; i < k && ok; i++) v.push_back(ef()); }

    void get(SumcheckProofEF& p) {
        size_t k = len(8);
        p.round_polys.clear();
        for (size_t i = 0; i < k && ok; i++) { p.round_polys.emplace_back(); vec_ef(p.round_polys.back()); }
        vec_ef(p.challenges);
    }
    void get(WeightCommitment& c) { bytes(c.root); c.num_weights = u64(); c.log_height = u64(); c.kind = u32(); }
    void get(MleEvalProofEF& p) { get(p.eval_sumcheck); p.eq_at_s = ef(); p.w_at_s = ef(); }
    void get(MatmulProofEF& p) { get(p.sumcheck_proof); p.w_at_rs = ef(); p.x_at_s = ef(); vec_ef(p.r_point); vec_ef(p.s_point); }
    void get(BatchMerkleProof& p) {
        vec_u32(p.indices); vec_u32(p.values);
        size_t k = len(8);
        p.auth_nodes.clear();
        for (size_t l = 0; l < k && ok; l++) {
            size_t cnt = len(16);
            std::vector<Digest> lv(cnt);
            for (auto& d : lv) bytes(d);
            p.auth_nodes.push_back(std::move(lv));
        }
    }
    void get(BasefoldOpeningProof& p) {
        size_t k = len(16);
        p.fold_roots.assign(k, Digest{});
        for (auto& d : p.fold_roots) bytes(d);
        size_t q = len(48);
        p.fold_queries.clear();
        for (size_t i = 0; i < q && ok; i++) { p.fold_queries.emplace_back(); get(p.fold_queries.back().prev_batch_proof); get(p.fold_queries.back().folded_batch_proof); }
        p.final_value = u32();
        vec_u32(p.final_coeffs);
    }
    void get(SuccinctMatmulProofEF& p) {
        get(p.matmul_proof); get(p.w_eval_proof); p.w_claimed_value = ef(); get(p.w_partial_commitment);
        p.bound = u8() != 0;
        uint8_t tag = u8();
        if (tag > 1) ok = false;
        p.has_basefold = tag == 1;
        if (p.has_basefold && ok) get(p.basefold_proof);
    }
    void get(HadamardProofEF& p) { get(p.product_sumcheck); p.fin_eq = ef(); p.fin_a = ef(); p.fin_b = ef(); p.c_eval = ef(); get(p.c_eval_proof); get(p.c_commitment); }
    void get(AddProofEF& p) {
        get(p.a_sumcheck); p.a_fin_eq = ef(); p.a_fin = ef(); get(p.b_sumcheck); p.b_fin_eq = ef(); p.b_fin = ef();
        p.c_eval = ef(); get(p.c_eval_proof); get(p.c_commitment);
    }
    void get(RmsNormProofEF& p) {
        p.perturbation_delta = int32_t(u32());
        get(p.var_proof); p.var_fin_a = ef(); p.var_fin_b = ef(); p.sum_sq_value = u32();
        get(p.h_sq_proof); for (auto& e : p.h_sq_fin) e = ef(); p.s_h = ef();
        get(p.g_sq_proof); for (auto& e : p.g_sq_fin) e = ef(); p.s_g = ef();
        get(p.g_prod_proof); for (auto& e : p.g_prod_fin) e = ef();
        get(p.g_triple_proof); for (auto& e : p.g_triple_fin) e = ef(); p.t_g_claimed = ef();
        get(p.x_commitment); get(p.gamma_commitment); get(p.g_commitment); get(p.h_commitment);
        get(p.x_var_eval_proof); p.x_at_var_s = ef();
        get(p.g_prod_eval_proof); p.g_at_prod_s = ef();
        get(p.x_triple_eval_proof); p.x_at_triple_s = ef();
        get(p.gamma_triple_eval_proof); p.gamma_at_triple_s = ef();
        get(p.h_sq_eval_proof); p.h_at_sq_s = ef();
        get(p.g_sq_eval_proof); p.g_at_gsq_s = ef();
    }
    void get(LookupProofEF& p) {
        get(p.table_commitment); get(p.multiplicity_commitment); get(p.sumcheck_proof); p.h_at_s = ef();
        for (int k = 0; k < 2; k++) { uint8_t tag = u8(); if (tag == 1) ef(); else if (tag != 0) ok = false; }
        vec_u32(p.inputs); vec_u32(p.outputs); vec_u32(p.multiplicities);
        bytes(p.external_data_digest);
    }
    void get(GateProofEF& p) { get(p.lookup_proof); get(p.hadamard_proof); }
    void get(RowAttentionProof& a) {
        uint64_t rows = u64();
        if (rows != 0) ok = false;                      // row proofs exist only for seq_len > 1
        a.num_heads = u64(); a.seq_len = u64(); a.d_head = u64();
        if (u8() != 1) ok = false;
        a.attn_out_at_r = u32(); a.v_at_r = u32(); a.is_gqa = u8() != 0;
    }
    bool get(QwenLayerProofEF& p) {
        get(p.norm1_proof); get(p.q_proof); get(p.k_proof); get(p.v_proof); get(p.attn_proof);
        get(p.o_proj_proof); get(p.g_proj_proof); get(p.sigmoid_gate_proof); get(p.residual1_proof); get(p.norm2_proof);
        get(p.gate_proj_proof); get(p.up_proj_proof); get(p.swiglu_proof); get(p.down_proj_proof); get(p.residual2_proof);
        QwenLayerCommitments& cm = p.commitments;
        for (WeightCommitment* k : {&cm.w_q, &cm.w_k, &cm.w_v, &cm.w_o, &cm.w_g_proj, &cm.w_gate, &cm.w_up, &cm.w_down}) get(*k);
        return ok && at == n;
    }
};

}  // namespace zko
