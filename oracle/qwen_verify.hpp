// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// verify_qwen_layer_ef_indexed (rust/zk_ml_prover/src/transformer/qwen.rs:932-1097) and the
// bincode image of QwenLayerProofEF (qwen.rs:711-737), RowAttentionProof (attention.rs:81-95).
#pragma once
#include "qwen.hpp"

namespace zko {

inline bool verify_qwen_layer_ef(const QwenLayerProofEF& p, const VF& x, const VF& y, const QwenLayerWeights& w,
                                 const ModelConfig& c, const LookupTable& silu, const LookupTable& sigmoid, Transcript& tr) {
    size_t d_model = c.d_model, d_ff = c.d_ff, aod = c.attn_out_dim();
    QwenForwardTrace t = qwen_forward(x, w, c, silu, sigmoid);
    if (t.output.size() != y.size()) return false;
    for (size_t i = 0; i < y.size(); i++) if (t.output[i] != y[i]) return false;
    absorb_qwen_dims(c, tr);
    const QwenLayerCommitments& cm = p.commitments;
    for (const WeightCommitment* k : {&cm.w_q, &cm.w_k, &cm.w_v, &cm.w_o, &cm.w_g_proj, &cm.w_gate, &cm.w_up, &cm.w_down})
        tr.absorb_bytes(k->root);
    if (!verify_rmsnorm_ef(p.norm1_proof, t.norm1_out, d_model, tr)) return false;
    if (!verify_matmul_succinct_ef(p.q_proof, t.q, c.q_dim(), d_model, tr).valid) return false;
    if (!verify_matmul_succinct_ef(p.k_proof, t.k, c.k_dim(), d_model, tr).valid) return false;
    if (!verify_matmul_succinct_ef(p.v_proof, t.v, c.v_dim(), d_model, tr).valid) return false;
    {
        size_t log_attn = log2_ceil(aod);
        VF r_attn = tr.squeeze_many(log_attn), r_v;
        F a = mle_evaluate(padded(t.attn_out, size_t(1) << log_attn), r_attn);
        seq1_points(c, r_attn, r_v);
        F v = mle_evaluate(padded(t.v, size_t(1) << log2_ceil(c.v_dim())), r_v);
        if (p.attn_proof.attn_out_at_r != a.v || p.attn_proof.v_at_r != v.v) return false;
        if (!p.attn_proof.is_gqa && p.attn_proof.attn_out_at_r != p.attn_proof.v_at_r) return false;
        tr.absorb(p.attn_proof.attn_out_at_r); tr.absorb(p.attn_proof.v_at_r);
    }
    if (!verify_matmul_succinct_ef(p.o_proj_proof, t.gated_out, d_model, aod, tr).valid) return false;
    if (!verify_matmul_succinct_ef(p.g_proj_proof, t.g_proj_out_raw, aod, d_model, tr).valid) return false;
    if (!verify_gate_ef_with_data(p.sigmoid_gate_proof, aod, t.g_proj_out, t.g_proj_sigmoid, tr)) return false;
    size_t log_d = log2_ceil(d_model);
    VEF res1 = tr.squeeze_ef_many(log_d);
    if (!verify_add_ef(p.residual1_proof, res1, tr)) return false;
    if (!verify_rmsnorm_ef(p.norm2_proof, t.norm2_out, d_model, tr)) return false;
    if (!verify_matmul_succinct_ef(p.gate_proj_proof, t.gate_out_raw, d_ff, d_model, tr).valid) return false;
    if (!verify_matmul_succinct_ef(p.up_proj_proof, t.up_out, d_ff, d_model, tr).valid) return false;
    if (!verify_gate_ef_with_data(p.swiglu_proof, d_ff, t.gate_out, t.gate_silu, tr)) return false;
    if (!verify_matmul_succinct_ef(p.down_proj_proof, t.down_out, d_model, d_ff, tr).valid) return false;
    VEF res2 = tr.squeeze_ef_many(log_d);
    return verify_add_ef(p.residual2_proof, res2, tr);
}

inline void put_attn(Bin& b, const RowAttentionProof& a) {
    b.u64(0);   // row_proofs: empty at seq_len = 1
    b.u64(a.num_heads); b.u64(a.seq_len); b.u64(a.d_head);
    b.u8(1); b.u32(a.attn_out_at_r); b.u32(a.v_at_r); b.u8(a.is_gqa ? 1 : 0);
}
inline std::vector<uint8_t> serialize(const QwenLayerProofEF& p) {
    Bin b;
    b.put(p.norm1_proof);
    b.put(p.q_proof); b.put(p.k_proof); b.put(p.v_proof);
    put_attn(b, p.attn_proof);
    b.put(p.o_proj_proof); b.put(p.g_proj_proof);
    b.put(p.sigmoid_gate_proof);
    b.put(p.residual1_proof);
    b.put(p.norm2_proof);
    b.put(p.gate_proj_proof); b.put(p.up_proj_proof);
    b.put(p.swiglu_proof);
    b.put(p.down_proj_proof);
    b.put(p.residual2_proof);
    const QwenLayerCommitments& cm = p.commitments;
    for (const WeightCommitment* k : {&cm.w_q, &cm.w_k, &cm.w_v, &cm.w_o, &cm.w_g_proj, &cm.w_gate, &cm.w_up, &cm.w_down}) b.put(*k);
    return b.b;
}

}  // namespace zko
