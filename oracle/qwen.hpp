// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Qwen3.5-style layer at seq_len = 1: forward trace, EF layer prover and verifier, restating
//   rust/zk_ml_prover/src/transformer/mod.rs:165-324  (compute_r, rmsnorm_forward, requantize)
//   rust/zk_ml_prover/src/transformer/qwen.rs:36-58, 211-325, 711-1097
//   rust/zk_ml_prover/src/pipeline/prove.rs:158-189 (per-layer transcript seed)
#pragma once
#include "bincode.hpp"

namespace zko {

// transformer/mod.rs:185-216 (fields used on this path)
struct ModelConfig {
    size_t d_model = 0, d_ff = 0, num_q_heads = 0, num_kv_heads = 0, d_head = 0, v_num_heads = 0, v_d_head = 0;
    size_t v_dim() const {
        size_t vh = v_num_heads == 0 ? num_kv_heads : v_num_heads;
        size_t vd = v_d_head == 0 ? d_head : v_d_head;
        return vh * vd;
    }
    size_t q_dim() const { return num_q_heads * d_head; }
    size_t k_dim() const { return num_kv_heads * d_head; }
    bool is_gqa() const { return num_q_heads != num_kv_heads; }
    size_t attn_out_dim() const { return is_gqa() ? q_dim() : v_dim(); }
};
// qwen.rs:62-73
struct QwenLayerWeights { VF norm1_gamma, w_q, w_k, w_v, w_o, w_g_proj, norm2_gamma, w_gate, w_up, w_down; };
struct QwenLayerCommitments { WeightCommitment w_q, w_k, w_v, w_o, w_g_proj, w_gate, w_up, w_down; };
// qwen.rs:148-161 (commit_weight_matrix hashes the unpadded matrix, transformer/mod.rs:353-357)
inline QwenLayerCommitments commit_qwen_layer(const QwenLayerWeights& w) {
    return {commit_weights_fast(w.w_q), commit_weights_fast(w.w_k), commit_weights_fast(w.w_v), commit_weights_fast(w.w_o),
            commit_weights_fast(w.w_g_proj), commit_weights_fast(w.w_gate), commit_weights_fast(w.w_up), commit_weights_fast(w.w_down)};
}

struct ForwardFailure : std::runtime_error { using std::runtime_error::runtime_error; };

// transformer/mod.rs:245-288
inline void rmsnorm_forward(const VF& x, const VF& gamma, VF& out, VF& x_used, int32_t& delta) {
    size_t d = x.size();
    F d_field = F(uint32_t(d));
    F sum_sq;
    for (F v : x) sum_sq += v * v;
    auto finish = [&](const VF& xs, F ssq) {
        F r = mod_sqrt_m31(d_field * inverse(ssq));
        out.resize(d);
        for (size_t i = 0; i < d; i++) out[i] = gamma[i] * xs[i] * r;
    };
    if (sum_sq != F::zero() && is_qr_m31(d_field * inverse(sum_sq))) { x_used = x; delta = 0; finish(x, sum_sq); return; }
    F x0 = x[0];
    for (int32_t dl = 1; dl < 100; dl++)
        for (int32_t sign : {1, -1}) {
            int32_t pert = dl * sign;
            F adj = pert > 0 ? F(uint32_t(pert)) : F::zero() - F(uint32_t(-pert));
            F nx0 = x0 + adj;
            F ssq = sum_sq - x0 * x0 + nx0 * nx0;
            if (ssq == F::zero()) continue;
            if (is_qr_m31(d_field * inverse(ssq))) {
                x_used = x; x_used[0] = nx0; delta = pert; finish(x_used, ssq); return;
            }
        }
    throw ForwardFailure("rmsnorm_forward: could not find QR perturbation in 200 attempts");
}

// transformer/mod.rs:293-324
inline VF requantize_to_i16_field(const VF& values) {
    uint64_t max_abs = 1;
    std::vector<int64_t> s(values.size());
    for (size_t i = 0; i < values.size(); i++) {
        s[i] = from_field(values[i]);
        uint64_t a = uint64_t(s[i] < 0 ? -s[i] : s[i]);
        if (a > max_abs) max_abs = a;
    }
    VF out(values.size());
    for (size_t i = 0; i < values.size(); i++) {
        int64_t v = s[i], scaled;
        if (max_abs <= 32767) scaled = v;
        else {
            int64_t half = int64_t(max_abs) / 2;
            scaled = v >= 0 ? (v * 32767 + half) / int64_t(max_abs) : (v * 32767 - half) / int64_t(max_abs);
        }
        if (scaled < -32768) scaled = -32768;
        if (scaled > 32767) scaled = 32767;
        out[i] = to_field(scaled);
    }
    return out;
}
inline F table_lookup(const LookupTable& t, F key) {
    size_t idx = field_to_table_index(key.v, t.inputs.size());
    if (idx >= t.inputs.size()) throw ForwardFailure("lookup_fast: key not found");
    return F(t.outputs[idx]);
}

// qwen.rs:163-192
struct QwenForwardTrace {
    VF x, norm1_x, norm1_out, q, k, v, attn_out, g_proj_out_raw, g_proj_out, g_proj_sigmoid, gated_out, h,
        norm2_x, norm2_out, gate_out_raw, gate_out, gate_silu, up_out, swiglu_out, down_out, output;
    int32_t norm1_delta = 0, norm2_delta = 0;
};
inline VF hadamard(const VF& a, const VF& b) { VF o(a.size()); for (size_t i = 0; i < a.size(); i++) o[i] = a[i] * b[i]; return o; }
inline VF vadd(const VF& a, const VF& b) { VF o(a.size()); for (size_t i = 0; i < a.size(); i++) o[i] = a[i] + b[i]; return o; }

// qwen.rs:211-325
inline QwenForwardTrace qwen_forward(const VF& x, const QwenLayerWeights& w, const ModelConfig& c,
                                     const LookupTable& silu, const LookupTable& sigmoid) {
    QwenForwardTrace t;
    t.x = x;
    rmsnorm_forward(x, w.norm1_gamma, t.norm1_out, t.norm1_x, t.norm1_delta);
    t.q = matmul_forward(w.w_q, t.norm1_out, c.q_dim(), c.d_model);
    t.k = matmul_forward(w.w_k, t.norm1_out, c.k_dim(), c.d_model);
    t.v = matmul_forward(w.w_v, t.norm1_out, c.v_dim(), c.d_model);
    t.g_proj_out_raw = matmul_forward(w.w_g_proj, t.norm1_out, c.attn_out_dim(), c.d_model);
    if (c.is_gqa()) {
        size_t per = c.num_q_heads / c.num_kv_heads;
        for (size_t h = 0; h < c.num_q_heads; h++)
            for (size_t d = 0; d < c.d_head; d++) t.attn_out.push_back(t.v[(h / per) * c.d_head + d]);
    } else t.attn_out = t.v;
    t.g_proj_out = requantize_to_i16_field(t.g_proj_out_raw);
    for (F v : t.g_proj_out) t.g_proj_sigmoid.push_back(table_lookup(sigmoid, v));
    VF gated_attn = hadamard(t.attn_out, t.g_proj_sigmoid);
    t.gated_out = matmul_forward(w.w_o, gated_attn, c.d_model, c.attn_out_dim());
    t.h = vadd(x, t.gated_out);
    rmsnorm_forward(t.h, w.norm2_gamma, t.norm2_out, t.norm2_x, t.norm2_delta);
    t.gate_out_raw = matmul_forward(w.w_gate, t.norm2_out, c.d_ff, c.d_model);
    t.up_out = matmul_forward(w.w_up, t.norm2_out, c.d_ff, c.d_model);
    t.gate_out = requantize_to_i16_field(t.gate_out_raw);
    for (F v : t.gate_out) t.gate_silu.push_back(table_lookup(silu, v));
    t.swiglu_out = hadamard(t.gate_silu, t.up_out);
    t.down_out = matmul_forward(w.w_down, t.swiglu_out, c.d_model, c.d_ff);
    t.output = vadd(t.h, t.down_out);
    return t;
}

// qwen.rs:36-58
inline void absorb_qwen_dims(const ModelConfig& c, Transcript& tr) {
    tr.absorb_bytes("qwen-dims-v1");
    for (size_t v : {c.d_model, c.d_ff, c.num_q_heads, c.num_kv_heads, c.d_head, c.v_num_heads, c.v_d_head, c.v_dim(),
                     c.q_dim(), c.k_dim(), c.attn_out_dim(), size_t(c.is_gqa() ? 1 : 0)})
        tr.absorb(uint32_t(v));
}

// attention.rs:69-95 (seq_len = 1 form)
struct RowAttentionProof { uint64_t num_heads = 0, seq_len = 1, d_head = 0; uint32_t attn_out_at_r = 0, v_at_r = 0; bool is_gqa = false; };

// qwen.rs:711-737
struct QwenLayerProofEF {
    RmsNormProofEF norm1_proof;
    SuccinctMatmulProofEF q_proof, k_proof, v_proof;
    RowAttentionProof attn_proof;
    SuccinctMatmulProofEF o_proj_proof, g_proj_proof;
    GateProofEF sigmoid_gate_proof;
    AddProofEF residual1_proof;
    RmsNormProofEF norm2_proof;
    SuccinctMatmulProofEF gate_proj_proof, up_proj_proof;
    GateProofEF swiglu_proof;
    SuccinctMatmulProofEF down_proj_proof;
    AddProofEF residual2_proof;
    QwenLayerCommitments commitments;
};

inline void seq1_points(const ModelConfig& c, const VF& r_attn, VF& r_v) {
    if (!c.is_gqa()) { r_v = r_attn; return; }
    size_t log_d = log2_ceil(c.d_head), log_kv = log2_ceil(c.num_kv_heads);
    r_v.assign(r_attn.begin(), r_attn.begin() + log_kv);
    r_v.insert(r_v.end(), r_attn.end() - log_d, r_attn.end());
}
inline void strip_matmul(SuccinctMatmulProofEF& p) {
    p.matmul_proof.r_point.clear(); p.matmul_proof.s_point.clear();
    p.matmul_proof.sumcheck_proof.challenges.clear(); p.w_eval_proof.eval_sumcheck.challenges.clear();
}
inline void strip_norm(RmsNormProofEF& n) {
    n.var_proof.challenges.clear(); n.g_prod_proof.challenges.clear(); n.g_triple_proof.challenges.clear();
    n.h_sq_proof.challenges.clear(); n.g_sq_proof.challenges.clear();
    for (MleEvalProofEF* e : {&n.x_var_eval_proof, &n.g_prod_eval_proof, &n.gamma_triple_eval_proof, &n.x_triple_eval_proof,
                              &n.h_sq_eval_proof, &n.g_sq_eval_proof}) e->eval_sumcheck.challenges.clear();
}
// qwen.rs:739-791
inline void strip_redundant(QwenLayerProofEF& p) {
    for (SuccinctMatmulProofEF* m : {&p.q_proof, &p.k_proof, &p.v_proof, &p.o_proj_proof, &p.g_proj_proof, &p.gate_proj_proof,
                                     &p.up_proj_proof, &p.down_proj_proof}) strip_matmul(*m);
    strip_norm(p.norm1_proof); strip_norm(p.norm2_proof);
    p.swiglu_proof.hadamard_proof.product_sumcheck.challenges.clear();
    p.sigmoid_gate_proof.hadamard_proof.product_sumcheck.challenges.clear();
    p.residual1_proof.a_sumcheck.challenges.clear(); p.residual1_proof.b_sumcheck.challenges.clear();
    p.residual2_proof.a_sumcheck.challenges.clear(); p.residual2_proof.b_sumcheck.challenges.clear();
    for (GateProofEF* g : {&p.swiglu_proof, &p.sigmoid_gate_proof}) {
        g->lookup_proof.sumcheck_proof.challenges.clear(); g->lookup_proof.inputs.clear(); g->lookup_proof.outputs.clear();
    }
}

// qwen.rs:795-912
inline QwenLayerProofEF prove_qwen_layer_precommitted_ef(const QwenForwardTrace& t, const QwenLayerWeights& w, const ModelConfig& c,
                                                         const QwenLayerCommitments& cm, const LookupTable& silu,
                                                         const LookupTable& sigmoid, Transcript& tr) {
    size_t d_model = c.d_model, d_ff = c.d_ff, aod = c.attn_out_dim();
    absorb_qwen_dims(c, tr);
    for (const WeightCommitment* k : {&cm.w_q, &cm.w_k, &cm.w_v, &cm.w_o, &cm.w_g_proj, &cm.w_gate, &cm.w_up, &cm.w_down})
        tr.absorb_bytes(k->root);
    QwenLayerProofEF p;
    p.commitments = cm;
    p.norm1_proof = prove_rmsnorm_ef(t.norm1_x, w.norm1_gamma, t.norm1_out, t.norm1_delta, tr);
    p.q_proof = prove_matmul_succinct_ef(w.w_q, t.norm1_out, t.q, c.q_dim(), d_model, tr);
    p.k_proof = prove_matmul_succinct_ef(w.w_k, t.norm1_out, t.k, c.k_dim(), d_model, tr);
    p.v_proof = prove_matmul_succinct_ef(w.w_v, t.norm1_out, t.v, c.v_dim(), d_model, tr);
    {
        size_t log_attn = log2_ceil(aod);
        VF r_attn = tr.squeeze_many(log_attn), r_v;
        F a = mle_evaluate(padded(t.attn_out, size_t(1) << log_attn), r_attn);
        seq1_points(c, r_attn, r_v);
        F v = mle_evaluate(padded(t.v, size_t(1) << log2_ceil(c.v_dim())), r_v);
        tr.absorb(a); tr.absorb(v);
        p.attn_proof = RowAttentionProof{c.num_q_heads, 1, c.d_head, a.v, v.v, c.is_gqa()};
    }
    VF gated_attn = hadamard(t.attn_out, t.g_proj_sigmoid);
    p.o_proj_proof = prove_matmul_succinct_ef(w.w_o, gated_attn, t.gated_out, d_model, aod, tr);
    p.g_proj_proof = prove_matmul_succinct_ef(w.w_g_proj, t.norm1_out, t.g_proj_out_raw, aod, d_model, tr);
    p.sigmoid_gate_proof = prove_sigmoid_gate_ef(t.g_proj_out, t.g_proj_sigmoid, t.attn_out, gated_attn, sigmoid, tr);
    size_t log_d = log2_ceil(d_model);
    VEF res1 = tr.squeeze_ef_many(log_d);
    p.residual1_proof = prove_add_ef(t.x, t.gated_out, t.h, res1, tr);
    p.norm2_proof = prove_rmsnorm_ef(t.norm2_x, w.norm2_gamma, t.norm2_out, t.norm2_delta, tr);
    p.gate_proj_proof = prove_matmul_succinct_ef(w.w_gate, t.norm2_out, t.gate_out_raw, d_ff, d_model, tr);
    p.up_proj_proof = prove_matmul_succinct_ef(w.w_up, t.norm2_out, t.up_out, d_ff, d_model, tr);
    p.swiglu_proof = prove_swiglu_ef(t.gate_out, t.gate_silu, t.up_out, t.swiglu_out, silu, tr);
    p.down_proj_proof = prove_matmul_succinct_ef(w.w_down, t.swiglu_out, t.down_out, d_model, d_ff, tr);
    VEF res2 = tr.squeeze_ef_many(log_d);
    p.residual2_proof = prove_add_ef(t.h, t.down_out, t.output, res2, tr);
    strip_redundant(p);
    return p;
}

}  // namespace zko
