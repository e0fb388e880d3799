// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Row-decomposed attention for seq_len >= 2 (rust/zk_ml_prover/src/proving/attention.rs:25-42, 116-276)
// with the softmax proof it contains (rust/zk_ml_prover/src/proving/softmax.rs:20-131) and the plain
// matmul proof / verifier (matmul.rs:134-263).  Every (head, row) has a transcript of its own, labelled
// "row-attn-h{h}-r{i}"; the caller's transcript absorbs the dimensions first and, after all rows, every
// row's scores and outputs.  The reference pins these with prove -> verify round trips
// (attention.rs tests, softmax.rs tests), repeated on this restatement.
#pragma once
#include "bincode.hpp"
#include "matmul.hpp"

namespace zko {

// softmax.rs:20-43
struct SoftmaxProof {
    LookupProof exp_lookup_proof;
    uint32_t sum_value = 0;
    SumcheckProof sum_proof;
    uint32_t sum_finals[2] = {0, 0};
    SumcheckProof output_proof;
    uint32_t output_finals[3] = {0, 0, 0};
    uint32_t inv_s = 0;
    std::vector<uint32_t> e_values, y_values;
};
// softmax.rs:56-131
inline SoftmaxProof prove_softmax(const VF& z, const VF& e, const VF& y, const LookupTable& exp_table, Transcript& tr) {
    size_t n = z.size();
    SoftmaxProof p;
    p.exp_lookup_proof = prove_lookup(exp_table, z, e, tr);
    F sum = F::zero();
    for (F v : e) sum += v;
    p.sum_value = sum.v;
    size_t log_n = log2_ceil(n), n_pad = size_t(1) << log_n;
    VF e_pad = padded(e, n_pad), y_pad = padded(y, n_pad);
    tr.absorb(p.sum_value);
    VF ones(n_pad, F::one());
    Prod sp = prove_product(ones, e_pad, log_n, tr);
    p.sum_proof = sp.proof;
    p.sum_finals[0] = sp.f_at_s.v; p.sum_finals[1] = sp.g_at_s.v;
    VF r_point = tr.squeeze_many(log_n);
    VF eq_r = eq_evals(r_point);
    VF s_expanded(n_pad, sum);
    Trip op = prove_triple(eq_r, y_pad, s_expanded, log_n, tr);
    p.output_proof = op.proof;
    p.output_finals[0] = op.f_at_s.v; p.output_finals[1] = op.g_at_s.v; p.output_finals[2] = op.h_at_s.v;
    p.inv_s = inverse(sum).v;
    for (F v : e) p.e_values.push_back(v.v);
    for (F v : y) p.y_values.push_back(v.v);
    return p;
}
// softmax.rs:139-238
inline bool verify_softmax(const SoftmaxProof& p, size_t num_elements, Transcript& tr) {
    if (!verify_lookup(p.exp_lookup_proof, num_elements, tr)) return false;
    if (p.e_values.size() != p.exp_lookup_proof.outputs.size()) return false;
    for (size_t i = 0; i < p.e_values.size(); i++) if (p.e_values[i] != p.exp_lookup_proof.outputs[i]) return false;
    F sum(p.sum_value), inv_s(p.inv_s);
    if (inv_s * sum != F::one()) return false;
    size_t log_n = log2_ceil(num_elements), n_pad = size_t(1) << log_n;
    tr.absorb(p.sum_value);
    F ones_at_s(p.sum_finals[0]), e_at_s(p.sum_finals[1]);
    if (p.sum_proof.round_polys.size() != log_n) return false;
    if (!verify_product(sum, p.sum_proof, ones_at_s, e_at_s, tr)) return false;                 // softmax.rs:183
    if (ones_at_s != F::one()) return false;
    VF r_point = tr.squeeze_many(log_n);
    VF e_vals;
    for (uint32_t v : p.e_values) e_vals.push_back(F(v));
    F e_at_r = mle_evaluate(padded(e_vals, n_pad), r_point);
    F eq_at_s2(p.output_finals[0]), y_at_s2(p.output_finals[1]), s_at_s2(p.output_finals[2]);
    if (p.output_proof.round_polys.size() != log_n) return false;
    for (auto& rp : p.output_proof.round_polys) if (rp.size() < 4) return false;
    if (!verify_triple(e_at_r, p.output_proof, eq_at_s2, y_at_s2, s_at_s2, tr)) return false;   // softmax.rs:213
    VF s_point;
    for (uint32_t v : p.output_proof.challenges) s_point.push_back(F(v));
    if (compute_eq_at_point(r_point, s_point) != eq_at_s2) return false;
    return s_at_s2 == sum;
}

// matmul.rs:183-263: the verifier holds W and checks W(r, s) itself
inline bool verify_matmul(const MatmulProof& p, const VF& w, const VF& y, size_t m, size_t n, Transcript& tr) {
    size_t log_m = log2_ceil(m), log_n = log2_ceil(n), m_pad = size_t(1) << log_m, n_pad = size_t(1) << log_n;
    VF y_pad = padded(y, m_pad);
    tr.absorb_many(y_pad);
    VF r = tr.squeeze_many(log_m);
    std::vector<uint32_t> r_raw;
    for (F v : r) r_raw.push_back(v.v);
    if (r_raw != p.r_point) return false;
    F claim = mle_evaluate(y_pad, r);
    F w_at_rs(p.w_at_rs), x_at_s(p.x_at_s);
    if (p.sumcheck_proof.round_polys.size() != log_n) return false;
    if (!verify_product(claim, p.sumcheck_proof, w_at_rs, x_at_s, tr)) return false;             // matmul.rs:227
    VF w_pad(m_pad * n_pad, F::zero());
    for (size_t i = 0; i < m; i++) for (size_t j = 0; j < n; j++) w_pad[i * n_pad + j] = w[i * n + j];
    VF point = r;
    for (uint32_t v : p.s_point) point.push_back(F(v));
    if (point.size() != log_m + log_n) return false;
    return mle_evaluate(w_pad, point) == w_at_rs;
}

// attention.rs:25-42
struct RowProof {
    MatmulProof score_proof;
    SoftmaxProof softmax_proof;
    MatmulProof output_proof;
    std::vector<uint32_t> scores, attn_weights, output;
};
// The table's input -> output map as a flat array over the 16-bit (or 8-bit) raw index (attention.rs:131-135 builds a HashMap).
inline uint32_t exp_lookup(const LookupTable& t, F s, bool* ok) {
    size_t idx = field_to_table_index(s.v, t.inputs.size());
    if (idx >= t.inputs.size()) { *ok = false; return 0; }
    return t.outputs[idx];
}
// One row of attention.rs:160-262: k_head, v_head are seq_len x d_head, q_row has d_head entries.
inline RowProof prove_attention_row(size_t h, size_t i, const VF& k_head, const VF& v_head, const VF& q_row, size_t seq_len, size_t d_head,
                                    const LookupTable& exp_table, bool* ok, const char* label = "row-attn-h") {
    Transcript tr(label + std::to_string(h) + "-r" + std::to_string(i));
    VF scores(seq_len, F::zero());
    for (size_t j = 0; j < seq_len; j++) { F acc = F::zero(); for (size_t l = 0; l < d_head; l++) acc += k_head[j * d_head + l] * q_row[l]; scores[j] = acc; }
    RowProof rp;
    rp.score_proof = prove_matmul(k_head, q_row, scores, seq_len, d_head, tr, nullptr);
    VF e(seq_len), y(seq_len);
    F sum = F::zero();
    for (size_t j = 0; j < seq_len; j++) { e[j] = F(exp_lookup(exp_table, scores[j], ok)); sum += e[j]; }
    if (sum == F::zero()) *ok = false;                        // the reference's inverse() panics on zero
    if (!*ok) return rp;                                      // ... and on a score that is not a table input (attention.rs:105)
    F inv_s = inverse(sum);
    for (size_t j = 0; j < seq_len; j++) y[j] = e[j] * inv_s;
    rp.softmax_proof = prove_softmax(scores, e, y, exp_table, tr);
    VF v_t(d_head * seq_len, F::zero());
    for (size_t r = 0; r < seq_len; r++) for (size_t c = 0; c < d_head; c++) v_t[c * seq_len + r] = v_head[r * d_head + c];
    VF out_row(d_head, F::zero());
    for (size_t j = 0; j < d_head; j++) { F acc = F::zero(); for (size_t l = 0; l < seq_len; l++) acc += y[l] * v_head[l * d_head + j]; out_row[j] = acc; }
    rp.output_proof = prove_matmul(v_t, y, out_row, d_head, seq_len, tr, nullptr);
    for (F v : scores) rp.scores.push_back(v.v);
    for (F v : y) rp.attn_weights.push_back(v.v);
    for (F v : out_row) rp.output.push_back(v.v);
    return rp;
}
// One row of attention.rs:311-362
inline bool verify_attention_row(const RowProof& rp, size_t h, size_t i, const VF& k_head, const VF& v_head, size_t seq_len, size_t d_head,
                                 const char* label = "row-attn-h") {
    Transcript tr(label + std::to_string(h) + "-r" + std::to_string(i));
    VF scores, output;
    for (uint32_t v : rp.scores) scores.push_back(F(v));
    for (uint32_t v : rp.output) output.push_back(F(v));
    if (scores.size() != seq_len || output.size() != d_head) return false;
    if (!verify_matmul(rp.score_proof, k_head, scores, seq_len, d_head, tr)) return false;
    if (!verify_softmax(rp.softmax_proof, seq_len, tr)) return false;
    VF v_t(d_head * seq_len, F::zero());
    for (size_t r = 0; r < seq_len; r++) for (size_t c = 0; c < d_head; c++) v_t[c * seq_len + r] = v_head[r * d_head + c];
    return verify_matmul(rp.output_proof, v_t, output, d_head, seq_len, tr);
}


// attention.rs:90-98, :116-276: dimensions into the caller's transcript, independent rows, then every row's scores and outputs.
// (the reference's RowAttentionProof with seq1_consistency = None; the seq_len = 1 form of the same struct lives beside the layer prover)
struct SeqAttentionProof {
    std::vector<std::vector<RowProof>> row_proofs;
    size_t num_heads = 0, seq_len = 0, d_head = 0;
};
// num_kv_heads = 0: prove_row_attention.  Otherwise prove_row_attention_gqa (attention.rs:386-500): k, v have num_kv_heads heads, query
// head h reads K/V head h / (num_heads / num_kv_heads), the rows' labels are "gqa-h{h}-r{i}" and num_kv_heads is absorbed as well.
inline SeqAttentionProof prove_row_attention(const VF& q, const VF& k, const VF& v, size_t num_heads, size_t seq_len, size_t d_head,
                                             const LookupTable& exp_table, Transcript& tr, bool* ok, size_t num_kv_heads = 0) {
    size_t hs = seq_len * d_head;
    const size_t hpg = num_kv_heads ? num_heads / num_kv_heads : 1;
    const char* label = num_kv_heads ? "gqa-h" : "row-attn-h";
    tr.absorb(uint32_t(num_heads));
    if (num_kv_heads) tr.absorb(uint32_t(num_kv_heads));
    tr.absorb(uint32_t(seq_len)); tr.absorb(uint32_t(d_head));
    SeqAttentionProof P;
    P.num_heads = num_heads; P.seq_len = seq_len; P.d_head = d_head;
    P.row_proofs.resize(num_heads);
    for (size_t h = 0; h < num_heads; h++) {
        const size_t g = h / hpg;
        VF kh(k.begin() + g * hs, k.begin() + (g + 1) * hs), vh(v.begin() + g * hs, v.begin() + (g + 1) * hs);
        P.row_proofs[h].resize(seq_len);
        par_rows(seq_len, [&](size_t lo, size_t hi, int) {
            for (size_t i = lo; i < hi; i++) {
                VF qr(q.begin() + h * hs + i * d_head, q.begin() + h * hs + (i + 1) * d_head);
                bool row_ok = true;
                P.row_proofs[h][i] = prove_attention_row(h, i, kh, vh, qr, seq_len, d_head, exp_table, &row_ok, label);
                if (!row_ok) *ok = false;
            }
        });
    }
    for (auto& hp : P.row_proofs) for (auto& rp : hp) { for (uint32_t x : rp.scores) tr.absorb(x); for (uint32_t x : rp.output) tr.absorb(x); }
    return P;
}
// attention.rs:279-385 (and :503-590 with num_kv_heads)
inline bool verify_row_attention(const SeqAttentionProof& P, const VF& k, const VF& v, Transcript& tr, size_t num_kv_heads = 0) {
    size_t hs = P.seq_len * P.d_head;
    const size_t hpg = num_kv_heads ? P.num_heads / num_kv_heads : 1;
    const char* label = num_kv_heads ? "gqa-h" : "row-attn-h";
    tr.absorb(uint32_t(P.num_heads));
    if (num_kv_heads) tr.absorb(uint32_t(num_kv_heads));
    tr.absorb(uint32_t(P.seq_len)); tr.absorb(uint32_t(P.d_head));
    if (P.row_proofs.size() != P.num_heads) return false;
    for (size_t h = 0; h < P.num_heads; h++) {
        if (P.row_proofs[h].size() != P.seq_len) return false;
        const size_t g = h / hpg;
        VF kh(k.begin() + g * hs, k.begin() + (g + 1) * hs), vh(v.begin() + g * hs, v.begin() + (g + 1) * hs);
        for (size_t i = 0; i < P.seq_len; i++) if (!verify_attention_row(P.row_proofs[h][i], h, i, kh, vh, P.seq_len, P.d_head, label)) return false;
    }
    for (auto& hp : P.row_proofs) for (auto& rp : hp) { for (uint32_t x : rp.scores) tr.absorb(x); for (uint32_t x : rp.output) tr.absorb(x); }
    return true;
}
// The forward pass of the op (pipeline/forward.rs:233-276): out[h][i] = softmax_table(Q[h][i] K[h]^T) V[h].
inline VF row_attention_forward(const VF& q, const VF& k, const VF& v, size_t num_heads, size_t seq_len, size_t d_head, const LookupTable& t, bool* ok,
                                size_t num_kv_heads = 0) {
    size_t hs = seq_len * d_head;
    const size_t hpg = num_kv_heads ? num_heads / num_kv_heads : 1;
    VF out(num_heads * hs, F::zero());
    for (size_t h = 0; h < num_heads; h++) for (size_t i = 0; i < seq_len; i++) {
        const size_t g = h / hpg;
        VF e(seq_len);
        F sum = F::zero();
        for (size_t j = 0; j < seq_len; j++) {
            F acc = F::zero();
            for (size_t l = 0; l < d_head; l++) acc += k[g * hs + j * d_head + l] * q[h * hs + i * d_head + l];
            e[j] = F(exp_lookup(t, acc, ok)); sum += e[j];
        }
        if (sum == F::zero()) *ok = false;
        F inv_s = inverse(sum);
        for (size_t j = 0; j < d_head; j++) {
            F acc = F::zero();
            for (size_t l = 0; l < seq_len; l++) acc += e[l] * inv_s * v[g * hs + l * d_head + j];
            out[h * hs + i * d_head + j] = acc;
        }
    }
    return out;
}

inline void put(Bin& b, const SoftmaxProof& p) {           // softmax.rs:20-43
    b.put(p.exp_lookup_proof); b.u32(p.sum_value); b.put(p.sum_proof); b.u32(p.sum_finals[0]); b.u32(p.sum_finals[1]);
    b.put(p.output_proof); for (int i = 0; i < 3; i++) b.u32(p.output_finals[i]);
    b.u32(p.inv_s); b.vec_u32(p.e_values); b.vec_u32(p.y_values);
}
inline void put(Bin& b, const RowProof& p) {               // attention.rs:25-42
    b.put(p.score_proof); put(b, p.softmax_proof); b.put(p.output_proof);
    b.vec_u32(p.scores); b.vec_u32(p.attn_weights); b.vec_u32(p.output);
}
inline void put(Bin& b, const SeqAttentionProof& P) {      // attention.rs:82-98; seq1_consistency is None at seq_len >= 2
    b.u64(P.row_proofs.size());
    for (auto& hp : P.row_proofs) { b.u64(hp.size()); for (auto& rp : hp) put(b, rp); }
    b.u64(P.num_heads); b.u64(P.seq_len); b.u64(P.d_head); b.u8(0);
}

}  // namespace zko
