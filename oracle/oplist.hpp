// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// The op-list mode of the reference (MLP / GPT-2 shaped models, base-field challenges on one
// transcript "structured-ml-proof", ops proved in reverse order), restating
//   rust/zk_ml_prover/src/pipeline/forward.rs:24-520     forward pass of the ops used here
//   rust/zk_ml_prover/src/pipeline/prove.rs:36, 191-648  sequential prover
//   rust/zk_ml_prover/src/proving/layernorm.rs:445-916   LayerNormSqrProof, prove / verify
//   rust/zk_ml_prover/src/transformer/gpt2.rs:912-953    layernorm_forward_simple
//   rust/zk_ml_prover/src/protocol.rs:653-694            SerializedLayerProof (bincode variant order)
// Ops: linear (with bias), relu, layernorm, gelu (caller-supplied requantised pairs), attention at
// seq_len = 1 (pass-through), save, add_saved, set_input, passthrough.
#pragma once
#include "attention.hpp"
#include "qwen_verify.hpp"
#include <map>

namespace zko {

// ---- LayerNorm, squared form ------------------------------------------------------------------
struct LayerNormSqrProof {
    uint32_t mu = 0;
    SumcheckProof mean_check_proof; uint32_t mean_fin[2] = {0, 0};
    SumcheckProof var_proof;        uint32_t var_fin[2] = {0, 0};
    uint32_t sum_sq_value = 0;
    SumcheckProof g_prod_proof;     uint32_t g_prod_fin[2] = {0, 0};
    SumcheckProof g_triple_proof;   uint32_t g_triple_fin[3] = {0, 0, 0};
    uint32_t t_g_claimed = 0;
    SumcheckProof h_sq_proof;       uint32_t h_sq_fin[3] = {0, 0, 0};
    uint32_t s_h = 0;
    SumcheckProof g_sq_proof;       uint32_t g_sq_fin[3] = {0, 0, 0};
    uint32_t s_g = 0;
    WeightCommitment xc_commitment, gamma_commitment, g_commitment, h_commitment;
    MleEvalProof xc_mean_eval_proof;      uint32_t xc_at_mean_s = 0;
    MleEvalProof xc_var_eval_proof;       uint32_t xc_at_var_s = 0;
    MleEvalProof g_prod_eval_proof;       uint32_t g_at_prod_s = 0;
    MleEvalProof xc_triple_eval_proof;    uint32_t xc_at_triple_s = 0;
    MleEvalProof gamma_triple_eval_proof; uint32_t gamma_at_triple_s = 0;
    MleEvalProof h_sq_eval_proof;         uint32_t h_at_sq_s = 0;
    MleEvalProof g_sq_eval_proof;         uint32_t g_at_gsq_s = 0;
};

// gpt2.rs:912-953: the first perturbation 0, +1, -1, +2, ... of x[0] for which d / sum (x - mu)^2 is
// a quadratic residue; returns (y, mu, r, perturbation).
struct LnForward { VF y; F mu, r; int32_t perturbation = 0; };
inline LnForward layernorm_forward_simple(const VF& x, const VF& gamma, const VF& beta) {
    const size_t d = x.size();
    const F d_field = F(uint32_t(d)), d_inv = inverse(d_field);
    for (int32_t delta = 0; delta < 100; delta++) {
        for (int32_t sign : {1, -1}) {
            const int32_t pert = delta == 0 ? 0 : delta * sign;
            VF xp = x;
            if (pert != 0) xp[0] = xp[0] + (pert > 0 ? F(uint32_t(pert)) : F::zero() - F(uint32_t(-pert)));
            F sum_x;
            for (F v : xp) sum_x += v;
            const F mu = sum_x * d_inv;
            F sum_sq;
            for (F v : xp) sum_sq += (v - mu) * (v - mu);
            if (sum_sq == F::zero()) continue;          // (the reference `continue`s here too, without the delta == 0 break)
            const F target = d_field * inverse(sum_sq);
            if (is_qr_m31(target)) {
                LnForward o;
                o.mu = mu; o.r = mod_sqrt_m31(target); o.perturbation = pert;
                o.y.resize(d);
                for (size_t i = 0; i < d; i++) o.y[i] = gamma[i] * (xp[i] - mu) * o.r + beta[i];
                return o;
            }
            if (delta == 0) break;
        }
    }
    throw ForwardFailure("layernorm_forward_simple: could not find QR perturbation in 200 attempts");
}

// layernorm.rs:522-695
inline LayerNormSqrProof prove_layernorm_sqr(const VF& x, const VF& gamma, const VF& beta, const VF& y, F mu, Transcript& tr) {
    const size_t d = x.size(), log_n = log2_ceil(d), n_pad = size_t(1) << log_n;
    VF gamma_pad = padded(gamma, n_pad), xc_pad(n_pad, F::zero()), g_pad(n_pad, F::zero()), h_pad(n_pad, F::zero());
    for (size_t i = 0; i < d; i++) {
        xc_pad[i] = x[i] - mu;
        g_pad[i] = gamma_pad[i] * xc_pad[i];
        h_pad[i] = y[i] - beta[i];
    }
    F sum_sq;
    for (F v : xc_pad) sum_sq += v * v;
    LayerNormSqrProof p;
    p.mu = mu.v;
    p.sum_sq_value = sum_sq.v;
    p.xc_commitment = commit_weights_fast(xc_pad);
    p.gamma_commitment = commit_weights_fast(gamma_pad);
    p.g_commitment = commit_weights_fast(g_pad);
    p.h_commitment = commit_weights_fast(h_pad);
    tr.absorb_bytes(p.xc_commitment.root); tr.absorb_bytes(p.gamma_commitment.root);
    tr.absorb_bytes(p.g_commitment.root); tr.absorb_bytes(p.h_commitment.root);
    tr.absorb(mu.v);
    tr.absorb(sum_sq.v);
    // step 1: sum xc = 0
    tr.squeeze_many(log_n);
    VF ones(n_pad, F::one());
    Prod mc = prove_product(ones, xc_pad, log_n, tr);
    p.mean_check_proof = mc.proof; p.mean_fin[0] = mc.f_at_s.v; p.mean_fin[1] = mc.g_at_s.v;
    VF s_mean = base_points_of(mc.proof.challenges);
    p.xc_at_mean_s = mle_evaluate(xc_pad, s_mean).v;
    p.xc_mean_eval_proof = prove_mle_eval_bound(xc_pad, s_mean, "lnsqr-xc-mean", p.xc_commitment, tr);
    // step 2: sum xc^2 = sum_sq
    Prod var = prove_product(xc_pad, xc_pad, log_n, tr);
    p.var_proof = var.proof; p.var_fin[0] = var.f_at_s.v; p.var_fin[1] = var.g_at_s.v;
    VF s_var = base_points_of(var.proof.challenges);
    p.xc_at_var_s = mle_evaluate(xc_pad, s_var).v;
    p.xc_var_eval_proof = prove_mle_eval_bound(xc_pad, s_var, "lnsqr-xc-var", p.xc_commitment, tr);
    // step 3: g consistency
    VF gc_point = tr.squeeze_many(log_n);
    VF eq_gc = eq_evals(gc_point);
    F t_g;
    for (size_t i = 0; i < n_pad; i++) t_g += eq_gc[i] * g_pad[i];
    Prod gp = prove_product(eq_gc, g_pad, log_n, tr);
    p.g_prod_proof = gp.proof; p.g_prod_fin[0] = gp.f_at_s.v; p.g_prod_fin[1] = gp.g_at_s.v;
    VF s_gp = base_points_of(gp.proof.challenges);
    p.g_at_prod_s = mle_evaluate(g_pad, s_gp).v;
    p.g_prod_eval_proof = prove_mle_eval_bound(g_pad, s_gp, "lnsqr-g-prod", p.g_commitment, tr);
    Trip gt = prove_triple(eq_gc, gamma_pad, xc_pad, log_n, tr);
    p.g_triple_proof = gt.proof;
    p.g_triple_fin[0] = gt.f_at_s.v; p.g_triple_fin[1] = gt.g_at_s.v; p.g_triple_fin[2] = gt.h_at_s.v;
    p.t_g_claimed = t_g.v;
    VF s_gt = base_points_of(gt.proof.challenges);
    p.xc_at_triple_s = mle_evaluate(xc_pad, s_gt).v;
    p.xc_triple_eval_proof = prove_mle_eval_bound(xc_pad, s_gt, "lnsqr-xc-triple", p.xc_commitment, tr);
    p.gamma_at_triple_s = mle_evaluate(gamma_pad, s_gt).v;
    p.gamma_triple_eval_proof = prove_mle_eval_bound(gamma_pad, s_gt, "lnsqr-gamma-triple", p.gamma_commitment, tr);
    // step 4: squared checks
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
    p.h_sq_eval_proof = prove_mle_eval_bound(h_pad, s_hs, "lnsqr-h-sq", p.h_commitment, tr);
    for (size_t i = 0; i < n_pad; i++) s_g += eq_sq[i] * g_pad[i] * g_pad[i];
    Trip gs = prove_triple(eq_sq, g_pad, g_pad, log_n, tr);
    p.g_sq_proof = gs.proof;
    p.g_sq_fin[0] = gs.f_at_s.v; p.g_sq_fin[1] = gs.g_at_s.v; p.g_sq_fin[2] = gs.h_at_s.v;
    p.s_g = s_g.v;
    VF s_gs = base_points_of(gs.proof.challenges);
    p.g_at_gsq_s = mle_evaluate(g_pad, s_gs).v;
    p.g_sq_eval_proof = prove_mle_eval_bound(g_pad, s_gs, "lnsqr-g-sq", p.g_commitment, tr);
    return p;
}

// layernorm.rs:698-916
inline bool verify_layernorm_sqr(const LayerNormSqrProof& p, const VF& y, const VF& beta, size_t d, Transcript& tr) {
    const size_t log_n = log2_ceil(d), n_pad = size_t(1) << log_n;
    const F sum_sq(p.sum_sq_value), d_field = F(uint32_t(d));
    tr.absorb_bytes(p.xc_commitment.root); tr.absorb_bytes(p.gamma_commitment.root);
    tr.absorb_bytes(p.g_commitment.root); tr.absorb_bytes(p.h_commitment.root);
    tr.absorb(p.mu);
    tr.absorb(p.sum_sq_value);
    tr.squeeze_many(log_n);
    if (!verify_product_with_challenges(F::zero(), p.mean_check_proof, F(p.mean_fin[0]), F(p.mean_fin[1]), tr)) return false;
    if (p.mean_fin[0] != 1 || p.xc_at_mean_s != p.mean_fin[1]) return false;
    VF s_mean = base_points_of(p.mean_check_proof.challenges);
    if (!verify_mle_eval_bound(p.xc_commitment, F(p.xc_at_mean_s), s_mean, p.xc_mean_eval_proof, "lnsqr-xc-mean", tr)) return false;
    if (!verify_product_with_challenges(sum_sq, p.var_proof, F(p.var_fin[0]), F(p.var_fin[1]), tr)) return false;
    if (p.var_fin[0] != p.var_fin[1] || p.xc_at_var_s != p.var_fin[0]) return false;
    VF s_var = base_points_of(p.var_proof.challenges);
    if (!verify_mle_eval_bound(p.xc_commitment, F(p.xc_at_var_s), s_var, p.xc_var_eval_proof, "lnsqr-xc-var", tr)) return false;
    VF gc_point = tr.squeeze_many(log_n);
    const F t_g(p.t_g_claimed);
    if (!verify_product_with_challenges(t_g, p.g_prod_proof, F(p.g_prod_fin[0]), F(p.g_prod_fin[1]), tr)) return false;
    VF s_gp = base_points_of(p.g_prod_proof.challenges);
    if (compute_eq_at_point(gc_point, s_gp) != F(p.g_prod_fin[0]) || p.g_at_prod_s != p.g_prod_fin[1]) return false;
    if (!verify_mle_eval_bound(p.g_commitment, F(p.g_at_prod_s), s_gp, p.g_prod_eval_proof, "lnsqr-g-prod", tr)) return false;
    if (!verify_triple_with_challenges(t_g, p.g_triple_proof, F(p.g_triple_fin[0]), F(p.g_triple_fin[1]), F(p.g_triple_fin[2]), tr)) return false;
    VF s_gt = base_points_of(p.g_triple_proof.challenges);
    if (compute_eq_at_point(gc_point, s_gt) != F(p.g_triple_fin[0]) || p.xc_at_triple_s != p.g_triple_fin[2]) return false;
    if (!verify_mle_eval_bound(p.xc_commitment, F(p.xc_at_triple_s), s_gt, p.xc_triple_eval_proof, "lnsqr-xc-triple", tr)) return false;
    if (p.gamma_at_triple_s != p.g_triple_fin[1]) return false;
    if (!verify_mle_eval_bound(p.gamma_commitment, F(p.gamma_at_triple_s), s_gt, p.gamma_triple_eval_proof, "lnsqr-gamma-triple", tr)) return false;
    VF sq_point = tr.squeeze_many(log_n);
    const F s_h(p.s_h), s_g(p.s_g);
    if (!verify_triple_with_challenges(s_h, p.h_sq_proof, F(p.h_sq_fin[0]), F(p.h_sq_fin[1]), F(p.h_sq_fin[2]), tr)) return false;
    VF s_hs = base_points_of(p.h_sq_proof.challenges);
    if (compute_eq_at_point(sq_point, s_hs) != F(p.h_sq_fin[0])) return false;
    if (p.h_sq_fin[1] != p.h_sq_fin[2] || p.h_at_sq_s != p.h_sq_fin[1]) return false;
    if (!verify_mle_eval_bound(p.h_commitment, F(p.h_at_sq_s), s_hs, p.h_sq_eval_proof, "lnsqr-h-sq", tr)) return false;
    VF h_expected(n_pad, F::zero());
    for (size_t i = 0; i < d; i++) h_expected[i] = y[i] - beta[i];
    if (commit_weights_fast(h_expected).root != p.h_commitment.root) return false;
    if (!verify_triple_with_challenges(s_g, p.g_sq_proof, F(p.g_sq_fin[0]), F(p.g_sq_fin[1]), F(p.g_sq_fin[2]), tr)) return false;
    VF s_gs = base_points_of(p.g_sq_proof.challenges);
    if (compute_eq_at_point(sq_point, s_gs) != F(p.g_sq_fin[0])) return false;
    if (p.g_sq_fin[1] != p.g_sq_fin[2] || p.g_at_gsq_s != p.g_sq_fin[1]) return false;
    if (!verify_mle_eval_bound(p.g_commitment, F(p.g_at_gsq_s), s_gs, p.g_sq_eval_proof, "lnsqr-g-sq", tr)) return false;
    return sum_sq * s_h == d_field * s_g;
}

// bincode of LayerNormSqrProof in serde field order (layernorm.rs:468-519)
inline void put_lnsqr(Bin& o, const LayerNormSqrProof& p) {
    o.u32(p.mu);
    o.put(p.mean_check_proof); o.u32(p.mean_fin[0]); o.u32(p.mean_fin[1]);
    o.put(p.var_proof); o.u32(p.var_fin[0]); o.u32(p.var_fin[1]); o.u32(p.sum_sq_value);
    o.put(p.g_prod_proof); o.u32(p.g_prod_fin[0]); o.u32(p.g_prod_fin[1]);
    o.put(p.g_triple_proof); for (uint32_t v : p.g_triple_fin) o.u32(v);
    o.u32(p.t_g_claimed);
    o.put(p.h_sq_proof); for (uint32_t v : p.h_sq_fin) o.u32(v);
    o.u32(p.s_h);
    o.put(p.g_sq_proof); for (uint32_t v : p.g_sq_fin) o.u32(v);
    o.u32(p.s_g);
    o.put(p.xc_commitment); o.put(p.gamma_commitment); o.put(p.g_commitment); o.put(p.h_commitment);
    o.put(p.xc_mean_eval_proof); o.u32(p.xc_at_mean_s);
    o.put(p.xc_var_eval_proof); o.u32(p.xc_at_var_s);
    o.put(p.g_prod_eval_proof); o.u32(p.g_at_prod_s);
    o.put(p.xc_triple_eval_proof); o.u32(p.xc_at_triple_s);
    o.put(p.gamma_triple_eval_proof); o.u32(p.gamma_at_triple_s);
    o.put(p.h_sq_eval_proof); o.u32(p.h_at_sq_s);
    o.put(p.g_sq_eval_proof); o.u32(p.g_at_gsq_s);
}

// ---- the op list --------------------------------------------------------------------------------
struct Op {
    std::string type, name;
    size_t m = 0, n = 0;
    VF w, b;                    // linear
    VF gamma, beta;             // layernorm
    VF gelu_in, gelu_out;       // gelu: requantised (input, output) pairs as the caller supplies them
    std::vector<uint32_t> table_out;   // gelu: output column of the 65536- (or 256-) entry table
    std::string save_name, add_name;
    VF new_input;               // set_input
    size_t heads = 0, kv_heads = 0, seq = 0, d_head = 0;   // attention_rows (seq_len >= 2; kv_heads != 0: gqa_attention): table_out = the exp table, att_k / att_v when given by the request
    VF att_k, att_v;
};
struct LayerData {
    std::string type, name;
    const Op* op = nullptr;
    VF input, output;           // activation before / after the op
    VF pre_relu;
    LnForward ln; VF ln_x;
    VF att_q, att_k, att_v;
};
inline std::array<uint8_t, 32> hash_values(const VF& v) {     // common.rs:78-85
    std::vector<uint8_t> buf;
    uint32_t len = uint32_t(v.size());
    for (int i = 0; i < 4; i++) buf.push_back(uint8_t(len >> (8 * i)));
    for (F x : v) for (int i = 0; i < 4; i++) buf.push_back(uint8_t(x.v >> (8 * i)));
    return sha256(buf.data(), buf.size());
}

// forward.rs:24-520 for the ops above
inline std::vector<LayerData> oplist_forward(const std::vector<Op>& ops, const VF& input) {
    std::vector<LayerData> layers;
    std::map<std::string, VF> saved;
    VF cur = input;
    for (const Op& op : ops) {
        LayerData L;
        L.type = op.type; L.name = op.name; L.op = &op; L.input = cur;
        if (op.type == "linear") {
            VF y = matmul_forward(op.w, cur, op.m, op.n);       // the reference reads min(n, len) columns; lengths agree here
            for (size_t i = 0; i < op.m && i < op.b.size(); i++) y[i] += op.b[i];
            cur = y;
        } else if (op.type == "relu") {
            L.pre_relu = cur;
            for (F& v : cur) if (from_field(v) < 0) v = F::zero();
        } else if (op.type == "gelu") {
            cur = op.gelu_out;
        } else if (op.type == "layernorm") {
            L.ln = layernorm_forward_simple(cur, op.gamma, op.beta);
            L.ln_x = cur;
            if (L.ln.perturbation != 0) {
                int32_t pt = L.ln.perturbation;
                L.ln_x[0] = L.ln_x[0] + (pt > 0 ? F(uint32_t(pt)) : F::zero() - F(uint32_t(-pt)));
            }
            cur = L.ln.y;
        } else if (op.type == "attention") {                   // seq_len = 1: softmax of one score is 1, the output is V
            size_t third = cur.size() / 3;
            cur = VF(cur.begin() + 2 * third, cur.end());
        } else if (op.type == "attention_rows") {              // forward.rs:202-306 (attention), :555-660 (gqa_attention) at seq_len >= 2
            size_t total = op.heads * op.seq * op.d_head, total_kv = (op.kv_heads ? op.kv_heads : op.heads) * op.seq * op.d_head;
            bool ext = !op.att_k.empty();
            if (ext ? cur.size() < total : (op.kv_heads ? cur.size() < total + 2 * total_kv : cur.size() != 3 * total))
                throw std::runtime_error("attention: activation length");
            L.att_q = VF(cur.begin(), cur.begin() + total);
            L.att_k = ext ? op.att_k : VF(cur.begin() + total, cur.begin() + total + total_kv);
            L.att_v = ext ? op.att_v : VF(cur.begin() + total + total_kv, cur.begin() + total + 2 * total_kv);
            bool ok = true;
            cur = row_attention_forward(L.att_q, L.att_k, L.att_v, op.heads, op.seq, op.d_head, table_from_outputs(op.table_out), &ok, op.kv_heads);
            if (!ok) throw std::runtime_error("attention: a score outside the exp table or a zero denominator");
        } else if (op.type == "save") {
            saved[op.save_name] = cur;
        } else if (op.type == "add_saved") {
            const VF& s = saved.at(op.add_name);
            for (size_t i = 0; i < cur.size(); i++) cur[i] += s[i];
        } else if (op.type == "set_input") {
            cur = op.new_input;
        } else if (op.type != "passthrough") {
            throw std::runtime_error("unknown op " + op.type);
        }
        L.output = cur;
        layers.push_back(std::move(L));
    }
    return layers;
}

// prove.rs:36, 191-648: bincode(Vec<SerializedLayerProof>), proofs pushed in reverse op order.
inline std::vector<uint8_t> oplist_prove(const std::vector<LayerData>& layers) {
    Transcript tr("structured-ml-proof");
    Bin out;
    size_t count = 0;
    Bin body;
    bool last_was_matmul = false;
    std::vector<uint32_t> last_s_point;
    auto tag = [&](uint32_t t) { body.u32(t); count++; };
    for (size_t idx = layers.size(); idx-- > 0;) {
        const LayerData& L = layers[idx];
        const Op& op = *L.op;
        if (L.type == "linear") {
            WeightCommitment wc = commit_weights_fast(op.w);
            tr.absorb_bytes(wc.root);
            SuccinctMatmulProof p = prove_matmul_succinct(op.w, L.input, L.output, op.m, op.n, tr);
            tag(0); body.put(p);
            last_was_matmul = true;
            last_s_point = p.matmul_proof.s_point;
            continue;
        }
        if (L.type == "relu") {
            const size_t log_n = log2_ceil(L.pre_relu.size()), n_pad = size_t(1) << log_n;
            VF z_pad = padded(L.pre_relu, n_pad), a_pad(n_pad), b_vals(n_pad), one_minus_b(n_pad);
            for (size_t i = 0; i < n_pad; i++) {
                const bool pos = from_field(z_pad[i]) >= 0;
                a_pad[i] = pos ? z_pad[i] : F::zero();
                b_vals[i] = pos ? F::one() : F::zero();
                one_minus_b[i] = F::one() - b_vals[i];
            }
            WeightCommitment ac = commit_weights_fast(a_pad);
            bool have_chain = false;
            MleEvalProof chain_proof;
            F chain_value;
            if (last_was_matmul) {
                chain_proof = prove_mle_eval_bound(a_pad, base_points_of(last_s_point), "relu-chain", ac, tr, &chain_value);
                have_chain = true;
            }
            tr.absorb_bytes(ac.root);
            VF r_point = tr.squeeze_many(log_n);
            F a_at_r = mle_evaluate(a_pad, r_point);
            MleEvalProof a_eval = prove_mle_eval_bound(a_pad, r_point, "relu-eval", ac, tr);
            Trip prod = prove_triple(eq_evals(r_point), b_vals, z_pad, log_n, tr);
            VF r2 = tr.squeeze_many(log_n);
            Trip boo = prove_triple(eq_evals(r2), b_vals, one_minus_b, log_n, tr);
            tag(1);
            body.put(ac); body.u32(a_at_r.v); body.put(a_eval);
            body.u8(have_chain ? 1 : 0); if (have_chain) body.put(chain_proof);
            body.u8(have_chain ? 1 : 0); if (have_chain) body.u32(chain_value.v);
            body.put(prod.proof); body.u32(prod.f_at_s.v); body.u32(prod.g_at_s.v); body.u32(prod.h_at_s.v);
            body.put(boo.proof); body.u32(boo.f_at_s.v); body.u32(boo.g_at_s.v); body.u32(boo.h_at_s.v);
            last_was_matmul = false;
            continue;
        }
        last_was_matmul = false;       // every other variant is not SerializedLayerProof::Matmul
        if (L.type == "layernorm") {
            LayerNormSqrProof p = prove_layernorm_sqr(L.ln_x, op.gamma, op.beta, L.ln.y, L.ln.mu, tr);
            tag(3); put_lnsqr(body, p);
        } else if (L.type == "gelu") {
            LookupProof p = prove_lookup(table_from_outputs(op.table_out), op.gelu_in, op.gelu_out, tr);
            tag(4); body.put(p);
        } else if (L.type == "attention_rows") {               // prove.rs:419-432
            bool ok = true;
            SeqAttentionProof p = prove_row_attention(L.att_q, L.att_k, L.att_v, op.heads, op.seq, op.d_head, table_from_outputs(op.table_out), tr, &ok,
                                                      op.kv_heads);
            tag(op.kv_heads ? 12 : 5); put(body, p);               // Attention / GqaAttention (prove.rs:419-432, 572-584)
        } else if (L.type == "attention" || L.type == "passthrough") {
            tr.absorb_bytes(hash_values(L.output));
            tag(16);
        } else if (L.type == "add_saved") {
            std::string save_layer = L.name;
            if (save_layer.rfind("add_", 0) == 0) save_layer = "save_" + save_layer.substr(4);      // replacen("add_", "save_", 1) on a name that starts with it
            else { size_t at = save_layer.find("add_"); if (at != std::string::npos) save_layer.replace(at, 4, "save_"); }
            tag(6); body.str(save_layer);
        } else if (L.type == "save") {
            auto h = hash_values(L.output);
            tr.absorb_bytes(h);
            tag(8); body.str(L.name); body.bytes(h);
        } else if (L.type == "set_input") {
            auto nh = hash_values(L.output);
            std::array<uint8_t, 32> ph{};
            if (idx > 0) ph = hash_values(layers[idx - 1].output);
            tr.absorb_bytes(ph);
            tr.absorb_bytes(nh);
            tag(7); body.bytes(ph); body.bytes(nh);
        }
    }
    out.u64(count);
    out.b.insert(out.b.end(), body.b.begin(), body.b.end());
    return out.b;
}

}  // namespace zko
