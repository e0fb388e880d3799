// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Weight commitments and MLE-evaluation proofs, restating
// rust/zk_ml_prover/src/proving/weight_commitment.rs and derive_query_indices from
// rust/zk_ml_prover/src/proving/pcs.rs:442-451 (default build: no `pcs` feature).
#pragma once
#include "field.hpp"
#include "hash.hpp"
#include "mle.hpp"
#include "sumcheck.hpp"
#include "transcript.hpp"

namespace zko {

constexpr size_t NUM_QUERIES = 24;   // pcs.rs:19

// weight_commitment.rs:31-61
struct WeightCommitment {
    std::array<uint8_t, 32> root{};
    uint64_t num_weights = 0;
    uint64_t log_height = 0;
    uint32_t kind = 0;   // 0 = Blake3Fast, 1 = MerkleAesMmo
};

// weight_commitment.rs:82-107 — blake3("weights" || u32 LE buffer).
inline WeightCommitment commit_weights_fast(const VF& w) {
    std::vector<uint8_t> buf(7 + 4 * w.size());
    memcpy(buf.data(), "weights", 7);
    for (size_t i = 0; i < w.size(); i++) {
        uint32_t v = w[i].v;
        buf[7 + 4 * i] = uint8_t(v); buf[8 + 4 * i] = uint8_t(v >> 8);
        buf[9 + 4 * i] = uint8_t(v >> 16); buf[10 + 4 * i] = uint8_t(v >> 24);
    }
    WeightCommitment c;
    c.root = blake3(buf);
    c.num_weights = w.size();
    c.log_height = w.size() <= 1 ? 1 : log2_ceil(w.size());
    c.kind = 0;
    return c;
}

// pcs.rs:442-451 — 24 squeezes; the indices are unused outside Basefold.
inline std::vector<size_t> derive_query_indices(Transcript& tr, size_t log_n) {
    size_t n_pad = size_t(1) << log_n;
    std::vector<size_t> idx;
    for (size_t i = 0; i < NUM_QUERIES; i++) idx.push_back(size_t(tr.squeeze().v) % n_pad);
    return idx;
}

// weight_commitment.rs:65-73 (merkle_opening is always None on this path)
struct MleEvalProof {
    SumcheckProof eval_sumcheck;
    uint32_t eq_at_s = 0, w_at_s = 0;
};
// weight_commitment.rs:340-345
struct MleEvalProofEF {
    SumcheckProofEF eval_sumcheck;
    EFElement eq_at_s{}, w_at_s{};
};

inline VF padded(const VF& v, size_t n) { VF o = v; o.resize(n, F::zero()); return o; }
inline VEF padded(const VEF& v, size_t n) { VEF o = v; o.resize(n, EF::zero()); return o; }

// weight_commitment.rs:177-206 (prove_mle_eval_no_merkle); :248-274 (_with_claim_no_merkle) is
// the same transcript trace without returning the claim.
inline MleEvalProof prove_mle_eval_no_merkle(const VF& weights, const VF& point, Transcript& tr, F* claimed = nullptr) {
    size_t log_n = point.size(), n_pad = size_t(1) << log_n;
    VF w = padded(weights, n_pad);
    VF eq = eq_evals(point);
    if (claimed) *claimed = mle_evaluate(w, point);
    Prod r = prove_product(eq, w, log_n, tr);
    derive_query_indices(tr, log_n);
    MleEvalProof p;
    p.eval_sumcheck = r.proof; p.eq_at_s = r.f_at_s.v; p.w_at_s = r.g_at_s.v;
    return p;
}
// weight_commitment.rs:437-447
inline MleEvalProof prove_mle_eval_bound(const VF& w, const VF& point, const std::string& label,
                                         const WeightCommitment& c, Transcript& tr, F* claimed = nullptr) {
    tr.absorb_bytes(label);
    tr.absorb_bytes(c.root);
    return prove_mle_eval_no_merkle(w, point, tr, claimed);
}
// weight_commitment.rs:285-332
inline bool verify_mle_eval(F claimed, const VF& point, const MleEvalProof& p, Transcript& tr) {
    VF s;
    if (!verify_product_with_challenges(claimed, p.eval_sumcheck, F(p.eq_at_s), F(p.w_at_s), tr, &s)) return false;
    if (compute_eq_at_point(point, s) != F(p.eq_at_s)) return false;
    derive_query_indices(tr, point.size());
    return true;
}
// weight_commitment.rs:453-464
inline bool verify_mle_eval_bound(const WeightCommitment& c, F claimed, const VF& point, const MleEvalProof& p,
                                  const std::string& label, Transcript& tr) {
    tr.absorb_bytes(label);
    tr.absorb_bytes(c.root);
    return verify_mle_eval(claimed, point, p, tr);
}

// weight_commitment.rs:349-374
inline MleEvalProofEF prove_mle_eval_ef_with_claim_no_merkle(const VEF& weights, const VEF& point, Transcript& tr) {
    size_t log_n = point.size(), n_pad = size_t(1) << log_n;
    VEF w = padded(weights, n_pad);
    VEF eq = eq_evals_ef(point);
    ProdEF r = prove_product_ef_full(eq, w, log_n, tr);
    derive_query_indices(tr, log_n);
    MleEvalProofEF p;
    p.eval_sumcheck = r.proof; p.eq_at_s = r.f_at_s.arr(); p.w_at_s = r.g_at_s.arr();
    return p;
}
// weight_commitment.rs:470-502
inline MleEvalProofEF prove_mle_eval_no_merkle_ef_base(const VF& weights, const VEF& point, Transcript& tr, EF* claimed = nullptr) {
    size_t log_n = point.size(), n_pad = size_t(1) << log_n;
    VF w = padded(weights, n_pad);
    VEF eq = eq_evals_ef(point);
    if (claimed) *claimed = mle_evaluate_ef(w, point);
    ProdEF r = prove_product_ef_full(eq, widen(w), log_n, tr);
    derive_query_indices(tr, log_n);
    MleEvalProofEF p;
    p.eval_sumcheck = r.proof; p.eq_at_s = r.f_at_s.arr(); p.w_at_s = r.g_at_s.arr();
    return p;
}
// weight_commitment.rs:507-517
inline MleEvalProofEF prove_mle_eval_ef_base_bound(const VF& w, const VEF& point, const std::string& label,
                                                   const WeightCommitment& c, Transcript& tr, EF* claimed = nullptr) {
    tr.absorb_bytes(label);
    tr.absorb_bytes(c.root);
    return prove_mle_eval_no_merkle_ef_base(w, point, tr, claimed);
}
// weight_commitment.rs:377-415
inline bool verify_mle_eval_ef(EF claimed, const VEF& point, const MleEvalProofEF& p, Transcript& tr) {
    VEF s;
    if (!verify_product_ef_with_challenges(claimed, p.eval_sumcheck, ef_of(p.eq_at_s), ef_of(p.w_at_s), tr, &s)) return false;
    if (compute_eq_at_point_ef(point, s) != ef_of(p.eq_at_s)) return false;
    derive_query_indices(tr, point.size());
    return true;
}
// weight_commitment.rs:521-532
inline bool verify_mle_eval_ef_bound(const WeightCommitment& c, EF claimed, const VEF& point, const MleEvalProofEF& p,
                                     const std::string& label, Transcript& tr) {
    tr.absorb_bytes(label);
    tr.absorb_bytes(c.root);
    return verify_mle_eval_ef(claimed, point, p, tr);
}

}  // namespace zko
