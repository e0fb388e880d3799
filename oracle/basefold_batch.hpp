// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Batch Basefold: k polynomials, possibly of different sizes, opened with ONE fold chain
// (rust/zk_ml_prover/src/proving/basefold.rs:769-1590).
//   BasefoldBatchProof                        :769-795
//   batch_commit_and_prove (same size)        :801-956
//   batch_verify_opening                      :959-1137
//   batch_precommit_multi_height              :1183-1216   (transcript-independent: encodings and trees)
//   batch_prove_with_precommit                :1221-1378   (== batch_commit_and_prove_multi_height(_owned) :1383-1590 after the precommit)
// The reference pins these with three round-trip tests (:1849-1960), repeated on this restatement.
#pragma once
#include "bincode.hpp"
#include <algorithm>

namespace zko {

struct BasefoldBatchProof {
    uint64_t num_polys = 0;
    std::vector<uint64_t> poly_log_ns;
    std::vector<Digest> roots;
    Digest batched_root{};
    std::vector<Digest> fold_roots;
    std::vector<FoldLevelQueries> fold_queries;
    std::vector<BatchMerkleProof> query_openings;
    uint32_t final_value = 0;
    std::vector<std::pair<uint64_t, std::vector<std::pair<uint64_t, BatchMerkleProof>>>> add_round_openings;
};

struct BatchPoly { VF coeffs; size_t log_n; };
struct BatchPrecommitEntry { VF coeffs_padded, cw; std::unique_ptr<MerkleTree> tree; size_t log_n, orig; };
struct BatchPrecommit {
    std::vector<BatchPrecommitEntry> encoded;    // sorted by log_n descending, ties in input order (Rust's sort_by is stable)
    size_t max_log_n = 0;
    std::shared_ptr<const FoldableTables> tables;
    std::vector<BasefoldCommitment> commitments; // input order
    int kind = NODE_BLAKE3;
};

// basefold.rs:1183-1216: every polynomial is encoded with the tables of the LARGEST one (seed of max_log_n).
inline BatchPrecommit batch_precommit_multi_height(const std::vector<BatchPoly>& polys, int kind) {
    BatchPrecommit pre;
    pre.kind = kind;
    size_t k = polys.size();
    std::vector<size_t> order(k);
    for (size_t i = 0; i < k; i++) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return polys[a].log_n > polys[b].log_n; });
    pre.max_log_n = polys[order[0]].log_n;
    pre.tables = basefold_tables(pre.max_log_n);
    pre.commitments.resize(k);
    for (size_t idx : order) {
        const BatchPoly& p = polys[idx];
        BatchPrecommitEntry e;
        e.coeffs_padded = padded(p.coeffs, size_t(1) << p.log_n);
        e.cw = basefold_encode(e.coeffs_padded, p.log_n, *pre.tables);
        e.tree = std::make_unique<MerkleTree>(e.cw, kind);
        e.log_n = p.log_n; e.orig = idx;
        BasefoldCommitment c;
        c.root = e.tree->root(); c.num_coeffs = p.coeffs.size(); c.log_n = p.log_n;
        pre.commitments[idx] = c;
        pre.encoded.push_back(std::move(e));
    }
    return pre;
}

// basefold.rs:1221-1378.  individual_openings: additionally open every individual tree at the final query
// positions, as the same-size batch_commit_and_prove does (:916-927); the multi-height functions leave them out.
inline BasefoldBatchProof batch_prove_with_precommit(const BatchPrecommit& pre, Transcript& tr, bool individual_openings = false) {
    const auto& enc = pre.encoded;
    const size_t k = enc.size(), max_log_n = pre.max_log_n;
    const FoldableTables& tb = *pre.tables;
    BasefoldBatchProof P;
    P.num_polys = k;
    for (auto& e : enc) { P.roots.push_back(e.tree->root()); P.poly_log_ns.push_back(e.log_n); }
    for (auto& r : P.roots) tr.absorb_bytes(r);
    F rho = tr.squeeze();
    VF bc;
    F pw = F::one();
    for (size_t i = 0; i < k; i++) { bc.push_back(pw); pw = pw * rho; }
    struct Group { size_t log_n, s, e; };
    std::vector<Group> groups;
    for (size_t gs = 0; gs < k;) {
        size_t ge = gs + 1;
        while (ge < k && enc[ge].log_n == enc[gs].log_n) ge++;
        groups.push_back({enc[gs].log_n, gs, ge});
        gs = ge;
    }
    size_t cw_len = size_t(2) << max_log_n;
    VF cw(cw_len, F::zero());
    for (size_t i = groups[0].s; i < groups[0].e; i++)
        for (size_t j = 0; j < enc[i].cw.size(); j++) cw[j] = cw[j] + bc[i] * enc[i].cw[j];
    MerkleTree batched_tree(cw, pre.kind);
    P.batched_root = batched_tree.root();
    tr.absorb_bytes(P.batched_root);
    VF fold_point = tr.squeeze_many(max_log_n);
    std::unique_ptr<MerkleTree> prev_owned;
    size_t next_group = 1;
    for (size_t round = 0; round < max_log_n; round++) {
        F alpha = fold_point[round];
        tr.absorb(alpha);
        size_t fold_level = max_log_n - 1 - round, prev_cw_len = cw_len;
        cw_len = fold_codeword_inplace(cw.data(), prev_cw_len, alpha, tb.w_level(fold_level), size_t(1) << fold_level);
        size_t target = max_log_n - 1 - round;
        while (next_group < groups.size() && groups[next_group].log_n == target) {
            for (size_t i = groups[next_group].s; i < groups[next_group].e; i++)
                for (size_t j = 0; j < std::min(enc[i].cw.size(), cw_len); j++) cw[j] = cw[j] + bc[i] * enc[i].cw[j];
            next_group++;
        }
        auto folded = std::make_unique<MerkleTree>(cw.data(), cw_len, pre.kind);
        Digest root = folded->root();
        P.fold_roots.push_back(root);
        tr.absorb_bytes(root);
        const MerkleTree& prev = round == 0 ? batched_tree : *prev_owned;
        size_t prev_half = prev_cw_len / 2;
        auto q = derive_query_indices(tr, prev.log_height);
        std::vector<size_t> prev_pos, folded_pos;
        for (size_t raw : q) { size_t idx = raw % prev_half; prev_pos.push_back(idx); prev_pos.push_back(idx + prev_half); folded_pos.push_back(idx % cw_len); }
        std::vector<std::pair<uint64_t, BatchMerkleProof>> round_openings;
        for (size_t gi = 1; gi < groups.size(); gi++) if (groups[gi].log_n == target)
            for (size_t i = groups[gi].s; i < groups[gi].e; i++) {
                size_t tree_half = size_t(1) << enc[i].log_n;
                std::vector<size_t> local;
                for (size_t raw : q) { size_t li = ((raw % prev_half) % cw_len) % tree_half; local.push_back(li); local.push_back(li + tree_half); }
                round_openings.emplace_back(i, enc[i].tree->batch_open(local));
            }
        if (!round_openings.empty()) P.add_round_openings.emplace_back(round, std::move(round_openings));
        FoldLevelQueries lq;
        lq.prev_batch_proof = prev.batch_open(prev_pos);
        lq.folded_batch_proof = folded->batch_open(folded_pos);
        P.fold_queries.push_back(std::move(lq));
        prev_owned = std::move(folded);
    }
    F fin = F::zero();
    for (size_t i = 0; i < k; i++) fin = fin + bc[i] * mle_evaluate(enc[i].coeffs_padded, VF(fold_point.begin(), fold_point.begin() + enc[i].log_n));
    P.final_value = fin.v;
    auto fq = derive_query_indices(tr, max_log_n + 1);
    if (individual_openings) {
        size_t initial_half = size_t(1) << max_log_n;
        std::vector<size_t> pos;
        for (size_t raw : fq) { size_t idx = raw % initial_half; pos.push_back(idx); pos.push_back(idx + initial_half); }
        for (auto& e : enc) P.query_openings.push_back(e.tree->batch_open(pos));
    }
    return P;
}

// basefold.rs:801-956: all polynomials already padded to the same power-of-two length.
inline std::pair<std::vector<BasefoldCommitment>, BasefoldBatchProof> batch_commit_and_prove(const std::vector<VF>& polys, Transcript& tr, int kind) {
    size_t n = polys[0].size(), log_n = n <= 1 ? 1 : log2_ceil(n);
    std::vector<BatchPoly> bp;
    for (auto& p : polys) bp.push_back({p, log_n});
    BatchPrecommit pre = batch_precommit_multi_height(bp, kind);
    return {pre.commitments, batch_prove_with_precommit(pre, tr, true)};
}

// basefold.rs:959-1137 (the claimed evaluations are not used by the reference's verifier either)
inline bool batch_verify_opening(const std::vector<BasefoldCommitment>& commitments, const BasefoldBatchProof& P, Transcript& tr, int kind) {
    size_t k = commitments.size();
    if (k != P.num_polys || k != P.roots.size() || P.poly_log_ns.size() != k) return false;
    if (k == 0) return true;
    size_t max_log_n = 1;
    for (uint64_t l : P.poly_log_ns) max_log_n = std::max<size_t>(max_log_n, l);
    if (max_log_n > 30 || P.fold_roots.size() < max_log_n || P.fold_queries.size() < max_log_n) return false;
    for (auto& r : P.roots) tr.absorb_bytes(r);
    F rho = tr.squeeze();
    VF bc;
    F pw = F::one();
    for (size_t i = 0; i < k; i++) { bc.push_back(pw); pw = pw * rho; }
    tr.absorb_bytes(P.batched_root);
    VF fold_point = tr.squeeze_many(max_log_n);
    const F two_inv = inverse(F(2));
    auto tb = basefold_tables(max_log_n);
    Digest current_root = P.batched_root;
    size_t current_log_len = max_log_n + 1;
    auto find = [](const BatchMerkleProof& b, uint32_t idx, uint32_t* val) {
        for (size_t i = 0; i < b.indices.size(); i++) if (b.indices[i] == idx) { if (i >= b.values.size()) return false; *val = b.values[i]; return true; }
        return false;
    };
    for (size_t round = 0; round < max_log_n; round++) {
        F alpha = fold_point[round];
        tr.absorb(alpha);
        const Digest& fold_root = P.fold_roots[round];
        tr.absorb_bytes(fold_root);
        const FoldLevelQueries& level = P.fold_queries[round];
        size_t prev_half = size_t(1) << (current_log_len - 1);
        auto q = derive_query_indices(tr, current_log_len);
        const std::vector<std::pair<uint64_t, BatchMerkleProof>>* adds = nullptr;
        for (auto& a : P.add_round_openings) if (a.first == round) adds = &a.second;     // a later duplicate wins, as in a HashMap insert
        for (size_t qi = 0; qi < NUM_QUERIES; qi++) {
            size_t idx = q[qi] % prev_half;
            uint32_t lv, rv, fv;
            if (!find(level.prev_batch_proof, uint32_t(idx), &lv) || !find(level.prev_batch_proof, uint32_t(idx + prev_half), &rv)) return false;
            size_t fold_level = max_log_n - 1 - round;
            F w = tb->w_level(fold_level)[idx % (size_t(1) << fold_level)];
            F l(lv), r(rv);
            F expect = (l + r) * two_inv + alpha * (l - r) * w;
            if (adds) for (auto& a : *adds) {
                if (a.first >= k || P.poly_log_ns[a.first] > 30) return false;
                size_t tree_half = size_t(1) << P.poly_log_ns[a.first];
                uint32_t v;
                if (find(a.second, uint32_t(idx % tree_half), &v)) expect = expect + bc[a.first] * F(v);
            }
            if (!find(level.folded_batch_proof, uint32_t(idx), &fv)) return false;
            if (F(fv) != expect) return false;
        }
        if (!verify_batch_opening(current_root, level.prev_batch_proof, current_log_len, kind)) return false;
        if (!verify_batch_opening(fold_root, level.folded_batch_proof, current_log_len - 1, kind)) return false;
        current_root = fold_root;
        current_log_len -= 1;
    }
    derive_query_indices(tr, max_log_n + 1);
    std::vector<const BasefoldCommitment*> sorted;
    for (auto& c : commitments) sorted.push_back(&c);
    std::stable_sort(sorted.begin(), sorted.end(), [](const BasefoldCommitment* a, const BasefoldCommitment* b) { return a->log_n > b->log_n; });
    for (size_t i = 0; i < sorted.size() && i < P.query_openings.size(); i++)
        if (!verify_batch_opening(sorted[i]->root, P.query_openings[i], sorted[i]->log_n + 1, kind)) return false;
    for (auto& a : P.add_round_openings) for (auto& o : a.second) {
        if (o.first >= k) return false;
        if (!verify_batch_opening(P.roots[o.first], o.second, P.poly_log_ns[o.first] + 1, kind)) return false;
    }
    return true;
}

inline void put(Bin& b, const BasefoldBatchProof& P) {     // basefold.rs:769-795
    b.u64(P.num_polys);
    b.u64(P.poly_log_ns.size()); for (uint64_t l : P.poly_log_ns) b.u64(l);
    b.u64(P.roots.size()); for (auto& d : P.roots) b.bytes(d);
    b.bytes(P.batched_root);
    b.u64(P.fold_roots.size()); for (auto& d : P.fold_roots) b.bytes(d);
    b.u64(P.fold_queries.size()); for (auto& q : P.fold_queries) { b.put(q.prev_batch_proof); b.put(q.folded_batch_proof); }
    b.u64(P.query_openings.size()); for (auto& q : P.query_openings) b.put(q);
    b.u32(P.final_value);
    b.u64(P.add_round_openings.size());
    for (auto& a : P.add_round_openings) {
        b.u64(a.first);
        b.u64(a.second.size());
        for (auto& o : a.second) { b.u64(o.first); b.put(o.second); }
    }
}

}  // namespace zko
