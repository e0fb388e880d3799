// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Basefold polynomial commitment (single polynomial), restating
// rust/zk_ml_prover/src/proving/basefold.rs:
//   table_seed, generate_tables, table/weight_level   basefold.rs:106-157, 323-328
//   encode                                            basefold.rs:169-238
//   fold_codeword_inplace                             basefold.rs:250-316
//   commit, commit_and_prove(_with_tables/_vec)       basefold.rs:332-467
//   prove_opening_with_tree                           basefold.rs:483-585
//   verify_opening(_with_tables)                      basefold.rs:611-748
// Parity unpinned: the reference holds no literal vectors for this scheme; its own tests are
// prove -> verify round trips and tamper rejections, which tests/ repeat on this restatement.
#pragma once
#include "pcs.hpp"
#include <map>
#include <memory>
#include <mutex>

namespace zko {

struct BasefoldCommitment {          // basefold.rs:39-47
    Digest root{};
    uint64_t num_coeffs = 0;
    uint64_t log_n = 0;
};
struct FoldLevelQueries {            // basefold.rs:73-81
    BatchMerkleProof prev_batch_proof, folded_batch_proof;
};
struct BasefoldOpeningProof {        // basefold.rs:50-64
    std::vector<Digest> fold_roots;
    std::vector<FoldLevelQueries> fold_queries;
    uint32_t final_value = 0;
    std::vector<uint32_t> final_coeffs;
};

struct FoldableTables {              // basefold.rs:96-102: level i holds 2^i values at offset 2^i - 1
    VF t_flat, w_flat;
    const F* t_level(size_t level) const { return t_flat.data() + ((size_t(1) << level) - 1); }
    const F* w_level(size_t level) const { return w_flat.data() + ((size_t(1) << level) - 1); }
};

// basefold.rs:323-328
inline std::array<uint8_t, 32> basefold_table_seed(size_t log_n) {
    std::vector<uint8_t> buf;
    const char* tag = "basefold-foldable-code";
    buf.insert(buf.end(), tag, tag + 22);
    for (int i = 0; i < 8; i++) buf.push_back(uint8_t(uint64_t(log_n) >> (8 * i)));
    return blake3(buf);
}

// basefold.rs:106-143: T = 1 + (u32 LE from the blake3 XOF of the seed) mod (p - 1);
// w = 1 / (2 T).  The reference inverts in a Montgomery batch; inverses are unique, so a
// per-element inverse gives the same numbers (the batch is used here too, for speed).
inline FoldableTables generate_tables(size_t num_levels, const std::array<uint8_t, 32>& seed) {
    size_t total = (size_t(1) << num_levels) - 1;
    std::vector<uint8_t> buf(total * 4);
    blake3_xof(seed.data(), 32, buf.data(), buf.size());
    FoldableTables tb;
    tb.t_flat.resize(total);
    for (size_t i = 0; i < total; i++) {
        uint32_t raw = uint32_t(buf[4 * i]) | uint32_t(buf[4 * i + 1]) << 8 | uint32_t(buf[4 * i + 2]) << 16 | uint32_t(buf[4 * i + 3]) << 24;
        tb.t_flat[i] = F(1 + raw % (P31 - 1));
    }
    VF prefix(total);
    F acc = F::one();
    for (size_t i = 0; i < total; i++) { prefix[i] = acc; acc = acc * (F(2) * tb.t_flat[i]); }
    F inv = inverse(acc);
    tb.w_flat.resize(total);
    for (size_t i = total; i-- > 0;) { tb.w_flat[i] = prefix[i] * inv; inv = inv * (F(2) * tb.t_flat[i]); }
    return tb;
}

// basefold.rs:377-393 keeps one table set per log_n for the life of the process.
inline std::shared_ptr<const FoldableTables> basefold_tables(size_t log_n) {
    static std::mutex mu;
    static std::map<size_t, std::shared_ptr<const FoldableTables>> cache;
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(log_n);
    if (it != cache.end()) return it->second;
    auto t = std::make_shared<const FoldableTables>(generate_tables(log_n, basefold_table_seed(log_n)));
    cache[log_n] = t;
    return t;
}

// basefold.rs:169-238 (the portable branch): cw = [c || c]; level l butterflies chunks of
// 2^(l+1): L' = L + T R, R' = L - T R with T = t_level(l)[j % 2^l].
inline VF basefold_encode(const VF& coeffs, size_t log_n, const FoldableTables& tb) {
    VF cw(coeffs);
    cw.insert(cw.end(), coeffs.begin(), coeffs.end());
    size_t chunk = 2;
    for (size_t level = 0; level < log_n; level++) {
        const F* t = tb.t_level(level);
        const size_t half = chunk / 2;
        // butterfly b of this level: chunk b / half, offset b % half (every butterfly touches its own two slots)
        par_rows(cw.size() / 2, [&](size_t lo, size_t hi, int) {
            for (size_t b = lo; b < hi; b++) {
                const size_t c0 = (b >> level) << (level + 1), j = b & (half - 1);     // half = t_len = 2^level
                F rhs = cw[c0 + j + half] * t[j];
                F left = cw[c0 + j];
                cw[c0 + j] = left + rhs;
                cw[c0 + j + half] = left - rhs;
            }
        });
        chunk *= 2;
    }
    return cw;
}

// basefold.rs:250-316: cw[j] = (l + r) / 2 + alpha (l - r) w[j % w_len], l = cw[j], r = cw[j + half].
inline size_t fold_codeword_inplace(F* cw, size_t n, F alpha, const F* weights, size_t w_len) {
    const F two_inv(1073741824u);
    size_t half = n / 2;
    par_rows(half, [&](size_t lo, size_t hi, int) {
        for (size_t j = lo; j < hi; j++) {
            F l = cw[j], r = cw[j + half];
            cw[j] = (l + r) * two_inv + alpha * ((l - r) * weights[j % w_len]);
        }
    });
    return half;
}

// basefold.rs:483-585
inline BasefoldOpeningProof basefold_prove_opening(VF eval_buf, VF cw, const VF& point, size_t log_n, const MerkleTree& initial_tree,
                                                   const FoldableTables& tb, Transcript& tr, int kind) {
    BasefoldOpeningProof proof;
    size_t cw_len = cw.size(), eval_size = size_t(1) << log_n;
    std::unique_ptr<MerkleTree> prev_owned;
    for (size_t round = 0; round < log_n; round++) {
        F alpha;
        if (round < point.size()) { tr.absorb(point[round]); alpha = point[round]; }
        else alpha = tr.squeeze();
        size_t half = eval_size / 2;
        F oma = F::one() - alpha;
        for (size_t j = 0; j < half; j++) eval_buf[j] = oma * eval_buf[j] + alpha * eval_buf[j + half];
        eval_size = half;

        size_t fold_level = log_n - 1 - round;
        size_t prev_cw_len = cw_len;
        cw_len = fold_codeword_inplace(cw.data(), prev_cw_len, alpha, tb.w_level(fold_level), size_t(1) << fold_level);
        auto folded = std::make_unique<MerkleTree>(cw.data(), cw_len, kind);
        Digest root = folded->root();
        proof.fold_roots.push_back(root);
        tr.absorb_bytes(root);

        const MerkleTree& prev = round == 0 ? initial_tree : *prev_owned;
        size_t prev_half = prev_cw_len / 2;
        auto q = derive_query_indices(tr, prev.log_height);
        std::vector<size_t> prev_pos, folded_pos;
        for (size_t raw : q) {
            size_t idx = raw % prev_half;
            prev_pos.push_back(idx);
            prev_pos.push_back(idx + prev_half);
            folded_pos.push_back(idx % cw_len);
        }
        FoldLevelQueries lq;
        lq.prev_batch_proof = prev.batch_open(prev_pos);
        lq.folded_batch_proof = folded->batch_open(folded_pos);
        proof.fold_queries.push_back(std::move(lq));
        prev_owned = std::move(folded);
    }
    proof.final_value = eval_buf[0].v;
    return proof;
}

// basefold.rs:368-396, 442-467 (commit_and_prove / _with_tables / _vec are the same computation)
inline std::pair<BasefoldCommitment, BasefoldOpeningProof> basefold_commit_and_prove(const VF& coeffs, const VF& point, Transcript& tr,
                                                                                     int kind) {
    size_t n = coeffs.size();
    size_t log_n = n <= 1 ? 1 : log2_ceil(n);
    VF padded_c = padded(coeffs, size_t(1) << log_n);
    auto tb = basefold_tables(log_n);
    VF cw = basefold_encode(padded_c, log_n, *tb);
    MerkleTree tree(cw, kind);
    BasefoldCommitment c;
    c.root = tree.root(); c.num_coeffs = n; c.log_n = log_n;
    tr.absorb_bytes(c.root);
    auto proof = basefold_prove_opening(std::move(padded_c), std::move(cw), point, log_n, tree, *tb, tr, kind);
    return {c, proof};
}

// basefold.rs:639-748
inline bool basefold_verify_opening(const BasefoldCommitment& c, F claimed, const VF& point, const BasefoldOpeningProof& proof,
                                    Transcript& tr, int kind) {
    size_t log_n = c.log_n;
    if (proof.fold_roots.size() != log_n || proof.fold_queries.size() != log_n) return false;
    auto tb = basefold_tables(log_n);
    const F two_inv = inverse(F(2));
    Digest current_root = c.root;
    size_t current_log_len = log_n + 1;
    for (size_t round = 0; round < log_n; round++) {
        F alpha;
        if (round < point.size()) { tr.absorb(point[round]); alpha = point[round]; }
        else alpha = tr.squeeze();
        const Digest& fold_root = proof.fold_roots[round];
        tr.absorb_bytes(fold_root);
        const FoldLevelQueries& level = proof.fold_queries[round];
        size_t prev_half = size_t(1) << (current_log_len - 1);
        auto q = derive_query_indices(tr, current_log_len);
        const auto& bp = level.prev_batch_proof;
        const auto& fbp = level.folded_batch_proof;
        auto find = [](const BatchMerkleProof& b, uint32_t idx, uint32_t* val) {
            for (size_t i = 0; i < b.indices.size(); i++)
                if (b.indices[i] == idx) { if (i >= b.values.size()) return false; *val = b.values[i]; return true; }
            return false;
        };
        for (size_t k = 0; k < NUM_QUERIES; k++) {
            size_t idx = q[k] % prev_half;
            uint32_t lv, rv, fv;
            if (!find(bp, uint32_t(idx), &lv) || !find(bp, uint32_t(idx + prev_half), &rv)) return false;
            size_t fold_level = log_n - 1 - round;
            F w = tb->w_level(fold_level)[idx % (size_t(1) << fold_level)];
            F l(lv), r(rv);
            F expect = (l + r) * two_inv + alpha * (l - r) * w;
            if (!find(fbp, uint32_t(idx % prev_half), &fv)) return false;
            if (F(fv) != expect) return false;
        }
        if (!verify_batch_opening(current_root, bp, current_log_len, kind)) return false;
        if (!verify_batch_opening(fold_root, fbp, current_log_len - 1, kind)) return false;
        current_root = fold_root;
        current_log_len -= 1;
    }
    return F(proof.final_value) == claimed;
}

}  // namespace zko
