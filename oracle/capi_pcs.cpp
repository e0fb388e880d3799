// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// C entry points for the Merkle tree and Basefold restatements (oracle/pcs.hpp,
// oracle/basefold.hpp).  Proofs come back as bincode bytes in serde field order:
//   BasefoldCommitment   { root: [u8;16], num_coeffs: u64, log_n: u64 }                      basefold.rs:39-47
//   BasefoldOpeningProof { fold_roots: Vec<[u8;16]>, fold_queries: Vec<FoldLevelQueries>,
//                          final_value: u32, final_coeffs: Vec<u32> }                        basefold.rs:50-64
//   FoldLevelQueries     { prev_batch_proof, folded_batch_proof }                            basefold.rs:73-81
//   BatchMerkleProof     { indices: Vec<u32>, values: Vec<u32>, auth_nodes: Vec<Vec<[u8;16]>> }   pcs.rs:43-53
#include "basefold_batch.hpp"
#include "unbincode.hpp"
#include <cstring>

using namespace zko;

static VF vf(const uint32_t* p, size_t n) { VF v(n); for (size_t i = 0; i < n; i++) v[i] = F(p[i]); return v; }
static Transcript& T(void* t) { return *static_cast<Transcript*>(t); }
static size_t emit(const std::vector<uint8_t>& b, uint8_t* out, size_t cap) {
    if (out && b.size() <= cap) memcpy(out, b.data(), b.size());
    return b.size();
}
extern "C" {

void zko_aes128_encrypt(const uint8_t* key, const uint8_t* in, uint8_t* out) { aes::encrypt128(key, in, out); }
void zko_hash_node(const uint8_t* l, const uint8_t* r, int kind, uint8_t* out) {
    Digest a, b;
    memcpy(a.data(), l, 16); memcpy(b.data(), r, 16);
    Digest o = hash_node(a, b, kind);
    memcpy(out, o.data(), 16);
}
void zko_merkle_root(const uint32_t* v, size_t n, int kind, uint8_t* root) {
    MerkleTree t(vf(v, n), kind);
    memcpy(root, t.root().data(), 16);
}
// Every internal layer, concatenated from layer 1 (n_pad / 2 nodes) to the root.
size_t zko_merkle_layers(const uint32_t* v, size_t n, int kind, uint8_t* out, size_t cap) {
    MerkleTree t(vf(v, n), kind);
    std::vector<uint8_t> b;
    for (size_t k = 1; k < t.layers.size(); k++) for (auto& d : t.layers[k]) b.insert(b.end(), d.begin(), d.end());
    return emit(b, out, cap);
}
size_t zko_merkle_batch_open(const uint32_t* v, size_t n, int kind, const uint64_t* idx, size_t n_idx, uint8_t* out, size_t cap) {
    MerkleTree t(vf(v, n), kind);
    Bin b;
    b.put(t.batch_open(std::vector<size_t>(idx, idx + n_idx)));
    return emit(b.b, out, cap);
}
// 1 = batch proof of the given positions verifies against the tree's root; tamper flips a value bit.
int zko_merkle_batch_roundtrip(const uint32_t* v, size_t n, int kind, const uint64_t* idx, size_t n_idx, int tamper) {
    MerkleTree t(vf(v, n), kind);
    auto p = t.batch_open(std::vector<size_t>(idx, idx + n_idx));
    if (tamper == 1) p.values[0] ^= 1;
    if (tamper == 2) { for (auto& l : p.auth_nodes) if (!l.empty()) { l[0][3] ^= 4; break; } }
    bool single = true;
    for (size_t i = 0; i < n_idx; i++) {
        auto o = t.open(idx[i]);
        single = single && verify_merkle_opening(t.root(), idx[i], o.first, o.second, t.log_height, kind);
    }
    return (verify_batch_opening(t.root(), p, t.log_height, kind) ? 1 : 0) | (single ? 2 : 0);
}
void zko_basefold_tables(size_t log_n, uint32_t* t_flat, uint32_t* w_flat) {
    auto tb = basefold_tables(log_n);
    for (size_t i = 0; i < tb->t_flat.size(); i++) { t_flat[i] = tb->t_flat[i].v; w_flat[i] = tb->w_flat[i].v; }
}
void zko_basefold_encode(const uint32_t* c, size_t log_n, uint32_t* cw) {
    auto tb = basefold_tables(log_n);
    VF o = basefold_encode(vf(c, size_t(1) << log_n), log_n, *tb);
    for (size_t i = 0; i < o.size(); i++) cw[i] = o[i].v;
}
// bincode(BasefoldCommitment) followed by bincode(BasefoldOpeningProof)
size_t zko_basefold_commit_and_prove(void* t, const uint32_t* c, size_t n, const uint32_t* point, size_t n_point, int kind,
                                     uint8_t* out, size_t cap) {
    auto r = basefold_commit_and_prove(vf(c, n), vf(point, n_point), T(t), kind);
    Bin b;
    b.put(r.first); b.put(r.second);
    return emit(b.b, out, cap);
}
// prove, then verify with a fresh transcript of the same label; claimed = MLE(coeffs)(point).
// tamper: 0 none, 1 final value, 2 a fold root, 3 an opened value, 4 wrong claimed value.
int zko_basefold_roundtrip(const uint32_t* c, size_t n, const uint32_t* point, size_t n_point, int kind, int tamper) {
    Transcript pt("bf"), vt("bf");
    VF co = vf(c, n), pnt = vf(point, n_point);
    auto r = basefold_commit_and_prove(co, pnt, pt, kind);
    size_t log_n = r.first.log_n;
    F claimed = mle_evaluate(padded(co, size_t(1) << log_n), pnt);
    if (F(r.second.final_value) != claimed) return -1;
    if (tamper == 1) r.second.final_value ^= 1;
    if (tamper == 2) r.second.fold_roots[r.second.fold_roots.size() / 2][5] ^= 1;
    if (tamper == 3) r.second.fold_queries[0].prev_batch_proof.values[0] ^= 2;
    if (tamper == 4) claimed = claimed + F::one();
    vt.absorb_bytes(r.first.root);
    return basefold_verify_opening(r.first, claimed, pnt, r.second, vt, kind) ? 1 : 0;
}

// Decode bincode(BasefoldCommitment) || bincode(BasefoldOpeningProof) and run verify_opening on it.
// The caller has absorbed the commitment root.  1 accept, 0 reject, -1 the bytes do not decode.
int zko_basefold_verify_bytes(void* t, const uint8_t* b, size_t n, const uint32_t* point, size_t n_point, uint32_t claimed, int kind) {
    size_t at = 0;
    bool ok = true;
    auto u64v = [&]() -> uint64_t { if (at + 8 > n) { ok = false; return 0; } uint64_t v = 0; for (int i = 0; i < 8; i++) v |= uint64_t(b[at + i]) << (8 * i); at += 8; return v; };
    auto u32v = [&]() -> uint32_t { if (at + 4 > n) { ok = false; return 0; } uint32_t v = 0; for (int i = 0; i < 4; i++) v |= uint32_t(b[at + i]) << (8 * i); at += 4; return v; };
    auto dig = [&]() -> Digest { Digest d{}; if (at + 16 > n) { ok = false; return d; } memcpy(d.data(), b + at, 16); at += 16; return d; };
    auto batch = [&]() -> BatchMerkleProof {
        BatchMerkleProof p;
        uint64_t ni = u64v(); if (!ok || ni > (1u << 20)) { ok = false; return p; }
        for (uint64_t i = 0; i < ni; i++) p.indices.push_back(u32v());
        uint64_t nv = u64v(); if (!ok || nv > (1u << 20)) { ok = false; return p; }
        for (uint64_t i = 0; i < nv; i++) p.values.push_back(u32v());
        uint64_t nl = u64v(); if (!ok || nl > 64) { ok = false; return p; }
        for (uint64_t l = 0; l < nl && ok; l++) {
            uint64_t cnt = u64v(); if (!ok || cnt > (1u << 20)) { ok = false; return p; }
            std::vector<Digest> lv;
            for (uint64_t i = 0; i < cnt; i++) lv.push_back(dig());
            p.auth_nodes.push_back(std::move(lv));
        }
        return p;
    };
    BasefoldCommitment c;
    c.root = dig(); c.num_coeffs = u64v(); c.log_n = u64v();
    BasefoldOpeningProof pr;
    uint64_t nr = u64v(); if (!ok || nr > 64) return -1;
    for (uint64_t i = 0; i < nr; i++) pr.fold_roots.push_back(dig());
    uint64_t nq = u64v(); if (!ok || nq > 64) return -1;
    for (uint64_t i = 0; i < nq && ok; i++) { FoldLevelQueries q; q.prev_batch_proof = batch(); q.folded_batch_proof = batch(); pr.fold_queries.push_back(std::move(q)); }
    pr.final_value = u32v();
    uint64_t nf = u64v();
    for (uint64_t i = 0; i < nf && ok; i++) pr.final_coeffs.push_back(u32v());
    if (!ok || at != n || c.log_n < 1 || c.log_n > 28) return -1;
    return basefold_verify_opening(c, F(claimed), vf(point, n_point), pr, T(t), kind) ? 1 : 0;
}

// Process-wide stand-ins for the reference's cargo features and target architecture.
void zko_set_features(int bind_mode, int node_kind) { features().bind_mode = bind_mode; features().node_kind = node_kind; }


// ---- batch Basefold (basefold.rs:769-1590).  Polynomial i has n[i] coefficients at flat[off[i]...] and the caller's log_n[i].
// bincode(Vec<BasefoldCommitment>) (input order) followed by bincode(BasefoldBatchProof).
static std::vector<BatchPoly> batch_polys(const uint32_t* flat, const uint64_t* n, const uint64_t* log_n, size_t k) {
    std::vector<BatchPoly> bp;
    size_t off = 0;
    for (size_t i = 0; i < k; i++) { bp.push_back({vf(flat + off, n[i]), size_t(log_n[i])}); off += n[i]; }
    return bp;
}
size_t zko_basefold_batch_prove(void* t, const uint32_t* flat, const uint64_t* n, const uint64_t* log_n, size_t k, int individual_openings, int kind,
                                uint8_t* out, size_t cap) {
    BatchPrecommit pre = batch_precommit_multi_height(batch_polys(flat, n, log_n, k), kind);
    BasefoldBatchProof P = batch_prove_with_precommit(pre, T(t), individual_openings != 0);
    Bin b;
    b.u64(pre.commitments.size());
    for (auto& c : pre.commitments) b.put(c);
    put(b, P);
    return emit(b.b, out, cap);
}
// prove -> verify with fresh transcripts of one label.  tamper: 1 a fold root (basefold.rs:1889-1921), 2 an opened value of the first
// round, 3 the batched root, 4 a value in an add-round opening (needs polynomials of different sizes), 5 an individual root.
int zko_basefold_batch_roundtrip(const uint32_t* flat, const uint64_t* n, const uint64_t* log_n, size_t k, int individual_openings, int kind, int tamper) {
    Transcript pt("batch"), vt("batch");
    BatchPrecommit pre = batch_precommit_multi_height(batch_polys(flat, n, log_n, k), kind);
    BasefoldBatchProof P = batch_prove_with_precommit(pre, pt, individual_openings != 0);
    if (tamper == 1) P.fold_roots[0].fill(0xDE);
    if (tamper == 2) P.fold_queries[0].prev_batch_proof.values[0] ^= 2;
    if (tamper == 3) P.batched_root[3] ^= 1;
    if (tamper == 4) { if (P.add_round_openings.empty()) return -1; P.add_round_openings[0].second[0].second.values[0] ^= 4; }
    if (tamper == 5) P.roots[k - 1][0] ^= 1;
    bool ok = batch_verify_opening(pre.commitments, P, vt, kind);
    return ok && pt.squeeze().v == vt.squeeze().v;
}

// Decode bincode(Vec<BasefoldCommitment>) || bincode(BasefoldBatchProof) and run batch_verify_opening (basefold.rs:959-1137) on it.
// 1 accept, 0 reject, -1 the bytes do not decode.  final_value_out (optional) receives the proof's final value, which the
// reference's verifier does not check.
int zko_basefold_batch_verify_bytes(void* t, const uint8_t* b, size_t n, int kind, uint32_t* final_value_out) {
    Rd r{b, n};
    size_t k = r.len(32);
    std::vector<BasefoldCommitment> cs(k);
    for (auto& c : cs) { r.bytes(c.root); c.num_coeffs = r.u64(); c.log_n = r.u64(); }
    BasefoldBatchProof P;
    P.num_polys = r.u64();
    size_t m = r.len(8);
    for (size_t i = 0; i < m && r.ok; i++) P.poly_log_ns.push_back(r.u64());
    m = r.len(16);
    P.roots.assign(m, Digest{});
    for (auto& d : P.roots) r.bytes(d);
    r.bytes(P.batched_root);
    m = r.len(16);
    P.fold_roots.assign(m, Digest{});
    for (auto& d : P.fold_roots) r.bytes(d);
    m = r.len(48);
    for (size_t i = 0; i < m && r.ok; i++) { P.fold_queries.emplace_back(); r.get(P.fold_queries.back().prev_batch_proof); r.get(P.fold_queries.back().folded_batch_proof); }
    m = r.len(24);
    for (size_t i = 0; i < m && r.ok; i++) { P.query_openings.emplace_back(); r.get(P.query_openings.back()); }
    P.final_value = r.u32();
    m = r.len(16);
    for (size_t i = 0; i < m && r.ok; i++) {
        uint64_t round = r.u64();
        size_t cnt = r.len(32);
        std::vector<std::pair<uint64_t, BatchMerkleProof>> v;
        for (size_t j = 0; j < cnt && r.ok; j++) { uint64_t pi = r.u64(); BatchMerkleProof bp; r.get(bp); v.emplace_back(pi, std::move(bp)); }
        P.add_round_openings.emplace_back(round, std::move(v));
    }
    if (!r.ok || r.at != n) return -1;
    for (uint64_t l : P.poly_log_ns) if (l < 1 || l > 28) return 0;
    if (final_value_out) *final_value_out = P.final_value;
    return batch_verify_opening(cs, P, T(t), kind) ? 1 : 0;
}

}  // extern "C"
