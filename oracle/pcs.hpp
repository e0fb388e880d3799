// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Merkle tree with 16-byte digests, restating rust/zk_ml_prover/src/proving/pcs.rs:
//   hash_leaf                 pcs.rs:71-75     u32 LE, zero-padded to 16 bytes (no hashing)
//   hash_node                 pcs.rs:87-135    two variants, chosen by target architecture in
//                                              the reference: blake3(L || R)[..16] everywhere
//                                              except aarch64, AES-MMO on aarch64
//   MerkleTree::new/new_full  pcs.rs:143-196   zero-pad to 2^log2_ceil(n), at least 2 leaves
//   open / batch_open         pcs.rs:204-217, 290-337
//   verify_merkle_opening     pcs.rs:241-259
//   verify_batch_opening      pcs.rs:345-438
//
// The AES primitives (S-box from the field inverse and the affine map, ShiftRows, MixColumns)
// follow FIPS-197; tests pin them by running a full AES-128 encryption built from the same
// three functions against a library implementation.
#pragma once
#include "commit.hpp"
#include <algorithm>
#include <set>

namespace zko {

using Digest = std::array<uint8_t, 16>;
enum NodeHash : int { NODE_BLAKE3 = 0, NODE_AES_MMO = 1 };

namespace aes {
inline uint8_t xtime(uint8_t a) { return uint8_t((a << 1) ^ ((a & 0x80) ? 0x1b : 0)); }
inline uint8_t gmul(uint8_t a, uint8_t b) {
    uint8_t r = 0;
    while (b) { if (b & 1) r ^= a; a = xtime(a); b >>= 1; }
    return r;
}
inline const uint8_t* sbox() {
    static uint8_t S[256];
    static bool init = false;
    if (!init) {
        for (int x = 0; x < 256; x++) {
            uint8_t inv = 0;
            if (x) { inv = 1; uint8_t a = uint8_t(x); for (int i = 0; i < 254; i++) inv = gmul(inv, a); }   // x^254
            uint8_t s = inv;
            for (int i = 1; i <= 4; i++) s ^= uint8_t((inv << i) | (inv >> (8 - i)));
            S[x] = s ^ 0x63;
        }
        init = true;
    }
    return S;
}
// State bytes are column-major: byte index = 4 * column + row.
inline void sub_bytes(uint8_t s[16]) { const uint8_t* S = sbox(); for (int i = 0; i < 16; i++) s[i] = S[s[i]]; }
inline void shift_rows(uint8_t s[16]) {
    uint8_t t[16];
    for (int c = 0; c < 4; c++) for (int r = 0; r < 4; r++) t[4 * c + r] = s[4 * ((c + r) & 3) + r];
    memcpy(s, t, 16);
}
inline void mix_columns(uint8_t s[16]) {
    for (int c = 0; c < 4; c++) {
        uint8_t* p = s + 4 * c;
        uint8_t a0 = p[0], a1 = p[1], a2 = p[2], a3 = p[3];
        p[0] = uint8_t(xtime(a0) ^ (xtime(a1) ^ a1) ^ a2 ^ a3);
        p[1] = uint8_t(a0 ^ xtime(a1) ^ (xtime(a2) ^ a2) ^ a3);
        p[2] = uint8_t(a0 ^ a1 ^ xtime(a2) ^ (xtime(a3) ^ a3));
        p[3] = uint8_t((xtime(a0) ^ a0) ^ a1 ^ a2 ^ xtime(a3));
    }
}
// AES-128 encryption of one block (only used to pin the primitives above).
inline void encrypt128(const uint8_t key[16], const uint8_t in[16], uint8_t out[16]) {
    uint8_t rk[11][16];
    memcpy(rk[0], key, 16);
    uint8_t rcon = 1;
    const uint8_t* S = sbox();
    for (int r = 1; r <= 10; r++) {
        uint8_t t[4] = {S[rk[r - 1][13]], S[rk[r - 1][14]], S[rk[r - 1][15]], S[rk[r - 1][12]]};
        t[0] ^= rcon; rcon = xtime(rcon);
        for (int i = 0; i < 4; i++) rk[r][i] = rk[r - 1][i] ^ t[i];
        for (int i = 4; i < 16; i++) rk[r][i] = rk[r - 1][i] ^ rk[r][i - 4];
    }
    uint8_t s[16];
    for (int i = 0; i < 16; i++) s[i] = in[i] ^ rk[0][i];
    for (int r = 1; r <= 10; r++) {
        sub_bytes(s); shift_rows(s);
        if (r < 10) mix_columns(s);
        for (int i = 0; i < 16; i++) s[i] ^= rk[r][i];
    }
    memcpy(out, s, 16);
}
}  // namespace aes

inline Digest hash_leaf(uint32_t v) {
    Digest d{};
    d[0] = uint8_t(v); d[1] = uint8_t(v >> 8); d[2] = uint8_t(v >> 16); d[3] = uint8_t(v >> 24);
    return d;
}

// pcs.rs:92-121: the ARM AESE instruction is AddRoundKey, SubBytes, ShiftRows (in that order),
// AESMC is MixColumns.  State starts as L^R, ten AESE steps with keys L, R, L, R, ..., MixColumns
// after the first nine, then the feed-forward XOR with L^R.
inline Digest hash_node_aes(const Digest& l, const Digest& r) {
    uint8_t x[16], s[16];
    for (int i = 0; i < 16; i++) { x[i] = l[i] ^ r[i]; s[i] = x[i]; }
    for (int round = 0; round < 10; round++) {
        const Digest& k = (round & 1) ? r : l;
        for (int i = 0; i < 16; i++) s[i] ^= k[i];
        aes::sub_bytes(s);
        aes::shift_rows(s);
        if (round < 9) aes::mix_columns(s);
    }
    Digest o;
    for (int i = 0; i < 16; i++) o[i] = s[i] ^ x[i];
    return o;
}
// pcs.rs:125-134
inline Digest hash_node_blake3(const Digest& l, const Digest& r) {
    // blake3 of a 32-byte message is one compression: a single chunk of one block that is also the
    // root (the general path in hash.hpp computes the same; tests/test_oracle_pcs.py checks it
    // against the blake3 wheel).
    uint32_t block[16] = {0}, out[16];
    for (int i = 0; i < 4; i++) {
        block[i] = uint32_t(l[4 * i]) | uint32_t(l[4 * i + 1]) << 8 | uint32_t(l[4 * i + 2]) << 16 | uint32_t(l[4 * i + 3]) << 24;
        block[4 + i] = uint32_t(r[4 * i]) | uint32_t(r[4 * i + 1]) << 8 | uint32_t(r[4 * i + 2]) << 16 | uint32_t(r[4 * i + 3]) << 24;
    }
    b3::compress(b3::IV, block, 0, 32, b3::CHUNK_START | b3::CHUNK_END | b3::ROOT, out);
    Digest o;
    for (int i = 0; i < 4; i++)
        for (int b = 0; b < 4; b++) o[4 * i + b] = uint8_t(out[i] >> (8 * b));
    return o;
}
inline Digest hash_node(const Digest& l, const Digest& r, int kind) {
    return kind == NODE_AES_MMO ? hash_node_aes(l, r) : hash_node_blake3(l, r);
}

// pcs.rs:43-53
struct BatchMerkleProof {
    std::vector<uint32_t> indices;
    std::vector<uint32_t> values;
    std::vector<std::vector<Digest>> auth_nodes;
};

struct MerkleTree {
    std::vector<std::vector<Digest>> layers;   // layers[0] empty (leaves are not stored), layers[last] = [root]
    std::vector<uint32_t> values;
    size_t log_height = 0;
    int kind = NODE_BLAKE3;

    MerkleTree() {}
    // pcs.rs:143-196
    MerkleTree(const F* w, size_t n, int kind_) : kind(kind_) {
        log_height = n <= 1 ? 1 : log2_ceil(n);
        size_t n_pad = size_t(1) << log_height;
        values.assign(n_pad, 0);
        for (size_t i = 0; i < n; i++) values[i] = w[i].v;
        layers.emplace_back();
        std::vector<Digest> first(n_pad / 2);
        par_rows(n_pad / 2, [&](size_t lo, size_t hi, int) {
            for (size_t i = lo; i < hi; i++) first[i] = hash_node(hash_leaf(values[2 * i]), hash_leaf(values[2 * i + 1]), kind);
        });
        layers.push_back(std::move(first));
        while (layers.back().size() > 1) {
            const auto& prev = layers.back();
            std::vector<Digest> next(prev.size() / 2);
            par_rows(next.size(), [&](size_t lo, size_t hi, int) {
                for (size_t i = lo; i < hi; i++) next[i] = hash_node(prev[2 * i], prev[2 * i + 1], kind);
            });
            layers.push_back(std::move(next));
        }
    }
    MerkleTree(const VF& w, int kind_) : MerkleTree(w.data(), w.size(), kind_) {}
    Digest root() const { return layers.back()[0]; }

    // pcs.rs:204-217
    std::pair<uint32_t, std::vector<Digest>> open(size_t index) const {
        std::vector<Digest> path;
        for (size_t k = 0; k < log_height; k++) {
            size_t sib = (index >> k) ^ 1;
            path.push_back(k == 0 ? hash_leaf(values[sib]) : layers[k][sib]);
        }
        return {values[index], path};
    }

    // pcs.rs:290-337: indices and values keep the caller's order (duplicates included); per
    // level the digests of siblings that are not themselves known, in ascending node index.
    BatchMerkleProof batch_open(const std::vector<size_t>& indices) const {
        BatchMerkleProof p;
        for (size_t i : indices) { p.indices.push_back(uint32_t(i)); p.values.push_back(values[i]); }
        std::set<size_t> known(indices.begin(), indices.end());
        for (size_t k = 0; k < log_height; k++) {
            std::vector<Digest> level;
            std::set<size_t> next;
            for (size_t node : known) {          // ascending, so the siblings come out ascending too
                size_t sib = node ^ 1;
                next.insert(node >> 1);
                if (!known.count(sib)) level.push_back(k == 0 ? hash_leaf(values[sib]) : layers[k][sib]);
            }
            p.auth_nodes.push_back(std::move(level));
            known = std::move(next);
        }
        return p;
    }
};

// pcs.rs:241-259
inline bool verify_merkle_opening(const Digest& root, size_t index, uint32_t value, const std::vector<Digest>& path,
                                  size_t log_height, int kind) {
    if (path.size() != log_height) return false;
    Digest cur = hash_leaf(value);
    for (size_t k = 0; k < log_height; k++) cur = ((index >> k) & 1) ? hash_node(path[k], cur, kind) : hash_node(cur, path[k], kind);
    return cur == root;
}

// pcs.rs:345-438
inline bool verify_batch_opening(const Digest& root, const BatchMerkleProof& p, size_t log_height, int kind) {
    if (p.indices.size() != p.values.size()) return false;
    std::vector<std::pair<uint32_t, Digest>> known;
    for (size_t i = 0; i < p.indices.size(); i++) known.push_back({p.indices[i], hash_leaf(p.values[i])});
    // sort_unstable_by_key + dedup_by_key: equal indices carry equal digests in an honest proof;
    // a stable sort keeps the first of equal keys, which is one of the outcomes the reference allows
    std::stable_sort(known.begin(), known.end(), [](auto& a, auto& b) { return a.first < b.first; });
    known.erase(std::unique(known.begin(), known.end(), [](auto& a, auto& b) { return a.first == b.first; }), known.end());
    for (size_t k = 0; k < log_height; k++) {
        if (k < p.auth_nodes.size() && !p.auth_nodes[k].empty()) {
            std::vector<uint32_t> unknown;
            for (auto& e : known) {
                uint32_t sib = e.first ^ 1;
                bool have = std::binary_search(known.begin(), known.end(), std::make_pair(sib, Digest{}),
                                               [](auto& a, auto& b) { return a.first < b.first; });
                if (!have) unknown.push_back(sib);
            }
            std::sort(unknown.begin(), unknown.end());
            unknown.erase(std::unique(unknown.begin(), unknown.end()), unknown.end());
            if (unknown.size() != p.auth_nodes[k].size()) return false;
            std::vector<std::pair<uint32_t, Digest>> merged;
            size_t i = 0, j = 0;
            while (i < known.size() && j < unknown.size()) {
                if (known[i].first <= unknown[j]) merged.push_back(known[i++]);
                else { merged.push_back({unknown[j], p.auth_nodes[k][j]}); j++; }
            }
            for (; i < known.size(); i++) merged.push_back(known[i]);
            for (; j < unknown.size(); j++) merged.push_back({unknown[j], p.auth_nodes[k][j]});
            known.swap(merged);
        }
        std::vector<std::pair<uint32_t, Digest>> parents;
        size_t pos = 0;
        while (pos < known.size()) {
            uint32_t idx = known[pos].first;
            if ((idx & 1) == 0 && pos + 1 < known.size() && known[pos + 1].first == (idx | 1)) {
                parents.push_back({idx >> 1, hash_node(known[pos].second, known[pos + 1].second, kind)});
                pos += 2;
            } else {
                return false;
            }
        }
        known.swap(parents);
    }
    return known.size() == 1 && known[0].first == 0 && known[0].second == root;
}

}  // namespace zko
