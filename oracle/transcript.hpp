// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Fiat-Shamir transcript, restating rust/zk_ml_prover/src/proving/sumcheck.rs:110-206.
#pragma once
#include "field.hpp"
#include "hash.hpp"
#include <string>

namespace zko {

struct Transcript {
    Sha256 hasher;

    // sumcheck.rs:115-119 — the SHA-256 stream starts with the label bytes.
    explicit Transcript(const std::string& label) { hasher.update(label.data(), label.size()); }
    Transcript(const void* label, size_t len) { hasher.update(label, len); }

    // sumcheck.rs:121-123 — 4 little-endian bytes.
    void absorb(uint32_t v) {
        uint8_t b[4] = {uint8_t(v), uint8_t(v >> 8), uint8_t(v >> 16), uint8_t(v >> 24)};
        hasher.update(b, 4);
    }
    void absorb(F v) { absorb(v.v); }
    // sumcheck.rs:125-129
    void absorb_many(const VF& vs) { for (F v : vs) absorb(v.v); }
    // sumcheck.rs:177-179
    void absorb_bytes(const void* p, size_t n) { hasher.update(p, n); }
    void absorb_bytes(const std::string& s) { hasher.update(s.data(), s.size()); }
    template <size_t N> void absorb_bytes(const std::array<uint8_t, N>& a) { hasher.update(a.data(), N); }
    // sumcheck.rs:196-204
    void absorb_ef(EF v) { uint32_t w[4]; v.to_u32x4(w); for (int i = 0; i < 4; i++) absorb(w[i]); }

    // sumcheck.rs:147-171 — digest, reseed with the digest, first 8-byte LE window below
    // 2^64-4 reduced mod p.
    F squeeze() {
        const uint64_t ACCEPT = UINT64_MAX - 3;
        for (;;) {
            auto d = hasher.finalize_reset();
            hasher.update(d.data(), 32);
            for (int c = 0; c < 4; c++) {
                uint64_t raw = 0;
                for (int i = 7; i >= 0; i--) raw = (raw << 8) | d[c * 8 + i];
                if (raw < ACCEPT) return F(uint32_t(raw % P31));
            }
        }
    }
    VF squeeze_many(size_t n) { VF o; o.reserve(n); for (size_t i = 0; i < n; i++) o.push_back(squeeze()); return o; }
    // sumcheck.rs:182-188
    EF squeeze_ef() {
        F c0 = squeeze(), c1 = squeeze(), c2 = squeeze(), c3 = squeeze();
        return EF(C(c0, c1), C(c2, c3));
    }
    VEF squeeze_ef_many(size_t n) { VEF o; o.reserve(n); for (size_t i = 0; i < n; i++) o.push_back(squeeze_ef()); return o; }
};

}  // namespace zko
