// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// SHA-256 (FIPS 180-4) and BLAKE3 (hash + extendable output, from the public BLAKE3
// specification), written out here because the reference takes them from un-vendored
// crates (sha2 0.10.9, blake3 1.8.3; rust/zk_ml_prover/Cargo.lock).  Both are pinned by
// the tests against Python's hashlib and the `blake3` wheel.
#pragma once
#include <cstdint>
#include <cstring>
#include <vector>
#include <array>
#include <algorithm>

namespace zko {

// ----------------------------------------------------------------------------- SHA-256
struct Sha256 {
    uint32_t h[8];
    uint8_t buf[64];
    uint32_t buflen;
    uint64_t total;

    Sha256() { reset(); }
    void reset() {
        static const uint32_t iv[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                                       0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
        memcpy(h, iv, sizeof h);
        buflen = 0;
        total = 0;
    }
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void compress(const uint8_t* p) {
        static const uint32_t K[64] = {
            0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
            0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
            0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
            0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
            0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
            0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
            0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
            0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; i++)
            w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
        for (int i = 16; i < 64; i++) {
            uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; i++) {
            uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
            uint32_t ch = (e & f) ^ (~e & g);
            uint32_t t1 = hh + S1 + ch + K[i] + w[i];
            uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
            uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
            uint32_t t2 = S0 + mj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const void* data, size_t len) {
        const uint8_t* p = static_cast<const uint8_t*>(data);
        total += len;
        if (buflen) {
            size_t take = std::min<size_t>(64 - buflen, len);
            memcpy(buf + buflen, p, take);
            buflen += uint32_t(take); p += take; len -= take;
            if (buflen == 64) { compress(buf); buflen = 0; }
        }
        while (len >= 64) { compress(p); p += 64; len -= 64; }
        if (len) { memcpy(buf, p, len); buflen = uint32_t(len); }
    }
    // Digest of everything absorbed so far; the object is left reset (sha2's finalize_reset).
    std::array<uint8_t, 32> finalize_reset() {
        uint64_t bits = total * 8;
        uint8_t pad[72];
        size_t padlen = (buflen < 56) ? (56 - buflen) : (120 - buflen);
        memset(pad, 0, sizeof pad);
        pad[0] = 0x80;
        for (int i = 0; i < 8; i++) pad[padlen + i] = uint8_t(bits >> (56 - 8 * i));
        update(pad, padlen + 8);
        std::array<uint8_t, 32> out;
        for (int i = 0; i < 8; i++) {
            out[4 * i] = uint8_t(h[i] >> 24); out[4 * i + 1] = uint8_t(h[i] >> 16);
            out[4 * i + 2] = uint8_t(h[i] >> 8); out[4 * i + 3] = uint8_t(h[i]);
        }
        reset();
        return out;
    }
};

inline std::array<uint8_t, 32> sha256(const void* data, size_t len) {
    Sha256 s; s.update(data, len); return s.finalize_reset();
}

// ----------------------------------------------------------------------------- BLAKE3
namespace b3 {
constexpr uint32_t IV[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                            0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
constexpr uint8_t PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum : uint32_t { CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8 };

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
    s[a] = s[a] + s[b] + mx; s[d] = rotr(s[d] ^ s[a], 16);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 12);
    s[a] = s[a] + s[b] + my; s[d] = rotr(s[d] ^ s[a], 8);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 7);
}
// Full 16-word compression output.
inline void compress(const uint32_t cv[8], const uint32_t block[16], uint64_t counter, uint32_t blen,
                     uint32_t flags, uint32_t out[16]) {
    uint32_t s[16] = {cv[0], cv[1], cv[2], cv[3], cv[4], cv[5], cv[6], cv[7],
                      IV[0], IV[1], IV[2], IV[3], uint32_t(counter), uint32_t(counter >> 32), blen, flags};
    uint32_t m[16];
    memcpy(m, block, sizeof m);
    for (int r = 0; r < 7; r++) {
        g(s, 0, 4, 8, 12, m[0], m[1]);   g(s, 1, 5, 9, 13, m[2], m[3]);
        g(s, 2, 6, 10, 14, m[4], m[5]);  g(s, 3, 7, 11, 15, m[6], m[7]);
        g(s, 0, 5, 10, 15, m[8], m[9]);  g(s, 1, 6, 11, 12, m[10], m[11]);
        g(s, 2, 7, 8, 13, m[12], m[13]); g(s, 3, 4, 9, 14, m[14], m[15]);
        uint32_t t[16];
        for (int i = 0; i < 16; i++) t[i] = m[PERM[i]];
        memcpy(m, t, sizeof m);
    }
    for (int i = 0; i < 8; i++) { out[i] = s[i] ^ s[i + 8]; out[i + 8] = s[i + 8] ^ cv[i]; }
}
inline void load_block(const uint8_t* p, size_t len, uint32_t w[16]) {
    uint8_t tmp[64];
    memset(tmp, 0, 64);
    memcpy(tmp, p, len);
    for (int i = 0; i < 16; i++)
        w[i] = uint32_t(tmp[4 * i]) | (uint32_t(tmp[4 * i + 1]) << 8) | (uint32_t(tmp[4 * i + 2]) << 16) | (uint32_t(tmp[4 * i + 3]) << 24);
}
// The last compression of a subtree, kept un-run so ROOT can be OR-ed in and so the
// extendable output can re-run it with increasing counters.
struct Output {
    uint32_t cv[8];
    uint32_t block[16];
    uint64_t counter;
    uint32_t blen, flags;
    void chaining(uint32_t out8[8]) const {
        uint32_t o[16];
        compress(cv, block, counter, blen, flags, o);
        memcpy(out8, o, 32);
    }
    void root_bytes(uint8_t* out, size_t n) const {
        uint64_t c = 0;
        size_t off = 0;
        while (off < n) {
            uint32_t o[16];
            compress(cv, block, c++, blen, flags | ROOT, o);
            for (int i = 0; i < 16 && off < n; i++)
                for (int b = 0; b < 4 && off < n; b++) out[off++] = uint8_t(o[i] >> (8 * b));
        }
    }
};
inline Output chunk_output(const uint8_t* p, size_t len, uint64_t chunk_index) {
    Output o;
    memcpy(o.cv, IV, 32);
    size_t nblocks = len == 0 ? 1 : (len + 63) / 64;
    for (size_t b = 0; b < nblocks; b++) {
        size_t bl = std::min<size_t>(64, len - b * 64);
        uint32_t w[16];
        load_block(p + b * 64, bl, w);
        uint32_t fl = (b == 0 ? CHUNK_START : 0) | (b + 1 == nblocks ? CHUNK_END : 0);
        if (b + 1 == nblocks) {
            memcpy(o.block, w, 64);
            o.counter = chunk_index; o.blen = uint32_t(bl); o.flags = fl;
        } else {
            uint32_t out[16];
            compress(o.cv, w, chunk_index, 64, fl, out);
            memcpy(o.cv, out, 32);
        }
    }
    return o;
}
inline Output subtree(const uint8_t* p, size_t len, uint64_t chunk_index) {
    if (len <= 1024) return chunk_output(p, len, chunk_index);
    // left subtree: the largest power-of-two number of whole chunks that leaves >= 1 byte right.
    size_t chunks = (len + 1023) / 1024;
    size_t left_chunks = 1;
    while (left_chunks * 2 < chunks) left_chunks *= 2;
    size_t left_len = left_chunks * 1024;
    Output l = subtree(p, left_len, chunk_index);
    Output r = subtree(p + left_len, len - left_len, chunk_index + left_chunks);
    Output o;
    memcpy(o.cv, IV, 32);
    l.chaining(o.block);
    r.chaining(o.block + 8);
    o.counter = 0; o.blen = 64; o.flags = PARENT;
    return o;
}
}  // namespace b3

// blake3(data) with `n` output bytes (n = 32: the plain hash; larger: the XOF stream).
inline void blake3_xof(const void* data, size_t len, uint8_t* out, size_t n) {
    b3::subtree(static_cast<const uint8_t*>(data), len, 0).root_bytes(out, n);
}
inline std::array<uint8_t, 32> blake3(const void* data, size_t len) {
    std::array<uint8_t, 32> o;
    blake3_xof(data, len, o.data(), 32);
    return o;
}
inline std::array<uint8_t, 32> blake3(const std::vector<uint8_t>& v) { return blake3(v.data(), v.size()); }

}  // namespace zko
