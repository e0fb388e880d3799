// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Multilinear-extension helpers, restating rust/zk_ml_prover/src/field/m31_ops.rs and
// rust/zk_ml_prover/src/field/common.rs.  Variable 0 is the most significant index bit.
#pragma once
#include "field.hpp"
#include "hash.hpp"

namespace zko {

// common.rs:16-21 — ceil(log2 n), minimum 1.
inline size_t log2_ceil(size_t n) {
    if (n <= 1) return 1;
    size_t k = 0;
    while ((size_t(1) << k) < n) k++;
    return k;
}

// m31_ops.rs:11-26
inline F mle_evaluate(const VF& evals, const VF& point) {
    VF t = evals;
    size_t size = t.size();
    for (size_t i = 0; i < point.size(); i++) {
        size_t half = size / 2;
        F r = point[i], omr = F::one() - r;
        for (size_t j = 0; j < half; j++) t[j] = omr * t[j] + r * t[j + half];
        size = half;
    }
    return t[0];
}

// m31_ops.rs:30-50 — out[2j] = in[j](1-r_i), out[2j+1] = in[j] r_i, r[0] = MSB.
inline VF eq_evals(const VF& r) {
    size_t k = r.size(), n = size_t(1) << k;
    VF e(n, F::one());
    size_t populated = 1;
    for (size_t i = 0; i < k; i++) {
        F ri = r[i], omr = F::one() - ri;
        for (size_t j = populated; j-- > 0;) {
            e[2 * j + 1] = e[j] * ri;
            e[2 * j] = e[j] * omr;
        }
        populated *= 2;
    }
    return e;
}

// m31_ops.rs:155-171
inline EF mle_evaluate_ef(const VF& evals, const VEF& point) {
    VEF t(evals.size());
    for (size_t i = 0; i < evals.size(); i++) t[i] = EF::from_f(evals[i]);
    size_t size = t.size();
    for (size_t i = 0; i < point.size(); i++) {
        size_t half = size / 2;
        EF r = point[i], omr = EF::one() - r;
        for (size_t j = 0; j < half; j++) t[j] = omr * t[j] + r * t[j + half];
        size = half;
    }
    return t[0];
}
// Same fold over a table that already lives in EF (used by the verifier restatements).
inline EF mle_evaluate_efef(const VEF& evals, const VEF& point) {
    VEF t = evals;
    size_t size = t.size();
    for (size_t i = 0; i < point.size(); i++) {
        size_t half = size / 2;
        EF r = point[i], omr = EF::one() - r;
        for (size_t j = 0; j < half; j++) t[j] = omr * t[j] + r * t[j + half];
        size = half;
    }
    return t[0];
}

// m31_ops.rs:175-191
inline VEF eq_evals_ef(const VEF& r) {
    size_t k = r.size(), n = size_t(1) << k;
    VEF e(n, EF::one());
    size_t populated = 1;
    for (size_t i = 0; i < k; i++) {
        EF ri = r[i], omr = EF::one() - ri;
        for (size_t j = populated; j-- > 0;) {
            e[2 * j + 1] = e[j] * ri;
            e[2 * j] = e[j] * omr;
        }
        populated *= 2;
    }
    return e;
}

// common.rs:24-30
inline F compute_eq_at_point(const VF& a, const VF& b) {
    F r = F::one();
    for (size_t i = 0; i < a.size() && i < b.size(); i++)
        r *= a[i] * b[i] + (F::one() - a[i]) * (F::one() - b[i]);
    return r;
}
// common.rs:91-97
inline EF compute_eq_at_point_ef(const VEF& a, const VEF& b) {
    EF r = EF::one();
    for (size_t i = 0; i < a.size() && i < b.size(); i++)
        r *= a[i] * b[i] + (EF::one() - a[i]) * (EF::one() - b[i]);
    return r;
}

// common.rs:34-40 — a^(2^29) = a^((p+1)/4).
inline F mod_sqrt_m31(F a) { F r = a; for (int i = 0; i < 29; i++) r = r * r; return r; }
// common.rs:44-53 — Euler criterion.
inline bool is_qr_m31(F a) {
    if (a == F::zero()) return true;
    F r = a;
    for (int i = 0; i < 30; i++) r = r * r;
    return r * inverse(a) == F::one();
}

// common.rs:78-85 — SHA-256(len u32 LE || values u32 LE).
inline std::array<uint8_t, 32> hash_values(const std::vector<uint32_t>& v) {
    Sha256 h;
    uint32_t n = uint32_t(v.size());
    uint8_t b[4] = {uint8_t(n), uint8_t(n >> 8), uint8_t(n >> 16), uint8_t(n >> 24)};
    h.update(b, 4);
    for (uint32_t x : v) {
        uint8_t c[4] = {uint8_t(x), uint8_t(x >> 8), uint8_t(x >> 16), uint8_t(x >> 24)};
        h.update(c, 4);
    }
    return h.finalize_reset();
}

}  // namespace zko
