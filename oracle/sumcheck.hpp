// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Product / triple / all-ones sumcheck provers and verifiers, restating
// rust/zk_ml_prover/src/proving/sumcheck.rs (base field :211-1157, extension field
// :1163-1553) and prove_product_ef_mixed from rust/zk_ml_prover/src/proving/matmul.rs:889-944.
// The reference's rayon ("_parallel") and Metal ("_gpu") variants produce the same proofs as
// the sequential ones (sumcheck.rs:1699-1886), so one sequential restatement covers all.
#pragma once
#include "field.hpp"
#include "transcript.hpp"

namespace zko {

using EFElement = std::array<uint32_t, 4>;

// sumcheck.rs:57-65
struct SumcheckProof {
    std::vector<std::vector<uint32_t>> round_polys;
    std::vector<uint32_t> challenges;
};
// sumcheck.rs:99-107
struct SumcheckProofEF {
    std::vector<std::vector<EFElement>> round_polys;
    std::vector<EFElement> challenges;
};

template <class T> inline void fold_table(std::vector<T>& t, size_t half, T r) {
    T omr = T::one() - r;
    for (size_t j = 0; j < half; j++) t[j] = omr * t[j] + r * t[j + half];
}

// ---------------------------------------------------------------- base field provers
struct Prod { SumcheckProof proof; F f_at_s, g_at_s; };
struct Trip { SumcheckProof proof; F f_at_s, g_at_s, h_at_s; };

// sumcheck.rs:211-272 (== prove_product_parallel :389-482 == prove_product_best :815-828)
inline Prod prove_product(const VF& f_in, const VF& g_in, size_t num_vars, Transcript& tr) {
    VF f = f_in, g = g_in;
    size_t size = f.size();
    Prod out;
    for (size_t rd = 0; rd < num_vars; rd++) {
        size_t half = size / 2;
        F s0, s1, s2;
        for (size_t j = 0; j < half; j++) {
            F f0 = f[j], f1 = f[j + half], g0 = g[j], g1 = g[j + half];
            s0 += f0 * g0;
            s1 += f1 * g1;
            s2 += (f1 + f1 - f0) * (g1 + g1 - g0);
        }
        out.proof.round_polys.push_back({s0.v, s1.v, s2.v});
        tr.absorb(s0); tr.absorb(s1); tr.absorb(s2);
        F r = tr.squeeze();
        fold_table(f, half, r);
        fold_table(g, half, r);
        out.proof.challenges.push_back(r.v);
        size = half;
    }
    out.f_at_s = f[0]; out.g_at_s = g[0];
    return out;
}

// sumcheck.rs:277-354 (== prove_triple_parallel :487-619 == prove_triple_best :831-845)
inline Trip prove_triple(const VF& f_in, const VF& g_in, const VF& h_in, size_t num_vars, Transcript& tr) {
    VF f = f_in, g = g_in, h = h_in;
    size_t size = f.size();
    Trip out;
    const F three(3), two(2);
    for (size_t rd = 0; rd < num_vars; rd++) {
        size_t half = size / 2;
        F s0, s1, s2, s3;
        for (size_t j = 0; j < half; j++) {
            F f0 = f[j], f1 = f[j + half], g0 = g[j], g1 = g[j + half], h0 = h[j], h1 = h[j + half];
            s0 += f0 * g0 * h0;
            s1 += f1 * g1 * h1;
            s2 += (f1 + f1 - f0) * (g1 + g1 - g0) * (h1 + h1 - h0);
            s3 += (three * f1 - two * f0) * (three * g1 - two * g0) * (three * h1 - two * h0);
        }
        out.proof.round_polys.push_back({s0.v, s1.v, s2.v, s3.v});
        tr.absorb(s0); tr.absorb(s1); tr.absorb(s2); tr.absorb(s3);
        F r = tr.squeeze();
        fold_table(f, half, r); fold_table(g, half, r); fold_table(h, half, r);
        out.proof.challenges.push_back(r.v);
        size = half;
    }
    out.f_at_s = f[0]; out.g_at_s = g[0]; out.h_at_s = h[0];
    return out;
}

// sumcheck.rs:857-902 (== _parallel :906-968 == _best :971-978): f == 1, stores [s0, s2].
inline Prod prove_product_ones(const VF& g_in, size_t num_vars, Transcript& tr) {
    VF g = g_in;
    size_t size = g.size();
    Prod out;
    for (size_t rd = 0; rd < num_vars; rd++) {
        size_t half = size / 2;
        F s0, s1;
        for (size_t j = 0; j < half; j++) { s0 += g[j]; s1 += g[j + half]; }
        F s2 = s1 + s1 - s0;
        out.proof.round_polys.push_back({s0.v, s2.v});
        tr.absorb(s0); tr.absorb(s1); tr.absorb(s2);
        F r = tr.squeeze();
        fold_table(g, half, r);
        out.proof.challenges.push_back(r.v);
        size = half;
    }
    out.f_at_s = F::one(); out.g_at_s = g[0];
    return out;
}

// ---------------------------------------------------------------- base field verifiers
// sumcheck.rs:1122-1136
inline F interpolate_quadratic(F y0, F y1, F y2, F x) {
    F x0 = F::zero(), x1 = F::one(), x2 = F::two();
    F l0 = (x - x1) * (x - x2) * inverse(F::two());
    F l1 = (x - x0) * (x - x2) * inverse(F::zero() - F::one());
    F l2 = (x - x0) * (x - x1) * inverse(F::two());
    return y0 * l0 + y1 * l1 + y2 * l2;
}
// sumcheck.rs:1139-1157
inline F interpolate_cubic(const VF& ev, F x) {
    size_t n = ev.size();
    F res;
    for (size_t i = 0; i < n; i++) {
        F num = F::one(), den = F::one();
        for (size_t j = 0; j < n; j++) {
            if (j == i) continue;
            num *= x - F(uint32_t(j));
            den *= F(uint32_t(i)) - F(uint32_t(j));
        }
        res += ev[i] * num * inverse(den);
    }
    return res;
}

// sumcheck.rs:1019-1051 (verify_product :981-1014 is the same check without the point).
inline bool verify_product_with_challenges(F claimed, const SumcheckProof& p, F f_at_s, F g_at_s,
                                           Transcript& tr, VF* derived = nullptr) {
    F claim = claimed;
    for (size_t i = 0; i < p.round_polys.size(); i++) {
        const auto& raw = p.round_polys[i];
        F s0, s1, s2;
        if (raw.size() == 2) { s0 = F(raw[0]); s1 = claim - s0; s2 = F(raw[1]); }
        else { s0 = F(raw[0]); s1 = F(raw[1]); s2 = F(raw[2]); }
        if (s0 + s1 != claim) return false;
        tr.absorb(s0); tr.absorb(s1); tr.absorb(s2);
        F r = tr.squeeze();
        if (!p.challenges.empty() && r.v != p.challenges[i]) return false;
        if (derived) derived->push_back(r);
        claim = interpolate_quadratic(s0, s1, s2, r);
    }
    return claim == f_at_s * g_at_s;
}
// sumcheck.rs:1054-1119
inline bool verify_triple_with_challenges(F claimed, const SumcheckProof& p, F f_at_s, F g_at_s, F h_at_s,
                                          Transcript& tr, VF* derived = nullptr) {
    F claim = claimed;
    for (size_t i = 0; i < p.round_polys.size(); i++) {
        VF poly;
        for (uint32_t v : p.round_polys[i]) poly.push_back(F(v));
        if (poly[0] + poly[1] != claim) return false;
        for (F v : poly) tr.absorb(v);
        F r = tr.squeeze();
        if (!p.challenges.empty() && r.v != p.challenges[i]) return false;
        if (derived) derived->push_back(r);
        claim = interpolate_cubic(poly, r);
    }
    return claim == f_at_s * g_at_s * h_at_s;
}

// sumcheck.rs:981-1014, 1054-1119: the variants without the point - the proof's `challenges` field is not looked at.
inline bool verify_product(F claimed, const SumcheckProof& p, F f_at_s, F g_at_s, Transcript& tr) {
    SumcheckProof q;
    q.round_polys = p.round_polys;
    return verify_product_with_challenges(claimed, q, f_at_s, g_at_s, tr);
}
inline bool verify_triple(F claimed, const SumcheckProof& p, F f_at_s, F g_at_s, F h_at_s, Transcript& tr) {
    SumcheckProof q;
    q.round_polys = p.round_polys;
    return verify_triple_with_challenges(claimed, q, f_at_s, g_at_s, h_at_s, tr);
}

// ---------------------------------------------------------------- extension field provers
struct ProdEF { SumcheckProofEF proof; EF f_at_s, g_at_s; };
struct TripEF { SumcheckProofEF proof; EF f_at_s, g_at_s, h_at_s; };

inline VEF widen(const VF& v) { VEF o(v.size()); for (size_t i = 0; i < v.size(); i++) o[i] = EF::from_f(v[i]); return o; }

// Shared body of the three EF product provers; `full` selects [s0,s1,s2] vs [s0,s2].
inline ProdEF prove_product_ef_impl(VEF f, VEF g, size_t num_vars, Transcript& tr, bool full) {
    size_t size = f.size();
    ProdEF out;
    for (size_t rd = 0; rd < num_vars; rd++) {
        size_t half = size / 2;
        EF s0, s1, s2;
        for (size_t j = 0; j < half; j++) {
            EF f0 = f[j], f1 = f[j + half], g0 = g[j], g1 = g[j + half];
            s0 += f0 * g0;
            s1 += f1 * g1;
            s2 += (f1 + f1 - f0) * (g1 + g1 - g0);
        }
        if (full) out.proof.round_polys.push_back({s0.arr(), s1.arr(), s2.arr()});
        else out.proof.round_polys.push_back({s0.arr(), s2.arr()});
        tr.absorb_ef(s0); tr.absorb_ef(s1); tr.absorb_ef(s2);
        EF r = tr.squeeze_ef();
        fold_table(f, half, r);
        fold_table(g, half, r);
        out.proof.challenges.push_back(r.arr());
        size = half;
    }
    out.f_at_s = f[0]; out.g_at_s = g[0];
    return out;
}
// sumcheck.rs:1204-1258 — base inputs, compressed [s0,s2].
inline ProdEF prove_product_ef(const VF& f, const VF& g, size_t nv, Transcript& tr) {
    return prove_product_ef_impl(widen(f), widen(g), nv, tr, false);
}
// sumcheck.rs:1262-1315 — EF inputs, full [s0,s1,s2].
inline ProdEF prove_product_ef_full(const VEF& f, const VEF& g, size_t nv, Transcript& tr) {
    return prove_product_ef_impl(f, g, nv, tr, true);
}
// matmul.rs:889-944 — f in EF, g base (widened), full [s0,s1,s2].
inline ProdEF prove_product_ef_mixed(const VEF& f, const VF& g, size_t nv, Transcript& tr) {
    return prove_product_ef_impl(f, widen(g), nv, tr, true);
}

// sumcheck.rs:1318-1384 — stores [s0,s2,s3], absorbs all four; f3 = f2 + (f1 - f0).
inline TripEF prove_triple_ef_full(const VEF& f_in, const VEF& g_in, const VEF& h_in, size_t num_vars, Transcript& tr) {
    VEF f = f_in, g = g_in, h = h_in;
    size_t size = f.size();
    TripEF out;
    for (size_t rd = 0; rd < num_vars; rd++) {
        size_t half = size / 2;
        EF s0, s1, s2, s3;
        for (size_t j = 0; j < half; j++) {
            EF f0 = f[j], f1 = f[j + half], g0 = g[j], g1 = g[j + half], h0 = h[j], h1 = h[j + half];
            s0 += f0 * g0 * h0;
            s1 += f1 * g1 * h1;
            EF f2 = f1 + f1 - f0, g2 = g1 + g1 - g0, h2 = h1 + h1 - h0;
            s2 += f2 * g2 * h2;
            EF f3 = f2 + (f1 - f0), g3 = g2 + (g1 - g0), h3 = h2 + (h1 - h0);
            s3 += f3 * g3 * h3;
        }
        out.proof.round_polys.push_back({s0.arr(), s2.arr(), s3.arr()});
        tr.absorb_ef(s0); tr.absorb_ef(s1); tr.absorb_ef(s2); tr.absorb_ef(s3);
        EF r = tr.squeeze_ef();
        fold_table(f, half, r); fold_table(g, half, r); fold_table(h, half, r);
        out.proof.challenges.push_back(r.arr());
        size = half;
    }
    out.f_at_s = f[0]; out.g_at_s = g[0]; out.h_at_s = h[0];
    return out;
}

// sumcheck.rs:1389-1435 — f == 1, stores [s0,s2].
inline ProdEF prove_product_ones_ef_full(const VEF& g_in, size_t num_vars, Transcript& tr) {
    VEF g = g_in;
    size_t size = g.size();
    ProdEF out;
    for (size_t rd = 0; rd < num_vars; rd++) {
        size_t half = size / 2;
        EF s0, s1;
        for (size_t j = 0; j < half; j++) { s0 += g[j]; s1 += g[j + half]; }
        EF s2 = s1 + s1 - s0;
        out.proof.round_polys.push_back({s0.arr(), s2.arr()});
        tr.absorb_ef(s0); tr.absorb_ef(s1); tr.absorb_ef(s2);
        EF r = tr.squeeze_ef();
        fold_table(g, half, r);
        out.proof.challenges.push_back(r.arr());
        size = half;
    }
    out.f_at_s = EF::one(); out.g_at_s = g[0];
    return out;
}

// ---------------------------------------------------------------- extension field verifiers
// sumcheck.rs:1164-1178
inline EF interpolate_quadratic_ef(EF y0, EF y1, EF y2, EF x) {
    EF x0 = EF::zero(), x1 = EF::one(), x2 = EF::two();
    EF l0 = (x - x1) * (x - x2) * inverse(EF::two());
    EF l1 = (x - x0) * (x - x2) * inverse(EF::zero() - EF::one());
    EF l2 = (x - x0) * (x - x1) * inverse(EF::two());
    return y0 * l0 + y1 * l1 + y2 * l2;
}
// sumcheck.rs:1181-1197
inline EF interpolate_cubic_ef(const VEF& ev, EF x) {
    size_t n = ev.size();
    EF res;
    for (size_t i = 0; i < n; i++) {
        EF num = EF::one(), den = EF::one();
        for (size_t j = 0; j < n; j++) {
            if (j == i) continue;
            num *= x - EF::from_f(F(uint32_t(j)));
            den *= EF::from_f(F(uint32_t(i))) - EF::from_f(F(uint32_t(j)));
        }
        res += ev[i] * num * inverse(den);
    }
    return res;
}
inline EF ef_of(const EFElement& e) { return EF::from_u32x4(e.data()); }

// sumcheck.rs:1477-1512 (verify_product_ef :1439-1472 is the same check without the point).
inline bool verify_product_ef_with_challenges(EF claimed, const SumcheckProofEF& p, EF f_at_s, EF g_at_s,
                                              Transcript& tr, VEF* derived = nullptr) {
    EF claim = claimed;
    for (size_t i = 0; i < p.round_polys.size(); i++) {
        const auto& raw = p.round_polys[i];
        EF s0, s1, s2;
        if (raw.size() == 2) { s0 = ef_of(raw[0]); s1 = claim - s0; s2 = ef_of(raw[1]); }
        else if (raw.size() >= 3) { s0 = ef_of(raw[0]); s1 = ef_of(raw[1]); s2 = ef_of(raw[2]); }
        else return false;                                   // the reference indexes out of bounds and panics
        if (s0 + s1 != claim) return false;
        tr.absorb_ef(s0); tr.absorb_ef(s1); tr.absorb_ef(s2);
        EF r = tr.squeeze_ef();
        if (!p.challenges.empty() && (i >= p.challenges.size() || r.arr() != p.challenges[i])) return false;
        if (derived) derived->push_back(r);
        claim = interpolate_quadratic_ef(s0, s1, s2, r);
    }
    return claim == f_at_s * g_at_s;
}
// sumcheck.rs:1517-1553
inline bool verify_triple_ef_with_challenges(EF claimed, const SumcheckProofEF& p, EF f_at_s, EF g_at_s, EF h_at_s,
                                             Transcript& tr, VEF* derived = nullptr) {
    EF claim = claimed;
    for (size_t i = 0; i < p.round_polys.size(); i++) {
        const auto& raw = p.round_polys[i];
        EF s0, s1, s2, s3;
        if (raw.size() == 3) { s0 = ef_of(raw[0]); s1 = claim - s0; s2 = ef_of(raw[1]); s3 = ef_of(raw[2]); }
        else if (raw.size() >= 4) { s0 = ef_of(raw[0]); s1 = ef_of(raw[1]); s2 = ef_of(raw[2]); s3 = ef_of(raw[3]); }
        else return false;                                   // the reference indexes out of bounds and panics
        if (s0 + s1 != claim) return false;
        tr.absorb_ef(s0); tr.absorb_ef(s1); tr.absorb_ef(s2); tr.absorb_ef(s3);
        EF r = tr.squeeze_ef();
        if (!p.challenges.empty() && (i >= p.challenges.size() || r.arr() != p.challenges[i])) return false;
        if (derived) derived->push_back(r);
        claim = interpolate_cubic_ef({s0, s1, s2, s3}, r);
    }
    return claim == f_at_s * g_at_s * h_at_s;
}

}  // namespace zko
