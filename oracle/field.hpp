// CPU ORACLE — TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links or calls this.
//
// Mersenne-31 base field F and the degree-4 extension EF = M31[i]/(i^2+1) [Y]/(Y^2-(2+i)).
//
// The reference takes both from un-vendored crates (p3-mersenne-31 0.2.0, p3-field 0.2.0;
// rust/zk_ml_prover/Cargo.lock) and names the tower only in a comment
// (rust/zk_ml_prover/src/proving/sumcheck.rs:19-21: "M31 -> Complex<M31> (x^2+1) -> EF (y^2-(2+i))").
// The wire order of the four coordinates is [re(c0), im(c0), re(c1), im(c1)]
// (sumcheck.rs:67-96).  Field results are canonical ([0,p)), so any correct algorithm
// reproduces the crate's values; the non-residue W = 2+i itself is "parity unpinned"
// (no literal test vector in the reference exercises an EF product).
#pragma once
#include <cstdint>
#include <cstddef>
#include <vector>
#include <array>
#include <thread>

namespace zko {

constexpr uint32_t P31 = 0x7fffffffu;

// rust/zk_ml_prover/src/field/m31_ops.rs:125-138 (reduce_u64_m31): fold 31-bit limbs.
inline uint32_t reduce64(uint64_t v) {
    uint64_t s = (v & P31) + ((v >> 31) & P31) + (v >> 62);
    uint32_t lo = uint32_t(s & P31), hi = uint32_t(s >> 31);
    uint32_t t = lo + hi;
    return t >= P31 ? t - P31 : t;
}

struct F {
    uint32_t v;  // canonical, [0, p)
    F() : v(0) {}
    explicit F(uint32_t x) : v(x) {}  // caller guarantees x < p
    static F zero() { return F(0); }
    static F one() { return F(1); }
    static F two() { return F(2); }
    static F from_u64(uint64_t x) { return F(reduce64(x)); }
    bool operator==(const F& o) const { return v == o.v; }
    bool operator!=(const F& o) const { return v != o.v; }
};
inline F operator+(F a, F b) { uint32_t s = a.v + b.v; return F(s >= P31 ? s - P31 : s); }
inline F operator-(F a, F b) { return F(a.v >= b.v ? a.v - b.v : a.v + P31 - b.v); }
inline F operator*(F a, F b) { return F(reduce64(uint64_t(a.v) * b.v)); }
inline F neg(F a) { return F(a.v == 0 ? 0 : P31 - a.v); }
inline F& operator+=(F& a, F b) { a = a + b; return a; }
inline F& operator-=(F& a, F b) { a = a - b; return a; }
inline F& operator*=(F& a, F b) { a = a * b; return a; }

inline F pow(F a, uint64_t e) {
    F r = F::one();
    while (e) { if (e & 1) r = r * a; a = a * a; e >>= 1; }
    return r;
}
// a^(p-2); inverse(0) is undefined in the reference (p3 panics) — callers never pass 0.
inline F inverse(F a) { return pow(a, uint64_t(P31) - 2); }

// rust/zk_ml_prover/src/field/m31_ops.rs:98-105 (to_field): signed integer -> F.
inline F to_field(int64_t x) {
    if (x >= 0) return F(uint32_t(uint64_t(x) % P31));
    uint64_t pos = uint64_t(-x) % P31;
    return F::zero() - F(uint32_t(pos));
}
// m31_ops.rs:108-116 (from_field): centered representative.
inline int64_t from_field(F x) {
    uint32_t half = P31 / 2;
    return x.v > half ? int64_t(x.v) - int64_t(P31) : int64_t(x.v);
}

// Complex<M31> = a + b i, i^2 = -1.
struct C {
    F re, im;
    C() {}
    C(F r, F i) : re(r), im(i) {}
    bool operator==(const C& o) const { return re == o.re && im == o.im; }
};
inline C operator+(C a, C b) { return C(a.re + b.re, a.im + b.im); }
inline C operator-(C a, C b) { return C(a.re - b.re, a.im - b.im); }
inline C operator*(C a, C b) { return C(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re); }
inline C cinv(C a) {
    F n = inverse(a.re * a.re + a.im * a.im);
    return C(a.re * n, neg(a.im) * n);
}
// W = 2 + i, the quadratic non-residue of Complex<M31> that defines EF.
inline C mul_w(C a) {
    // (2+i)(x+yi) = (2x - y) + (x + 2y) i
    return C(a.re + a.re - a.im, a.re + a.im + a.im);
}

// EF = c0 + c1 Y, Y^2 = W.
struct EF {
    C c0, c1;
    EF() {}
    EF(C a, C b) : c0(a), c1(b) {}
    static EF zero() { return EF(); }
    static EF one() { return EF(C(F::one(), F::zero()), C()); }
    static EF two() { return EF(C(F::two(), F::zero()), C()); }
    static EF from_f(F x) { return EF(C(x, F::zero()), C()); }  // m31_ops.rs:149-151 f_to_ef
    static EF from_u32x4(const uint32_t* w) {                  // sumcheck.rs:85-95 EFElement::to_ef
        return EF(C(F(w[0]), F(w[1])), C(F(w[2]), F(w[3])));
    }
    void to_u32x4(uint32_t* w) const {                          // sumcheck.rs:73-83 EFElement::from_ef
        w[0] = c0.re.v; w[1] = c0.im.v; w[2] = c1.re.v; w[3] = c1.im.v;
    }
    std::array<uint32_t, 4> arr() const { return {c0.re.v, c0.im.v, c1.re.v, c1.im.v}; }
    bool operator==(const EF& o) const { return c0 == o.c0 && c1 == o.c1; }
    bool operator!=(const EF& o) const { return !(*this == o); }
};
inline EF operator+(EF a, EF b) { return EF(a.c0 + b.c0, a.c1 + b.c1); }
inline EF operator-(EF a, EF b) { return EF(a.c0 - b.c0, a.c1 - b.c1); }
inline EF operator*(EF a, EF b) {
    return EF(a.c0 * b.c0 + mul_w(a.c1 * b.c1), a.c0 * b.c1 + a.c1 * b.c0);
}
inline EF operator*(EF a, F b) {
    return EF(C(a.c0.re * b, a.c0.im * b), C(a.c1.re * b, a.c1.im * b));
}
inline EF& operator+=(EF& a, EF b) { a = a + b; return a; }
inline EF& operator-=(EF& a, EF b) { a = a - b; return a; }
inline EF& operator*=(EF& a, EF b) { a = a * b; return a; }
inline EF neg(EF a) { return EF::zero() - a; }
// (c0 + c1 Y)^-1 = (c0 - c1 Y) / (c0^2 - W c1^2)
inline EF inverse(EF a) {
    C d = cinv(a.c0 * a.c0 - mul_w(a.c1 * a.c1));
    return EF(a.c0 * d, (C() - a.c1) * d);
}

using VF = std::vector<F>;

using VEF = std::vector<EF>;

// Data-parallel helper.  The reference splits these loops over rayon workers: matrix rows
// (transformer/mod.rs:141-150, matmul.rs:81-120, 770-832), Merkle layers of at least 256 nodes
// (pcs.rs:158-190).  Here a plain thread count, set by whoever times the oracle (1 = serial, the
// default).  Results do not depend on it.
inline int& matrix_threads() { static int n = 1; return n; }
inline bool& par_nested() { static thread_local bool n = false; return n; }
template <class Fn>
inline void par_rows(size_t rows, Fn fn) {          // fn(lo, hi, worker)
    bool& nested = par_nested();                    // a worker's own par_rows calls run in that worker
    const int T = matrix_threads();
    if (T <= 1 || rows < 64 || nested) { fn(size_t(0), rows, 0); return; }
    std::vector<std::thread> th;
    const size_t per = (rows + T - 1) / T;
    for (int t = 0; t < T; t++) {
        size_t lo = size_t(t) * per, hi = lo + per < rows ? lo + per : rows;
        if (lo < hi) th.emplace_back([&fn, lo, hi, t] { par_nested() = true; fn(lo, hi, t); });
    }
    for (auto& x : th) x.join();
}

}  // namespace zko
