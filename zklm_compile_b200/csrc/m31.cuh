// Mersenne-31 and M31^4 arithmetic for device code.
//
// F  = integers mod p = 2^31 - 1, canonical representatives in [0, p).
// EF = F[i]/(i^2+1) [Y]/(Y^2 - (2+i)); coordinates (x, y, z, w) = re(c0), im(c0), re(c1), im(c1),
//      the wire order of the reference's EFElement (rust/zk_ml_prover/src/proving/sumcheck.rs:67-96).
// Products go through a 32x32->64-bit multiply and a Mersenne fold (2^31 == 1 mod p); the EF
// product sums its sixteen partial products in 64-bit accumulators and folds six times instead
// of sixteen.  Every function returns canonical values, so results are independent of schedule.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace zkb {

typedef uint32_t u32;
typedef uint64_t u64;

#define ZKB_P 0x7fffffffu
#define ZKB_HD __host__ __device__ __forceinline__

struct Fp { u32 v; };
struct Fe { u32 x, y, z, w; };

// ---- base field ---------------------------------------------------------------------------
// The final conditional subtraction is an unsigned min (two instructions).  Measured on B200:
// folding with 2^32 == 2 through a 64-bit multiply-add is slower than the three-limb fold below
// (the wide multiply pipe is the scarce one), so reductions stay shift/mask/add.
ZKB_HD u32 umin32(u32 a, u32 b) { return a < b ? a : b; }
ZKB_HD u32 add31(u32 a, u32 b) { u32 s = a + b; return umin32(s, s - ZKB_P); }          // a, b < p
ZKB_HD u32 sub31(u32 a, u32 b) { u32 d = a - b; return umin32(d, d + ZKB_P); }          // a, b < p
ZKB_HD u32 neg31(u32 a) { return a ? ZKB_P - a : 0u; }
// Any 64-bit value -> canonical: v = lo + mid 2^31 + hi 2^62 == lo + mid + hi.
ZKB_HD u32 red64(u64 v) {
    u32 lo = (u32)v & ZKB_P;
    u32 mid = (u32)(v >> 31) & ZKB_P;
    u32 hi = (u32)(v >> 62);
    u32 s = lo + mid;                       // <= 2^32 - 2
    s = (s & ZKB_P) + (s >> 31) + hi;       // <= 2^31 + 3
    return umin32(s, s - ZKB_P);
}
// Product of two values below 2^32 whose product is below 2^63 (canonical inputs: < 2^62).
ZKB_HD u32 mul31(u32 a, u32 b) { return red64((u64)a * b); }
ZKB_HD u32 pow31(u32 a, u32 e) {
    u32 r = 1;
    while (e) { if (e & 1) r = mul31(r, a); a = mul31(a, a); e >>= 1; }
    return r;
}
ZKB_HD u32 inv31(u32 a) { return pow31(a, ZKB_P - 2); }

ZKB_HD Fp operator+(Fp a, Fp b) { return Fp{add31(a.v, b.v)}; }
ZKB_HD Fp operator-(Fp a, Fp b) { return Fp{sub31(a.v, b.v)}; }
ZKB_HD Fp operator*(Fp a, Fp b) { return Fp{mul31(a.v, b.v)}; }
ZKB_HD Fp fp_zero() { return Fp{0}; }
ZKB_HD Fp fp_one() { return Fp{1}; }

// ---- extension field ----------------------------------------------------------------------
ZKB_HD Fe fe_zero() { return Fe{0, 0, 0, 0}; }
ZKB_HD Fe fe_one() { return Fe{1, 0, 0, 0}; }
ZKB_HD Fe fe_from(Fp a) { return Fe{a.v, 0, 0, 0}; }
ZKB_HD Fe operator+(Fe a, Fe b) { return Fe{add31(a.x, b.x), add31(a.y, b.y), add31(a.z, b.z), add31(a.w, b.w)}; }
ZKB_HD Fe operator-(Fe a, Fe b) { return Fe{sub31(a.x, b.x), sub31(a.y, b.y), sub31(a.z, b.z), sub31(a.w, b.w)}; }
ZKB_HD Fe operator*(Fe a, Fp b) { return Fe{mul31(a.x, b.v), mul31(a.y, b.v), mul31(a.z, b.v), mul31(a.w, b.v)}; }
ZKB_HD Fe operator*(Fp b, Fe a) { return a * b; }
ZKB_HD bool fe_eq(Fe a, Fe b) { return a.x == b.x && a.y == b.y && a.z == b.z && a.w == b.w; }

// (c0 + c1 Y)(d0 + d1 Y) = (c0 d0 + W c1 d1) + (c0 d1 + c1 d0) Y, W = 2 + i.
ZKB_HD Fe operator*(Fe a, Fe b) {
    const u32 nby = ZKB_P - b.y, nbw = ZKB_P - b.w;   // in [1, p]; a*p == 0 mod p
    // u + v i = c1 * d1
    u32 u = red64((u64)a.z * b.z + (u64)a.w * nbw);
    u32 v = red64((u64)a.z * b.w + (u64)a.w * b.z);
    // W (u + v i) = (2u - v) + (u + 2v) i
    u64 r0 = (u64)a.x * b.x + (u64)a.y * nby + (u64)u + u + (ZKB_P - v);
    u64 r1 = (u64)a.x * b.y + (u64)a.y * b.x + (u64)u + v + v;
    u64 r2 = (u64)a.x * b.z + (u64)a.y * nbw + (u64)a.z * b.x + (u64)a.w * nby;
    u64 r3 = (u64)a.x * b.w + (u64)a.y * b.z + (u64)a.z * b.y + (u64)a.w * b.x;
    return Fe{red64(r0), red64(r1), red64(r2), red64(r3)};
}
// Complex<M31> helpers for the inverse.
ZKB_HD void cmul(u32 ar, u32 ai, u32 br, u32 bi, u32& cr, u32& ci) {
    cr = sub31(mul31(ar, br), mul31(ai, bi));
    ci = add31(mul31(ar, bi), mul31(ai, br));
}
// (c0 + c1 Y)^-1 = (c0 - c1 Y) / (c0^2 - W c1^2); the denominator is a Complex<M31>.
ZKB_HD Fe fe_inv(Fe a) {
    u32 sr, si, tr, ti;
    cmul(a.x, a.y, a.x, a.y, sr, si);          // c0^2
    cmul(a.z, a.w, a.z, a.w, tr, ti);          // c1^2
    u32 wr = sub31(add31(tr, tr), ti), wi = add31(tr, add31(ti, ti));   // W c1^2
    u32 dr = sub31(sr, wr), di = sub31(si, wi);
    u32 n = inv31(add31(mul31(dr, dr), mul31(di, di)));
    u32 ir = mul31(dr, n), ii = mul31(neg31(di), n);                    // 1 / (dr + di i)
    Fe o;
    cmul(a.x, a.y, ir, ii, o.x, o.y);
    cmul(neg31(a.z), neg31(a.w), ir, ii, o.z, o.w);
    return o;
}

// ---- mixed helpers used by the fold / reduce kernels --------------------------------------
// Challenge type x table type -> folded type: (Fp,Fp)->Fp, (Fe,Fp)->Fe, (Fe,Fe)->Fe.
// lerp(a, b, r) = (1 - r) a + r b = a + r (b - a), the reference's fold
// (rust/zk_ml_prover/src/proving/sumcheck.rs:256-260, 1245-1249).
ZKB_HD Fp lerp(Fp a, Fp b, Fp r) { return a + r * (b - a); }
ZKB_HD Fe lerp(Fe a, Fe b, Fe r) { return a + r * (b - a); }
ZKB_HD Fe lerp(Fp a, Fp b, Fe r) {
    Fe t = r * (b - a);
    t.x = add31(t.x, a.v);
    return t;
}
ZKB_HD Fp dbl_minus(Fp hi, Fp lo) { return hi + hi - lo; }   // value at t = 2
ZKB_HD Fe dbl_minus(Fe hi, Fe lo) { return hi + hi - lo; }

// Programmatic dependent launch.  A kernel launched with the attribute (zkb::launch_pdl) may start
// while its predecessor in the stream is still running: everything before pdl_wait() must not
// touch what the predecessor writes (weights may be prefetched, nothing else), everything after it
// sees the predecessor's memory complete.  pdl_launch_dependents() lets the successor start early.
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// First statements of the small kernels of a forward chain (norm, requantise, lookup, add), whose
// input comes from the kernel before them and whose successor is a matvec that prefetches its weights.
// (Releasing the successor before the wait, so that it becomes resident while the matvec in front is
// still draining, measured slower: 170 against 162 us per layer of the 4B shape.)
__device__ __forceinline__ void pdl_small_prologue() {
    pdl_wait();                  // the input comes from the kernel before this one
    pdl_launch_dependents();     // only now: the next matvec may start pulling its weights into L2 while this small kernel runs
}

// 16-byte vector load / store of an EF element.
__device__ __forceinline__ Fe ld_fe(const Fe* p) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    return Fe{t.x, t.y, t.z, t.w};
}
__device__ __forceinline__ void st_fe(Fe* p, Fe v) {
    *reinterpret_cast<uint4*>(p) = make_uint4(v.x, v.y, v.z, v.w);
}
__device__ __forceinline__ Fp ld_fe(const Fp* p) { return *p; }
__device__ __forceinline__ void st_fe(Fp* p, Fp v) { *p = v; }

}  // namespace zkb
