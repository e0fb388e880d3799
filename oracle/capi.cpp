// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// Flat C entry points over the oracle headers so the Python tests (ctypes) and the CPU
// baseline leg of the benchmark can drive it.  Nothing in the shipped CUDA library links this.
#include "field.hpp"
#include "hash.hpp"
#include "transcript.hpp"
#include "mle.hpp"
#include "sumcheck.hpp"
#include <cstring>

using namespace zko;

static VF vf(const uint32_t* p, size_t n) { VF v(n); for (size_t i = 0; i < n; i++) v[i] = F(p[i]); return v; }
static VEF vef(const uint32_t* p, size_t n) { VEF v(n); for (size_t i = 0; i < n; i++) v[i] = EF::from_u32x4(p + 4 * i); return v; }
static void put(EF e, uint32_t* o) { e.to_u32x4(o); }

static void flatten(const SumcheckProof& p, uint32_t* polys, uint32_t* chal) {
    size_t k = 0;
    for (auto& r : p.round_polys) for (uint32_t v : r) polys[k++] = v;
    for (size_t i = 0; i < p.challenges.size(); i++) chal[i] = p.challenges[i];
}
static void flatten(const SumcheckProofEF& p, uint32_t* polys, uint32_t* chal) {
    size_t k = 0;
    for (auto& r : p.round_polys) for (auto& e : r) { memcpy(polys + k, e.data(), 16); k += 4; }
    for (size_t i = 0; i < p.challenges.size(); i++) memcpy(chal + 4 * i, p.challenges[i].data(), 16);
}

extern "C" {

// ---- field
void zko_f_mul(uint32_t a, uint32_t b, uint32_t* o) { *o = (F(a) * F(b)).v; }
void zko_f_inv(uint32_t a, uint32_t* o) { *o = inverse(F(a)).v; }
void zko_ef_mul(const uint32_t* a, const uint32_t* b, uint32_t* o) { put(EF::from_u32x4(a) * EF::from_u32x4(b), o); }
void zko_ef_inv(const uint32_t* a, uint32_t* o) { put(inverse(EF::from_u32x4(a)), o); }
void zko_to_field(int64_t x, uint32_t* o) { *o = to_field(x).v; }
int64_t zko_from_field(uint32_t x) { return from_field(F(x)); }
int zko_is_qr(uint32_t a) { return is_qr_m31(F(a)) ? 1 : 0; }
uint32_t zko_mod_sqrt(uint32_t a) { return mod_sqrt_m31(F(a)).v; }

// ---- hashes
void zko_sha256(const uint8_t* d, size_t n, uint8_t* out) { auto h = sha256(d, n); memcpy(out, h.data(), 32); }
void zko_blake3(const uint8_t* d, size_t n, uint8_t* out, size_t outlen) { blake3_xof(d, n, out, outlen); }
void zko_hash_values(const uint32_t* v, size_t n, uint8_t* out) {
    auto h = hash_values(std::vector<uint32_t>(v, v + n)); memcpy(out, h.data(), 32);
}

// ---- transcript
void* zko_tr_new(const uint8_t* label, size_t n) { return new Transcript(label, n); }
void zko_tr_free(void* t) { delete static_cast<Transcript*>(t); }
void zko_tr_absorb_u32(void* t, uint32_t v) { static_cast<Transcript*>(t)->absorb(v); }
void zko_tr_absorb_many(void* t, const uint32_t* v, size_t n) { for (size_t i = 0; i < n; i++) static_cast<Transcript*>(t)->absorb(v[i]); }
void zko_tr_absorb_bytes(void* t, const uint8_t* p, size_t n) { static_cast<Transcript*>(t)->absorb_bytes(p, n); }
uint32_t zko_tr_squeeze(void* t) { return static_cast<Transcript*>(t)->squeeze().v; }
void zko_tr_squeeze_ef(void* t, uint32_t* o) { put(static_cast<Transcript*>(t)->squeeze_ef(), o); }

// ---- MLE
void zko_eq_evals(const uint32_t* r, size_t k, uint32_t* out) {
    VF e = eq_evals(vf(r, k)); for (size_t i = 0; i < e.size(); i++) out[i] = e[i].v;
}
void zko_eq_evals_ef(const uint32_t* r, size_t k, uint32_t* out) {
    VEF e = eq_evals_ef(vef(r, k)); for (size_t i = 0; i < e.size(); i++) put(e[i], out + 4 * i);
}
uint32_t zko_mle_evaluate(const uint32_t* ev, size_t n, const uint32_t* pt, size_t k) {
    return mle_evaluate(vf(ev, n), vf(pt, k)).v;
}
void zko_mle_evaluate_ef(const uint32_t* ev, size_t n, const uint32_t* pt, size_t k, uint32_t* o) {
    put(mle_evaluate_ef(vf(ev, n), vef(pt, k)), o);
}
void zko_mle_evaluate_efef(const uint32_t* ev, size_t n, const uint32_t* pt, size_t k, uint32_t* o) {
    put(mle_evaluate_efef(vef(ev, n), vef(pt, k)), o);
}

// ---- sumcheck provers.  polys: evals-per-round * (1 or 4) u32 per round; chal: 1 or 4 per round.
void zko_prove_product(void* t, const uint32_t* f, const uint32_t* g, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_product(vf(f, n), vf(g, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); fin[0] = r.f_at_s.v; fin[1] = r.g_at_s.v;
}
void zko_prove_triple(void* t, const uint32_t* f, const uint32_t* g, const uint32_t* h, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_triple(vf(f, n), vf(g, n), vf(h, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); fin[0] = r.f_at_s.v; fin[1] = r.g_at_s.v; fin[2] = r.h_at_s.v;
}
void zko_prove_product_ones(void* t, const uint32_t* g, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_product_ones(vf(g, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); fin[0] = r.f_at_s.v; fin[1] = r.g_at_s.v;
}
void zko_prove_product_ef(void* t, const uint32_t* f, const uint32_t* g, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_product_ef(vf(f, n), vf(g, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); put(r.f_at_s, fin); put(r.g_at_s, fin + 4);
}
void zko_prove_product_ef_full(void* t, const uint32_t* f, const uint32_t* g, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_product_ef_full(vef(f, n), vef(g, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); put(r.f_at_s, fin); put(r.g_at_s, fin + 4);
}
void zko_prove_product_ef_mixed(void* t, const uint32_t* f, const uint32_t* g, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_product_ef_mixed(vef(f, n), vf(g, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); put(r.f_at_s, fin); put(r.g_at_s, fin + 4);
}
void zko_prove_triple_ef_full(void* t, const uint32_t* f, const uint32_t* g, const uint32_t* h, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_triple_ef_full(vef(f, n), vef(g, n), vef(h, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); put(r.f_at_s, fin); put(r.g_at_s, fin + 4); put(r.h_at_s, fin + 8);
}
void zko_prove_product_ones_ef_full(void* t, const uint32_t* g, size_t nv, uint32_t* polys, uint32_t* chal, uint32_t* fin) {
    size_t n = size_t(1) << nv;
    auto r = prove_product_ones_ef_full(vef(g, n), nv, *static_cast<Transcript*>(t));
    flatten(r.proof, polys, chal); put(r.f_at_s, fin); put(r.g_at_s, fin + 4);
}

// ---- sumcheck verifiers.  `epr` = stored evals per round; challenges may be absent (nchal = 0).
static SumcheckProof unflat(const uint32_t* polys, size_t nv, size_t epr, const uint32_t* chal, size_t nchal) {
    SumcheckProof p;
    for (size_t i = 0; i < nv; i++) p.round_polys.emplace_back(polys + i * epr, polys + (i + 1) * epr);
    p.challenges.assign(chal, chal + nchal);
    return p;
}
static SumcheckProofEF unflat_ef(const uint32_t* polys, size_t nv, size_t epr, const uint32_t* chal, size_t nchal) {
    SumcheckProofEF p;
    for (size_t i = 0; i < nv; i++) {
        std::vector<EFElement> r(epr);
        for (size_t e = 0; e < epr; e++) memcpy(r[e].data(), polys + (i * epr + e) * 4, 16);
        p.round_polys.push_back(r);
    }
    for (size_t i = 0; i < nchal; i++) { EFElement e; memcpy(e.data(), chal + 4 * i, 16); p.challenges.push_back(e); }
    return p;
}
int zko_verify_product(void* t, uint32_t claimed, const uint32_t* polys, size_t nv, size_t epr, const uint32_t* chal, size_t nchal, const uint32_t* fin) {
    return verify_product_with_challenges(F(claimed), unflat(polys, nv, epr, chal, nchal), F(fin[0]), F(fin[1]), *static_cast<Transcript*>(t));
}
int zko_verify_triple(void* t, uint32_t claimed, const uint32_t* polys, size_t nv, size_t epr, const uint32_t* chal, size_t nchal, const uint32_t* fin) {
    return verify_triple_with_challenges(F(claimed), unflat(polys, nv, epr, chal, nchal), F(fin[0]), F(fin[1]), F(fin[2]), *static_cast<Transcript*>(t));
}
int zko_verify_product_ef(void* t, const uint32_t* claimed, const uint32_t* polys, size_t nv, size_t epr, const uint32_t* chal, size_t nchal, const uint32_t* fin) {
    return verify_product_ef_with_challenges(EF::from_u32x4(claimed), unflat_ef(polys, nv, epr, chal, nchal),
                                             EF::from_u32x4(fin), EF::from_u32x4(fin + 4), *static_cast<Transcript*>(t));
}
int zko_verify_triple_ef(void* t, const uint32_t* claimed, const uint32_t* polys, size_t nv, size_t epr, const uint32_t* chal, size_t nchal, const uint32_t* fin) {
    return verify_triple_ef_with_challenges(EF::from_u32x4(claimed), unflat_ef(polys, nv, epr, chal, nchal),
                                            EF::from_u32x4(fin), EF::from_u32x4(fin + 4), EF::from_u32x4(fin + 8), *static_cast<Transcript*>(t));
}

}  // extern "C"
