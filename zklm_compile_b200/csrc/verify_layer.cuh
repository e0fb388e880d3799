// Verifier of a Qwen-style layer proof (rust/zk_ml_prover/src/transformer/qwen.rs:932-1097) and of
// the sub-proofs it is made of: sumcheck.rs:1477-1553 (EF sumchecks with derived challenges),
// weight_commitment.rs:377-415, 521-532 (MLE-eval proofs), matmul.rs:1000-1117, rmsnorm.rs:670-862,
// elementwise.rs:483-523, 598-642, lookup.rs:912-976, sigmoid_gate.rs / swiglu.rs.
//
// The reference's verifier re-runs the forward pass and then replays the transcript.  Here the forward
// trace is the one the layer object holds after zkb_qwen_layer_forward; the host decodes the bincode
// bytes (it needs their structure to know what to enqueue), packs every value a kernel has to read into
// one word array, and enqueues, in the prover's order: transcript scripts (the same tr_script_kernel),
// one single-thread kernel per sumcheck that checks the rounds against the running claim and derives the
// challenges, and small kernels for the checks whose operands exist only on the device (eq at a derived
// point, MLE of a trace vector at a squeezed point, a recomputed commitment).  Checks between values of
// the proof itself are made on the host while decoding.  Every device check writes one word; the proof
// is accepted when all of them are 1 and no host check failed.  Nothing returns early on the device:
// after a failed check the remaining kernels still run (on a transcript that no longer matters).
#pragma once
#include "verify.cuh"
#include "qwen.cuh"

namespace zkb {

// ---- host: decoded proof ---------------------------------------------------------------------------
struct LvFe { u32 w[4]; };
// equality as field elements (proof words are reduced mod p when they are read)
inline bool lv_eq(const LvFe& a, const LvFe& b) { for (int i = 0; i < 4; i++) if (a.w[i] % ZKB_P != b.w[i] % ZKB_P) return false; return true; }
inline Fe lv_fe(const LvFe& a) { return Fe{a.w[0] % ZKB_P, a.w[1] % ZKB_P, a.w[2] % ZKB_P, a.w[3] % ZKB_P}; }

constexpr u32 LV_ROUND_STRIDE = 17;        // [count][4 EF values]
struct LvSumcheck { u32 off = 0, n_rounds = 0, chal_off = 0, n_chal = 0; LvFe first[2] = {}; bool uniform = true; u32 per_round = 0; };
struct LvEval { LvSumcheck sc; LvFe eq_at_s, w_at_s; u32 fin_off = 0; };
struct LvCommit { unsigned char root[32]; uint64_t num = 0, log_h = 0; u32 kind = 0; };
struct LvMatmul {
    LvSumcheck sc; LvFe w_at_rs, x_at_s; u32 fin_off = 0;
    u32 r_off = 0, n_r = 0, s_off = 0, n_s = 0;
    LvEval w_eval; LvFe w_claimed; LvCommit wc; bool bound = false, has_bf = false;
    BvParsed bf;
};
struct LvNorm {
    int32_t delta = 0; u32 sum_sq = 0;
    LvSumcheck var, h_sq, g_sq, g_prod, g_triple;
    LvFe var_fin[2], h_sq_fin[3], s_h, g_sq_fin[3], s_g, g_prod_fin[2], g_triple_fin[3], t_g;
    u32 var_fin_off = 0, h_sq_fin_off = 0, g_sq_fin_off = 0, g_prod_fin_off = 0, g_triple_fin_off = 0;
    LvCommit cx, cgamma, cg, ch;
    LvEval x_var, g_prod_ev, x_triple, gamma_triple, h_sq_ev, g_sq_ev;
    LvFe x_at_var_s, g_at_prod_s, x_at_triple_s, gamma_at_triple_s, h_at_sq_s, g_at_gsq_s;
};
struct LvHadamard { LvSumcheck sc; LvFe fin[3], c_eval; u32 fin_off = 0; LvEval c_ev; LvCommit cc; };
struct LvAdd { LvSumcheck a, b; LvFe a_fin[2], b_fin[2], c_eval; u32 a_fin_off = 0, b_fin_off = 0; LvEval c_ev; LvCommit cc; };
struct LvLookup { LvCommit ct, cm; LvSumcheck sc; LvFe h_at_s; u32 fin_off = 0; bool digest_zero = true; unsigned char digest[32]; };
struct LvGate { LvLookup lk; LvHadamard had; };
struct LvLayer {
    LvNorm norm1, norm2;
    LvMatmul mq, mk, mv, mo, mg, mgate, mup, mdown;
    uint64_t attn_heads = 0, attn_seq = 0, attn_d_head = 0; u32 attn_a = 0, attn_v = 0; bool attn_gqa = false;
    LvGate sig, swiglu;
    LvAdd res1, res2;
    LvCommit commits[8];
};

struct LvParser {
    const uint8_t* p; size_t n, at = 0; bool ok = true;
    std::vector<u32> pw;               // words the device reads (EF constants, round polynomials, challenges)
    LvParser(const uint8_t* b, size_t len) : p(b), n(len) { pw.assign(4, 0u); }       // offset 0 = "absent"
    uint8_t u8() { if (at + 1 > n) { ok = false; return 0; } return p[at++]; }
    u32 u32v() { if (at + 4 > n) { ok = false; return 0; } u32 v = 0; for (int i = 0; i < 4; i++) v |= (u32)p[at + i] << (8 * i); at += 4; return v; }
    uint64_t u64v() { if (at + 8 > n) { ok = false; return 0; } uint64_t v = 0; for (int i = 0; i < 8; i++) v |= (uint64_t)p[at + i] << (8 * i); at += 8; return v; }
    LvFe fe() { LvFe e; for (int i = 0; i < 4; i++) e.w[i] = u32v(); return e; }
    u32 put(const LvFe& e) { u32 off = (u32)pw.size(); for (int i = 0; i < 4; i++) pw.push_back(e.w[i] % ZKB_P); return off; }
    LvFe fe_put(u32* off) { LvFe e = fe(); *off = put(e); return e; }
    void sumcheck(LvSumcheck& s) {
        const uint64_t nr = u64v();
        if (!ok || nr > 64) { ok = false; return; }
        s.n_rounds = (u32)nr;
        while (pw.size() % 4) pw.push_back(0);
        s.off = (u32)pw.size();
        for (uint64_t r = 0; r < nr && ok; r++) {
            const uint64_t cnt = u64v();
            if (!ok || cnt > 4) { ok = false; return; }              // more than four evaluations: no verifier accepts that
            if (r == 0) s.per_round = (u32)cnt; else if (cnt != s.per_round) s.uniform = false;
            pw.push_back((u32)cnt);
            for (uint64_t i = 0; i < 4; i++) {
                LvFe e{};
                if (i < cnt) e = fe();
                if (r == 0 && i < 2) s.first[i] = e;
                for (int k = 0; k < 4; k++) pw.push_back(e.w[k] % ZKB_P);
            }
        }
        const uint64_t nc = u64v();
        if (!ok || nc > 64) { ok = false; return; }
        s.n_chal = (u32)nc;
        s.chal_off = (u32)pw.size();
        for (uint64_t i = 0; i < nc; i++) put(fe());
    }
    void commit(LvCommit& c) {
        for (int i = 0; i < 32; i++) c.root[i] = u8();
        c.num = u64v(); c.log_h = u64v(); c.kind = u32v();
    }
    void eval(LvEval& e) { sumcheck(e.sc); e.eq_at_s = fe_put(&e.fin_off); u32 t; e.w_at_s = fe_put(&t); }
    void matmul(LvMatmul& m) {
        sumcheck(m.sc);
        m.w_at_rs = fe_put(&m.fin_off); u32 t; m.x_at_s = fe_put(&t);
        uint64_t nr = u64v(); if (!ok || nr > 64) { ok = false; return; }
        m.n_r = (u32)nr; m.r_off = (u32)pw.size(); for (uint64_t i = 0; i < nr; i++) put(fe());
        uint64_t ns = u64v(); if (!ok || ns > 64) { ok = false; return; }
        m.n_s = (u32)ns; m.s_off = (u32)pw.size(); for (uint64_t i = 0; i < ns; i++) put(fe());
        eval(m.w_eval);
        m.w_claimed = fe();
        commit(m.wc);
        m.bound = u8() != 0;
        const uint8_t tag = u8();
        if (tag > 1) { ok = false; return; }
        m.has_bf = tag == 1;
        if (m.has_bf && ok) {
            // the opening proof follows; decode it as commitment || proof with the matmul's own commitment in front
            std::vector<uint8_t> tmp(m.wc.root, m.wc.root + 16);
            for (int i = 0; i < 8; i++) tmp.push_back((uint8_t)(m.wc.num >> (8 * i)));
            for (int i = 0; i < 8; i++) tmp.push_back((uint8_t)(m.wc.log_h >> (8 * i)));
            tmp.insert(tmp.end(), p + at, p + n);
            size_t used = 0;
            if (!bv_parse(tmp.data(), tmp.size(), m.bf, &used) || used < 32) { ok = false; return; }
            at += used - 32;
        }
    }
    void norm(LvNorm& q) {
        q.delta = (int32_t)u32v();
        sumcheck(q.var); q.var_fin[0] = fe_put(&q.var_fin_off); u32 t; q.var_fin[1] = fe_put(&t); q.sum_sq = u32v();
        sumcheck(q.h_sq); q.h_sq_fin[0] = fe_put(&q.h_sq_fin_off); q.h_sq_fin[1] = fe_put(&t); q.h_sq_fin[2] = fe_put(&t); q.s_h = fe();
        sumcheck(q.g_sq); q.g_sq_fin[0] = fe_put(&q.g_sq_fin_off); q.g_sq_fin[1] = fe_put(&t); q.g_sq_fin[2] = fe_put(&t); q.s_g = fe();
        sumcheck(q.g_prod); q.g_prod_fin[0] = fe_put(&q.g_prod_fin_off); q.g_prod_fin[1] = fe_put(&t);
        sumcheck(q.g_triple); q.g_triple_fin[0] = fe_put(&q.g_triple_fin_off); q.g_triple_fin[1] = fe_put(&t); q.g_triple_fin[2] = fe_put(&t);
        q.t_g = fe();
        commit(q.cx); commit(q.cgamma); commit(q.cg); commit(q.ch);
        eval(q.x_var); q.x_at_var_s = fe();
        eval(q.g_prod_ev); q.g_at_prod_s = fe();
        eval(q.x_triple); q.x_at_triple_s = fe();
        eval(q.gamma_triple); q.gamma_at_triple_s = fe();
        eval(q.h_sq_ev); q.h_at_sq_s = fe();
        eval(q.g_sq_ev); q.g_at_gsq_s = fe();
    }
    void hadamard(LvHadamard& h) {
        sumcheck(h.sc); h.fin[0] = fe_put(&h.fin_off); u32 t; h.fin[1] = fe_put(&t); h.fin[2] = fe_put(&t); h.c_eval = fe();
        eval(h.c_ev); commit(h.cc);
    }
    void add(LvAdd& a) {
        u32 t;
        sumcheck(a.a); a.a_fin[0] = fe_put(&a.a_fin_off); a.a_fin[1] = fe_put(&t);
        sumcheck(a.b); a.b_fin[0] = fe_put(&a.b_fin_off); a.b_fin[1] = fe_put(&t);
        a.c_eval = fe(); eval(a.c_ev); commit(a.cc);
    }
    void lookup(LvLookup& l) {
        commit(l.ct); commit(l.cm); sumcheck(l.sc);
        const LvFe one{{1, 0, 0, 0}};
        l.fin_off = put(one);                       // f = 1 (lookup.rs:975)
        l.h_at_s = fe(); put(l.h_at_s);
        for (int k = 0; k < 2; k++) { const uint8_t tag = u8(); if (tag == 1) fe(); else if (tag != 0) ok = false; }   // alpha, beta: Option<EFElement>
        for (int k = 0; k < 3; k++) {               // inputs, outputs, multiplicities: not read by verify_lookup_ef_with_data
            const uint64_t cnt = u64v();
            if (!ok || cnt > (1u << 24) || at + 4 * cnt > n) { ok = false; return; }
            at += 4 * cnt;
        }
        for (int i = 0; i < 32; i++) { l.digest[i] = u8(); if (l.digest[i]) l.digest_zero = false; }
    }
    void gate(LvGate& g) { lookup(g.lk); hadamard(g.had); }
    bool layer(LvLayer& L) {
        norm(L.norm1); matmul(L.mq); matmul(L.mk); matmul(L.mv);
        const uint64_t rows = u64v();
        if (!ok || rows != 0) { ok = false; return false; }          // row proofs exist only for seq_len > 1
        L.attn_heads = u64v(); L.attn_seq = u64v(); L.attn_d_head = u64v();
        const uint8_t some = u8();
        if (some != 1) { ok = false; return false; }
        L.attn_a = u32v(); L.attn_v = u32v(); L.attn_gqa = u8() != 0;
        matmul(L.mo); matmul(L.mg); gate(L.sig); add(L.res1); norm(L.norm2); matmul(L.mgate); matmul(L.mup); gate(L.swiglu); matmul(L.mdown); add(L.res2);
        for (int i = 0; i < 8; i++) commit(L.commits[i]);
        return ok && at == n;
    }
};

// ---- device ------------------------------------------------------------------------------------------
struct LvScArgs {
    u32 sc_off, n_rounds, degree;          // degree 2: product (rounds of 2 = [s0, s2] or 3 values); 3: triple (3 = [s0, s2, s3] or 4)
    u32 claim_off;                         // claim: pw[claim_off] when claim_slot is null
    const Fe* claim_slot;
    u32 fin_off, n_fin;                    // the final evaluations whose product the last claim must equal
    u32 chal_off, n_chal;                  // challenges stored in the proof (compared when present)
    Fe* chal_out;                          // derived challenges, n_rounds of them
    u32 post_squeezes;                     // derive_query_indices behind an MLE-eval proof: 24 squeezes, discarded
};
__device__ __forceinline__ Fe lv_ld(const u32* w) { return Fe{w[0], w[1], w[2], w[3]}; }
// sumcheck.rs:1477-1553
__global__ void lv_sumcheck_kernel(TrState* st, const u32* __restrict__ pw, LvScArgs a, u32* ok_out) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    if (threadIdx.x) return;
    Tr tr;
    tr_load(tr, st, trbuf);
    bool ok = true;
    Fe claim = a.claim_slot ? *a.claim_slot : lv_ld(pw + a.claim_off);
    const Fp half{(ZKB_P + 1) / 2}, sixth{inv31(6)};
    for (u32 i = 0; i < a.n_rounds; i++) {
        const u32* rp = pw + a.sc_off + i * LV_ROUND_STRIDE;
        const u32 cnt = rp[0];
        const Fe v0 = lv_ld(rp + 1), v1 = lv_ld(rp + 5), v2 = lv_ld(rp + 9), v3 = lv_ld(rp + 13);
        Fe s0 = v0, s1, s2, s3 = fe_zero();
        if (a.degree == 2) {
            if (cnt == 2) { s1 = claim - s0; s2 = v1; }
            else if (cnt >= 3) { s1 = v1; s2 = v2; }
            else { ok = false; s1 = claim - s0; s2 = fe_zero(); }
        } else {
            if (cnt == 3) { s1 = claim - s0; s2 = v1; s3 = v2; }
            else if (cnt == 4) { s1 = v1; s2 = v2; s3 = v3; }
            else { ok = false; s1 = claim - s0; s2 = fe_zero(); }
        }
        if (!fe_eq(s0 + s1, claim)) ok = false;
        tr_absorb_fe(tr, s0); tr_absorb_fe(tr, s1); tr_absorb_fe(tr, s2);
        if (a.degree == 3) tr_absorb_fe(tr, s3);
        const Fe r = tr_squeeze_fe(tr);
        if (a.n_chal) {
            if (i >= a.n_chal || !fe_eq(r, lv_ld(pw + a.chal_off + 4 * i))) ok = false;
        }
        if (a.chal_out) a.chal_out[i] = r;
        if (a.degree == 2) {
            // Lagrange basis on 0, 1, 2
            const Fe one = fe_one(), two = Fe{2, 0, 0, 0};
            const Fe l0 = (r - one) * (r - two) * half, l1 = fe_zero() - r * (r - two), l2 = r * (r - one) * half;
            claim = s0 * l0 + s1 * l1 + s2 * l2;
        } else {
            // Lagrange basis on 0, 1, 2, 3: denominators -6, 2, -2, 6
            const Fe x0 = r, x1 = r - fe_one(), x2 = r - Fe{2, 0, 0, 0}, x3 = r - Fe{3, 0, 0, 0};
            const Fe l0 = fe_zero() - x1 * x2 * x3 * sixth, l1 = x0 * x2 * x3 * half, l2 = fe_zero() - x0 * x1 * x3 * half, l3 = x0 * x1 * x2 * sixth;
            claim = s0 * l0 + s1 * l1 + s2 * l2 + s3 * l3;
        }
    }
    Fe prod = lv_ld(pw + a.fin_off);
    for (u32 k = 1; k < a.n_fin; k++) prod = prod * lv_ld(pw + a.fin_off + 4 * k);
    if (!fe_eq(claim, prod)) ok = false;
    for (u32 q = 0; q < a.post_squeezes; q++) (void)tr_squeeze(tr);
    tr_store(tr, st);
    *ok_out = ok ? 1u : 0u;
}
// compute_eq_at_point_ef(a, b) == expected
__global__ void lv_eq_check_kernel(const Fe* a, const Fe* b, u32 k, const u32* __restrict__ pw, u32 expect_off, u32* ok_out) {
    if (threadIdx.x) return;
    Fe r = fe_one();
    for (u32 i = 0; i < k; i++) r = r * (a[i] * b[i] + (fe_one() - a[i]) * (fe_one() - b[i]));
    *ok_out = fe_eq(r, lv_ld(pw + expect_off)) ? 1u : 0u;
}
// MLE of a base-field vector (len valid entries, zero beyond) at an EF point of k coordinates -> *out
__global__ void __launch_bounds__(1024) lv_mle_eval_kernel(const u32* __restrict__ v, u32 len, const Fe* point, u32 k, Fe* out) {
    __shared__ Fe pt[32];
    __shared__ u32 red[32 * 4];
    if (threadIdx.x < k) pt[threadIdx.x] = point[threadIdx.x];
    __syncthreads();
    Fe acc = fe_zero();
    for (u32 i = threadIdx.x; i < len; i += blockDim.x) acc = acc + eq_at_index<Fe>(pt, k, i) * Fp{v[i]};
    u32 w[4] = {acc.x, acc.y, acc.z, acc.w};
    block_sum_words<4>(w, red);
    if (threadIdx.x == 0) *out = Fe{w[0], w[1], w[2], w[3]};
}
__global__ void lv_cmp_words_kernel(const u32* __restrict__ a, const u32* __restrict__ pw, u32 off, u32 n, u32* ok_out) {
    if (threadIdx.x) return;
    bool ok = true;
    for (u32 i = 0; i < n; i++) ok = ok && a[i] == pw[off + i];
    *ok_out = ok ? 1u : 0u;
}
__global__ void lv_cmp_vec_kernel(const u32* __restrict__ a, const u32* __restrict__ b, u32 n, u32* ok_out) {
    __shared__ u32 bad;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    for (u32 i = threadIdx.x; i < n; i += blockDim.x) if (a[i] != b[i]) bad = 1;
    __syncthreads();
    if (threadIdx.x == 0) *ok_out = bad ? 0u : 1u;
}

__global__ void lv_all_ones_kernel(const u32* __restrict__ a, u32 n, u32* ok_out) {
    __shared__ u32 bad;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    for (u32 i = threadIdx.x; i < n; i += blockDim.x) if (a[i] != 1u) bad = 1;
    __syncthreads();
    if (threadIdx.x == 0) *ok_out = bad ? 0u : 1u;
}

// ---- host: the verifier's order of operations ----------------------------------------------------------
struct LvRun {
    zkb_ctx* c; TrState* tr; const u32* pw; LvParser* ps;
    Fe* slots; u32 slot_used = 0, slot_cap = 0;
    u32* ok; u32 ok_used = 0, ok_cap = 0;
    bool host_ok = true;
    int node_hash = 0;
    Fe* slot(u32 n) { if (slot_used + n > slot_cap) throw ArgFail{ZKB_E_TOO_LARGE, "verifier: out of challenge slots"}; Fe* p = slots + slot_used; slot_used += n; return p; }
    u32* flag() { if (ok_used >= ok_cap) throw ArgFail{ZKB_E_TOO_LARGE, "verifier: out of check slots"}; return ok + ok_used++; }
    void require(bool cond) { host_ok = host_ok && cond; }
};
inline u32 lv_put_words(LvParser& ps, const void* bytes, size_t n_words) {
    u32 off = (u32)ps.pw.size();
    const unsigned char* b = (const unsigned char*)bytes;
    for (size_t i = 0; i < n_words; i++) ps.pw.push_back((u32)b[4 * i] | ((u32)b[4 * i + 1] << 8) | ((u32)b[4 * i + 2] << 16) | ((u32)b[4 * i + 3] << 24));
    return off;
}
// Everything below only enqueues; offsets into pw were fixed while decoding (lv_prepare_* runs before the upload).
inline Fe* lv_sumcheck(LvRun& R, const LvSumcheck& s, u32 degree, u32 claim_off, const Fe* claim_slot, u32 fin_off, u32 n_fin, u32 post_squeezes = 0) {
    R.require(s.n_rounds <= 40);
    Fe* out = R.slot(s.n_rounds ? s.n_rounds : 1);
    LvScArgs a{s.off, s.n_rounds, degree, claim_off, claim_slot, fin_off, n_fin, s.chal_off, s.n_chal, out, post_squeezes};
    lv_sumcheck_kernel<<<1, 32, exclusive_smem(lv_sumcheck_kernel, R.c), R.c->stream>>>(R.tr, R.pw, a, R.flag());
    ZKB_LAUNCHED(R.c);
    return out;
}
inline void lv_eq_check(LvRun& R, const Fe* a, const Fe* b, u32 k, u32 expect_off) {
    lv_eq_check_kernel<<<1, 32, 0, R.c->stream>>>(a, b, k, R.pw, expect_off, R.flag());
    ZKB_LAUNCHED(R.c);
}
// verify_mle_eval_ef (weight_commitment.rs:377-415): `k` = point length; the sumcheck has its own number of rounds
inline void lv_eval(LvRun& R, const LvEval& e, u32 claim_off, const Fe* point, u32 k) {
    Fe* s = lv_sumcheck(R, e.sc, 2, claim_off, nullptr, e.fin_off, 2, BF_QUERIES);
    lv_eq_check(R, point, s, k < e.sc.n_rounds ? k : e.sc.n_rounds, e.fin_off);
}
inline void lv_eval_bound(LvRun& R, const LvEval& e, const LvCommit& c, u32 claim_off, const Fe* point, u32 k, const char* label) {
    ScriptBuilder sb;
    sb.str(label);
    sb.bytes(c.root, 32);
    sb.run(R.c, R.tr);
    lv_eval(R, e, claim_off, point, k);
}
inline Fe* lv_squeeze_point(LvRun& R, u32 k) {
    Fe* p = R.slot(k ? k : 1);
    ScriptBuilder sb;
    sb.squeeze(reinterpret_cast<u32*>(p), 4 * k);
    sb.run(R.c, R.tr);
    return p;
}

struct LvNormOff { u32 sum_sq, t_g, s_h, s_g, x_at_var_s, g_at_prod_s, x_at_triple_s, gamma_at_triple_s, h_at_sq_s, g_at_gsq_s, h_root; };
inline LvNormOff lv_prepare_norm(LvParser& ps, const LvNorm& p) {
    LvNormOff o{};
    const LvFe ss{{p.sum_sq % ZKB_P, 0, 0, 0}};
    o.sum_sq = ps.put(ss); o.t_g = ps.put(p.t_g); o.s_h = ps.put(p.s_h); o.s_g = ps.put(p.s_g);
    o.x_at_var_s = ps.put(p.x_at_var_s); o.g_at_prod_s = ps.put(p.g_at_prod_s); o.x_at_triple_s = ps.put(p.x_at_triple_s);
    o.gamma_at_triple_s = ps.put(p.gamma_at_triple_s); o.h_at_sq_s = ps.put(p.h_at_sq_s); o.g_at_gsq_s = ps.put(p.g_at_gsq_s);
    o.h_root = lv_put_words(ps, p.ch.root, 8);
    return o;
}
// rmsnorm.rs:670-862; y: the norm's output on the device, zero-padded to 2^k
inline void lv_norm(LvRun& R, const LvNorm& p, const LvNormOff& o, const u32* y, u32 d) {
    const u32 k = log2_ceil_u(d), n_pad = 1u << k;
    {
        ScriptBuilder sb;
        sb.str("rmsnorm-pert-v1");
        sb.word((u32)p.delta);
        sb.bytes(p.cx.root, 32); sb.bytes(p.cgamma.root, 32); sb.bytes(p.cg.root, 32); sb.bytes(p.ch.root, 32);
        sb.word(p.sum_sq);
        sb.run(R.c, R.tr);
    }
    Fe* s_var = lv_sumcheck(R, p.var, 2, o.sum_sq, nullptr, p.var_fin_off, 2);
    R.require(lv_eq(p.var_fin[0], p.var_fin[1]) && lv_eq(p.x_at_var_s, p.var_fin[0]));
    lv_eval_bound(R, p.x_var, p.cx, p.var_fin_off, s_var, p.var.n_rounds, "rmsnorm-x-var");
    Fe* gc = lv_squeeze_point(R, k);
    Fe* s_gp = lv_sumcheck(R, p.g_prod, 2, o.t_g, nullptr, p.g_prod_fin_off, 2);
    lv_eq_check(R, gc, s_gp, k < p.g_prod.n_rounds ? k : p.g_prod.n_rounds, p.g_prod_fin_off);
    R.require(lv_eq(p.g_at_prod_s, p.g_prod_fin[1]));
    lv_eval_bound(R, p.g_prod_ev, p.cg, o.g_at_prod_s, s_gp, p.g_prod.n_rounds, "rmsnorm-g-prod");
    Fe* s_gt = lv_sumcheck(R, p.g_triple, 3, o.t_g, nullptr, p.g_triple_fin_off, 3);
    lv_eq_check(R, gc, s_gt, k < p.g_triple.n_rounds ? k : p.g_triple.n_rounds, p.g_triple_fin_off);
    R.require(lv_eq(p.x_at_triple_s, p.g_triple_fin[2]));
    lv_eval_bound(R, p.x_triple, p.cx, o.x_at_triple_s, s_gt, p.g_triple.n_rounds, "rmsnorm-x-triple");
    R.require(lv_eq(p.gamma_at_triple_s, p.g_triple_fin[1]));
    lv_eval_bound(R, p.gamma_triple, p.cgamma, o.gamma_at_triple_s, s_gt, p.g_triple.n_rounds, "rmsnorm-gamma-triple");
    Fe* sq = lv_squeeze_point(R, k);
    Fe* s_hs = lv_sumcheck(R, p.h_sq, 3, o.s_h, nullptr, p.h_sq_fin_off, 3);
    lv_eq_check(R, sq, s_hs, k < p.h_sq.n_rounds ? k : p.h_sq.n_rounds, p.h_sq_fin_off);
    R.require(lv_eq(p.h_sq_fin[1], p.h_sq_fin[2]) && lv_eq(p.h_at_sq_s, p.h_sq_fin[1]));
    lv_eval_bound(R, p.h_sq_ev, p.ch, o.h_at_sq_s, s_hs, p.h_sq.n_rounds, "rmsnorm-h-sq");
    {   // commit_weights_fast(padded(y)) == h_commitment
        u32* root = (u32*)R.c->scratch(32);
        u32* cvs = (u32*)R.c->scratch((((size_t)n_pad * 4 + 7 + 1023) / 1024 + 1) * 32);
        b3_commit_kernel<<<1, R.c->single_cta_threads(), 0, R.c->stream>>>(b3_prefix("weights", 7), y, n_pad, nullptr, cvs, root, nullptr);
        ZKB_LAUNCHED(R.c);
        lv_cmp_words_kernel<<<1, 32, 0, R.c->stream>>>(root, R.pw, o.h_root, 8, R.flag());
        ZKB_LAUNCHED(R.c);
    }
    Fe* s_gs = lv_sumcheck(R, p.g_sq, 3, o.s_g, nullptr, p.g_sq_fin_off, 3);
    lv_eq_check(R, sq, s_gs, k < p.g_sq.n_rounds ? k : p.g_sq.n_rounds, p.g_sq_fin_off);
    R.require(lv_eq(p.g_sq_fin[1], p.g_sq_fin[2]) && lv_eq(p.g_at_gsq_s, p.g_sq_fin[1]));
    lv_eval_bound(R, p.g_sq_ev, p.cg, o.g_at_gsq_s, s_gs, p.g_sq.n_rounds, "rmsnorm-g-sq");
    // sum_sq * s_h == d * s_g
    const Fe lhs = Fe{p.sum_sq % ZKB_P, 0, 0, 0} * lv_fe(p.s_h), rhs = Fe{d % ZKB_P, 0, 0, 0} * lv_fe(p.s_g);
    R.require(fe_eq(lhs, rhs));
}

// matmul.rs:1000-1117; y: the matmul's output on the device, zero-padded to 2^log_m
inline void lv_matmul(LvRun& R, const LvMatmul& p, const u32* y, u32 m) {
    const u32 log_m = log2_ceil_u(m), m_pad = 1u << log_m;
    Fe* r = R.slot(log_m ? log_m : 1);
    {
        ScriptBuilder sb;
        sb.words_dev(y, m, m_pad);
        sb.squeeze(reinterpret_cast<u32*>(r), 4 * log_m);
        sb.run(R.c, R.tr);
    }
    if (p.n_r) {
        R.require(p.n_r == log_m);
        if (p.n_r == log_m) { lv_cmp_words_kernel<<<1, 32, 0, R.c->stream>>>(reinterpret_cast<const u32*>(r), R.pw, p.r_off, 4 * log_m, R.flag()); ZKB_LAUNCHED(R.c); }
    }
    Fe* claim = R.slot(1);
    lv_mle_eval_kernel<<<1, 1024, 0, R.c->stream>>>(y, m, r, log_m, claim);
    ZKB_LAUNCHED(R.c);
    Fe* derived = lv_sumcheck(R, p.sc, 2, 0, claim, p.fin_off, 2);
    const Fe* s = derived;
    u32 n_s = p.sc.n_rounds;
    if (p.n_s) {           // s_point kept in the proof: the eval proof below is checked at that point
        Fe* sp = R.slot(p.n_s);
        ZKB_CUDA(cudaMemcpyAsync(sp, R.pw + p.s_off, (size_t)p.n_s * 16, cudaMemcpyDeviceToDevice, R.c->stream));
        s = sp; n_s = p.n_s;
    }
    if (p.has_bf) {
        const u32 log_n = p.bf.log_n;
        u32* bf_point = (u32*)R.c->scratch((size_t)log_n * 4 + 16);
        ScriptBuilder sb;
        sb.squeeze(bf_point, log_n);
        sb.bytes(p.wc.root, 16);
        sb.run(R.c, R.tr);
        if (p.bf.trees.empty() || p.bf.too_large) R.require(false);
        else {
            // claimed = the proof's own final value (matmul.rs:1086): only the internal checks count
            BvRun run = basefold_verify_enqueue(R.c, R.tr, p.bf, bf_point, log_n, R.node_hash);
            u32* f = R.flag();
            lv_all_ones_kernel<<<1, 256, 0, R.c->stream>>>(run.result_dev, run.n_results, f);
            ZKB_LAUNCHED(R.c);
        }
    }
    {
        ScriptBuilder sb;
        sb.bytes(p.wc.root, 32);
        sb.run(R.c, R.tr);
    }
    lv_eval(R, p.w_eval, p.fin_off, s, n_s);
}

struct LvHadOff { u32 c_eval; };
// elementwise.rs:483-523
inline void lv_hadamard(LvRun& R, const LvHadamard& p, u32 c_eval_off, const Fe* point, u32 k) {
    { ScriptBuilder sb; sb.bytes(p.cc.root, 32); sb.run(R.c, R.tr); }
    Fe* s = lv_sumcheck(R, p.sc, 3, c_eval_off, nullptr, p.fin_off, 3);
    lv_eq_check(R, point, s, k < p.sc.n_rounds ? k : p.sc.n_rounds, p.fin_off);
    lv_eval_bound(R, p.c_ev, p.cc, c_eval_off, point, k, "hadamard-c-eval-ef");
}
struct LvAddOff { u32 a_eval, b_eval, c_eval; };
inline LvAddOff lv_prepare_add(LvParser& ps, const LvAdd& p) {
    LvAddOff o{};
    const Fe a = lv_fe(p.a.first[0]) + lv_fe(p.a.first[1]), b = lv_fe(p.b.first[0]) + lv_fe(p.b.first[1]);
    o.a_eval = ps.put(LvFe{{a.x, a.y, a.z, a.w}}); o.b_eval = ps.put(LvFe{{b.x, b.y, b.z, b.w}}); o.c_eval = ps.put(p.c_eval);
    return o;
}
// elementwise.rs:598-642
inline void lv_add(LvRun& R, const LvAdd& p, const LvAddOff& o, const Fe* point, u32 k) {
    { ScriptBuilder sb; sb.bytes(p.cc.root, 32); sb.run(R.c, R.tr); }
    R.require(p.a.n_rounds >= 1 && p.b.n_rounds >= 1 && p.a.per_round >= 2 && p.b.per_round >= 2);      // round_polys[0][0], [0][1] are read
    Fe* sa = lv_sumcheck(R, p.a, 2, o.a_eval, nullptr, p.a_fin_off, 2);
    lv_eq_check(R, point, sa, k < p.a.n_rounds ? k : p.a.n_rounds, p.a_fin_off);
    Fe* sb2 = lv_sumcheck(R, p.b, 2, o.b_eval, nullptr, p.b_fin_off, 2);
    lv_eq_check(R, point, sb2, k < p.b.n_rounds ? k : p.b.n_rounds, p.b_fin_off);
    const Fe a = lv_fe(p.a.first[0]) + lv_fe(p.a.first[1]), b = lv_fe(p.b.first[0]) + lv_fe(p.b.first[1]);
    R.require(fe_eq(a + b, lv_fe(p.c_eval)));
    lv_eval_bound(R, p.c_ev, p.cc, o.c_eval, point, k, "add-c-eval-ef");
}
struct LvGateOff { u32 zero, c_eval, digest; };
inline LvGateOff lv_prepare_gate(LvParser& ps, const LvGate& g) {
    LvGateOff o{};
    o.zero = ps.put(LvFe{{0, 0, 0, 0}});
    o.c_eval = ps.put(g.had.c_eval);
    o.digest = lv_put_words(ps, g.lk.digest, 8);
    return o;
}
// lookup.rs:912-976 + sigmoid_gate.rs / swiglu.rs; lk_in / lk_out: the requantised inputs and the table outputs on the device
inline void lv_gate(LvRun& R, const LvGate& g, const LvGateOff& o, u32 n, const u32* lk_in, const u32* lk_out) {
    const u32 k = log2_ceil_u(n);
    if (!g.lk.digest_zero) {        // compute_lookup_external_digest(inputs, outputs) == the proof's digest
        u32* cat = (u32*)R.c->scratch(((size_t)2 * n + 2) * 4 + 16);
        logup_digest_concat_kernel<<<grid_for(R.c, 2 * (size_t)n + 2), 256, 0, R.c->stream>>>(lk_in, lk_out, n, cat);
        ZKB_LAUNCHED(R.c);
        unsigned char pre[31];
        memcpy(pre, "lookup-external-data-v1", 23);
        for (int i = 0; i < 8; i++) pre[23 + i] = (unsigned char)((uint64_t)n >> (8 * i));
        u32* root = (u32*)R.c->scratch(32);
        commit_large(R.c, b3_prefix(pre, 31), cat, 2 * (size_t)n + 2, root);
        lv_cmp_words_kernel<<<1, 32, 0, R.c->stream>>>(root, R.pw, o.digest, 8, R.flag());
        ZKB_LAUNCHED(R.c);
    }
    {
        unsigned char zero[32] = {0};
        u32* sink = (u32*)R.c->scratch(32 + 16);
        ScriptBuilder sb;
        sb.bytes(zero, 32);
        sb.word(n);
        sb.pairs_dev(lk_in, lk_out, n);
        sb.squeeze(sink, 8);
        sb.bytes(g.lk.ct.root, 32);
        sb.bytes(g.lk.cm.root, 32);
        sb.run(R.c, R.tr);
    }
    lv_sumcheck(R, g.lk.sc, 2, o.zero, nullptr, g.lk.fin_off, 2);
    Fe* point = lv_squeeze_point(R, k);
    lv_hadamard(R, g.had, o.c_eval, point, k);
}

// verify_qwen_layer_ef_indexed (qwen.rs:932-1097) on the layer's current forward trace.  Returns the number of
// device check words at *ok_dev_out (each must be 1); *host_ok carries the checks made while decoding.
struct LvResult { u32* ok_dev = nullptr; u32 n_ok = 0; bool host_ok = true; };
inline LvResult qwen_verify_enqueue(zkb_qwen_layer* L, u32 layer_idx, const uint8_t input_hash[32], const uint8_t* bytes, size_t len,
                                    const u32* y_expected_host) {
    zkb_ctx* c = L->ctx;
    if (!L->have_trace) throw ArgFail{ZKB_E_ARG, "zkb_qwen_layer_verify: run the forward pass first"};
    LvParser ps(bytes, len);
    LvLayer P;
    if (!ps.layer(P)) throw ArgFail{ZKB_E_ARG, "the bytes do not decode as a QwenLayerProofEF at seq_len 1"};
    if (L->fwd_on_shared) {
        ZKB_CUDA(cudaStreamWaitEvent(c->stream, L->fwd_done, 0));
        L->fwd_on_shared = false;
    }
    const QwenDims& d = L->dm;
    const u32 dm = d.d_model, aod = d.aod(), log_d = log2_ceil_u(dm);
    // values the kernels read, appended to the packed words before they are uploaded
    const LvNormOff n1 = lv_prepare_norm(ps, P.norm1), n2 = lv_prepare_norm(ps, P.norm2);
    const LvGateOff g1 = lv_prepare_gate(ps, P.sig), g2 = lv_prepare_gate(ps, P.swiglu);
    const LvAddOff a1 = lv_prepare_add(ps, P.res1), a2 = lv_prepare_add(ps, P.res2);
    const u32 attn_off = (u32)ps.pw.size();
    ps.pw.push_back(P.attn_a); ps.pw.push_back(P.attn_v);
    {   // seed block -> device, as the prover does
        char seed[48];
        int n = snprintf(seed, sizeof seed, "qwen-layer-%u", layer_idx);
        unsigned char* b = reinterpret_cast<unsigned char*>(L->seed_host + 1);
        memset(L->seed_host, 0, 128);
        memcpy(b, seed, (size_t)n);
        memcpy(b + n, input_hash, 32);
        L->seed_host[0] = (u32)n + 32;
        ZKB_CUDA(cudaMemcpyAsync(L->seed_dev, L->seed_host, 128, cudaMemcpyHostToDevice, c->stream));
    }
    c->scratch_reset();
    LvRun R{};
    R.c = c; R.ps = &ps; R.node_hash = L->node_hash;
    R.tr = (TrState*)c->scratch(sizeof(TrState));
    u32* pw_dev = (u32*)c->scratch(ps.pw.size() * 4 + 16);
    R.pw = pw_dev;
    R.slot_cap = 4096; R.slots = (Fe*)c->scratch((size_t)R.slot_cap * 16);
    R.ok_cap = 1024; R.ok = (u32*)c->scratch((size_t)R.ok_cap * 4);
    ZKB_CUDA(cudaMemcpyAsync(pw_dev, ps.pw.data(), ps.pw.size() * 4, cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemsetAsync(R.ok, 0, (size_t)R.ok_cap * 4, c->stream));
    if (y_expected_host) {
        u32* ye = (u32*)c->scratch((size_t)dm * 4 + 16);
        ZKB_CUDA(cudaMemcpyAsync(ye, y_expected_host, (size_t)dm * 4, cudaMemcpyHostToDevice, c->stream));
        lv_cmp_vec_kernel<<<1, 256, 0, c->stream>>>(L->out, ye, dm, R.flag());
        ZKB_LAUNCHED(c);
    }
    tr_init_kernel<<<1, 1, 0, c->stream>>>(R.tr);
    ZKB_LAUNCHED(c);
    {
        ScriptBuilder sb;
        sb.bytes_dev_n(L->seed_dev);
        sb.str("qwen-dims-v1");
        u32 dims[12] = {d.d_model, d.d_ff, d.nq, d.nkv, d.d_head, d.v_heads, d.v_d_head, d.v_dim(), d.q_dim(), d.k_dim(), aod, d.is_gqa() ? 1u : 0u};
        sb.bytes(dims, sizeof dims);
        sb.run(c, R.tr);
        for (int i = 0; i < 8; i++) sb.bytes(P.commits[i].root, 32);
        sb.run(c, R.tr);
    }
    lv_norm(R, P.norm1, n1, L->norm1_out, dm);
    lv_matmul(R, P.mq, L->q, d.q_dim());
    lv_matmul(R, P.mk, L->k, d.k_dim());
    lv_matmul(R, P.mv, L->v, d.v_dim());
    {   // seq_len 1 attention: both evaluations recomputed from the trace and compared with the proof's
        u32* out2 = (u32*)c->scratch(16);
        seq1_consistency_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(R.tr, L->attn_out, aod, log2_ceil_u(aod), L->v, d.v_dim(), log2_ceil_u(d.v_dim()),
                                                                              d.is_gqa() ? 1u : 0u, log2_ceil_u(d.nkv), log2_ceil_u(d.d_head), out2);
        ZKB_LAUNCHED(c);
        lv_cmp_words_kernel<<<1, 32, 0, c->stream>>>(out2, R.pw, attn_off, 2, R.flag());
        ZKB_LAUNCHED(c);
        if (!P.attn_gqa) R.require(P.attn_a == P.attn_v);
    }
    lv_matmul(R, P.mo, L->gated_out, dm);
    lv_matmul(R, P.mg, L->g_raw, aod);
    lv_gate(R, P.sig, g1, aod, L->g_q, L->g_sig);
    { Fe* pt = lv_squeeze_point(R, log_d); lv_add(R, P.res1, a1, pt, log_d); }
    lv_norm(R, P.norm2, n2, L->norm2_out, dm);
    lv_matmul(R, P.mgate, L->gate_raw, d.d_ff);
    lv_matmul(R, P.mup, L->up, d.d_ff);
    lv_gate(R, P.swiglu, g2, d.d_ff, L->gate_q, L->gate_silu);
    lv_matmul(R, P.mdown, L->down, dm);
    { Fe* pt = lv_squeeze_point(R, log_d); lv_add(R, P.res2, a2, pt, log_d); }
    ZKB_CUDA(cudaGetLastError());
    LvResult out;
    out.ok_dev = R.ok; out.n_ok = R.ok_used; out.host_ok = R.host_ok;
    return out;
}

}  // namespace zkb
