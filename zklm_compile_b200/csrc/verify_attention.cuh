// Verifier of row-decomposed attention proofs (rust/zk_ml_prover/src/proving/attention.rs:279-385, :503-590 for GQA) with
// verify_matmul (matmul.rs:183-263), verify_softmax (softmax.rs:139-238), base verify_lookup (lookup.rs:803-874) and the plain
// verify_product / verify_triple (sumcheck.rs:981-1119) it calls.
//
// The host decodes bincode(RowAttentionProof) into one fixed-layout record per (head, row) - a proof whose vectors do not have
// the lengths the prover produces is rejected there - and one CTA per row replays the row's transcript on thread 0 while the
// other threads evaluate what the verifier recomputes itself: the multilinear evaluations of scores / e / output at the squeezed
// points, K(r, s) and V^T(r, s) from the K and V the caller supplies, the eq evaluation, the lookup's external-data digest.
// Like the reference's verifier it does not compare the lookup's inputs with the row's scores, nor attn_weights / y_values with
// anything; it checks what the reference checks.
#pragma once
#include "attention.cuh"

namespace zkb {

struct AvLayout {
    u32 S, D, log_s, log_d, s_pad, d_pad, nv_max;
    u32 o_hdr;                                                    // num_weights (low word), lookup rounds
    u32 o_sc1_polys, o_sc1_fin, o_r1, o_s1;
    u32 o_root_t, o_root_m, o_lk_polys, o_lk_fin, o_alpha_beta, o_lk_in, o_lk_out, o_digest;
    u32 o_sum, o_sc2_polys, o_sc2_fin;
    u32 o_sc3_polys, o_sc3_chal, o_sc3_fin, o_inv_s, o_e;
    u32 o_sc4_polys, o_sc4_fin, o_r4, o_s4;
    u32 words;
};
inline AvLayout av_layout(u32 S, u32 D) {
    AvLayout L{};
    L.S = S; L.D = D;
    L.log_s = att_log2_ceil(S); L.log_d = att_log2_ceil(D);
    L.s_pad = 1u << L.log_s; L.d_pad = 1u << L.log_d;
    L.nv_max = att_log2_ceil(2 * S);
    u32 o = 0;
    auto take = [&](u32 n) { u32 at = o; o += n; return at; };
    L.o_hdr = take(2);
    L.o_sc1_polys = take(3 * L.log_d); L.o_sc1_fin = take(2); L.o_r1 = take(L.log_s); L.o_s1 = take(L.log_d);
    L.o_root_t = take(8); L.o_root_m = take(8); L.o_lk_polys = take(2 * L.nv_max); L.o_lk_fin = take(2); L.o_alpha_beta = take(2);
    L.o_lk_in = take(S); L.o_lk_out = take(S); L.o_digest = take(8);
    L.o_sum = take(1); L.o_sc2_polys = take(3 * L.log_s); L.o_sc2_fin = take(2);
    L.o_sc3_polys = take(4 * L.log_s); L.o_sc3_chal = take(L.log_s); L.o_sc3_fin = take(3); L.o_inv_s = take(1); L.o_e = take(S);
    L.o_sc4_polys = take(3 * L.log_s); L.o_sc4_fin = take(2); L.o_r4 = take(L.log_d); L.o_s4 = take(L.log_s);
    L.words = (o + 3) & ~3u;
    return L;
}
inline size_t av_smem_bytes(const AvLayout& L) {
    const u32 m_pad = L.s_pad > L.d_pad ? L.s_pad : L.d_pad;
    const u32 cat = (2 * L.S + 2 > L.D ? 2 * L.S + 2 : L.D) + 16;
    const u32 part = L.d_pad > (u32)ATT_THREADS ? L.d_pad : (u32)ATT_THREADS;
    return ((size_t)2 * m_pad + cat + part + 128 + 64) * 4 + TR_SCRATCH_BYTES + 16;
}

// ---- host: bincode(RowAttentionProof) -> records ----------------------------------------------------------------
struct AvParsed {
    u32 num_heads = 0, S = 0, D = 0;
    AvLayout L{};
    std::vector<u32> rec, bind;           // per row: L.words; scores (S) | output (D)
    bool reject = false;                  // a length the prover does not produce: decided without looking at the values
};
struct AvReader {
    const uint8_t* p; size_t n, at = 0; bool ok = true;
    uint64_t u64v() { if (at + 8 > n) { ok = false; return 0; } uint64_t v; memcpy(&v, p + at, 8); at += 8; return v; }
    u32 u32v() { if (at + 4 > n) { ok = false; return 0; } u32 v; memcpy(&v, p + at, 4); at += 4; return v; }
    uint8_t u8v() { if (at + 1 > n) { ok = false; return 0; } return p[at++]; }
    // Vec<u32>: copied to dst when it has exactly `want` entries; any other length is skipped and reported
    bool vec(u32* dst, u32 want) {
        const uint64_t k = u64v();
        if (!ok || k > (n - at) / 4) { ok = false; return false; }
        if (k == want) { for (u32 i = 0; i < want; i++) dst[i] = u32v(); return true; }
        at += (size_t)k * 4;
        return false;
    }
    // SumcheckProof whose every round holds `per` values; the challenges (not read by verify_product / verify_triple) go to chal if asked
    bool sumcheck(u32* polys, u32 rounds, u32 per, u32* chal, u32 n_chal) {
        const uint64_t k = u64v();
        if (!ok || k > 64) { ok = false; return false; }
        bool good = k == rounds;
        for (uint64_t r = 0; r < k && ok; r++) {
            u32 tmp[4];
            const uint64_t cnt = u64v();
            if (!ok || cnt > (n - at) / 4) { ok = false; return false; }
            if (good && cnt == per) { for (u32 i = 0; i < per; i++) tmp[i] = u32v(); for (u32 i = 0; i < per; i++) polys[r * per + i] = tmp[i]; }
            else { at += (size_t)cnt * 4; good = false; }
        }
        const uint64_t c = u64v();
        if (!ok || c > (n - at) / 4) { ok = false; return false; }
        if (chal && c == n_chal) { for (u32 i = 0; i < n_chal; i++) chal[i] = u32v(); }
        else { at += (size_t)c * 4; if (chal) good = false; }
        return good;
    }
};
// `expect_*`: the dimensions the caller verifies against (q, k, v have those shapes).
inline bool av_parse(const uint8_t* bytes, size_t len, u32 expect_heads, u32 expect_S, u32 expect_D, AvParsed& out) {
    AvReader r{bytes, len};
    out.num_heads = expect_heads; out.S = expect_S; out.D = expect_D;
    const AvLayout L = av_layout(expect_S, expect_D);
    out.L = L;
    const uint64_t nh = r.u64v();
    if (!r.ok || nh > (1u << 22)) return false;
    bool good = nh == expect_heads;
    if (good) { out.rec.assign((size_t)expect_heads * expect_S * L.words, 0); out.bind.assign((size_t)expect_heads * expect_S * (expect_S + expect_D), 0); }
    std::vector<u32> scratch_rec(L.words), scratch_bind(expect_S + expect_D), tmp(expect_S > expect_D ? expect_S : expect_D);
    for (uint64_t h = 0; h < nh && r.ok; h++) {
        const uint64_t ns = r.u64v();
        if (!r.ok || ns > (1u << 22)) return false;
        if (ns != expect_S) good = false;
        for (uint64_t i = 0; i < ns && r.ok; i++) {
            const bool keep = good && h < expect_heads && i < expect_S;
            u32* rec = keep ? out.rec.data() + ((size_t)h * expect_S + i) * L.words : scratch_rec.data();
            u32* bind = keep ? out.bind.data() + ((size_t)h * expect_S + i) * (expect_S + expect_D) : scratch_bind.data();
            bool g = true;
            // score_proof: MatmulProof (matmul.rs:24-31)
            g &= r.sumcheck(rec + L.o_sc1_polys, L.log_d, 3, nullptr, 0);
            rec[L.o_sc1_fin] = r.u32v(); rec[L.o_sc1_fin + 1] = r.u32v();
            g &= r.vec(rec + L.o_r1, L.log_s);
            g &= r.vec(rec + L.o_s1, L.log_d);
            // softmax_proof: LookupProof first (lookup.rs:39-85)
            for (int w = 0; w < 8; w++) rec[L.o_root_t + w] = r.u32v();
            const uint64_t num_weights = r.u64v(); r.u64v(); r.u32v();
            for (int w = 0; w < 8; w++) rec[L.o_root_m + w] = r.u32v();
            r.u64v(); r.u64v(); r.u32v();
            // the number of rounds must be log2_ceil(num_lookups + table_commitment.num_weights) (lookup.rs:851-855)
            u32 nv = 0;
            if (num_weights <= 2 * (uint64_t)expect_S) nv = att_log2_ceil((u32)(expect_S + num_weights)); else g = false;
            rec[L.o_hdr] = (u32)num_weights; rec[L.o_hdr + 1] = nv;
            g &= r.sumcheck(rec + L.o_lk_polys, nv, 2, nullptr, 0);
            rec[L.o_lk_fin] = r.u32v(); rec[L.o_lk_fin + 1] = r.u32v();
            rec[L.o_alpha_beta] = r.u32v(); rec[L.o_alpha_beta + 1] = r.u32v();
            g &= r.vec(rec + L.o_lk_in, expect_S);
            g &= r.vec(rec + L.o_lk_out, expect_S);
            { const uint64_t m = r.u64v(); if (!r.ok || m > (r.n - r.at) / 4) return false; r.at += (size_t)m * 4; }     // multiplicities: not read
            for (int w = 0; w < 8; w++) rec[L.o_digest + w] = r.u32v();
            rec[L.o_sum] = r.u32v();
            g &= r.sumcheck(rec + L.o_sc2_polys, L.log_s, 3, nullptr, 0);
            rec[L.o_sc2_fin] = r.u32v(); rec[L.o_sc2_fin + 1] = r.u32v();
            g &= r.sumcheck(rec + L.o_sc3_polys, L.log_s, 4, rec + L.o_sc3_chal, L.log_s);
            for (int w = 0; w < 3; w++) rec[L.o_sc3_fin + w] = r.u32v();
            rec[L.o_inv_s] = r.u32v();
            g &= r.vec(rec + L.o_e, expect_S);
            g &= r.vec(tmp.data(), expect_S) || true;                                                                   // y_values: not read
            // output_proof
            g &= r.sumcheck(rec + L.o_sc4_polys, L.log_s, 3, nullptr, 0);
            rec[L.o_sc4_fin] = r.u32v(); rec[L.o_sc4_fin + 1] = r.u32v();
            g &= r.vec(rec + L.o_r4, L.log_d);
            g &= r.vec(rec + L.o_s4, L.log_s);
            g &= r.vec(bind, expect_S);
            r.vec(tmp.data(), expect_S);                                                                                 // attn_weights: not read
            g &= r.vec(bind + expect_S, expect_D);
            if (!g) good = false;
        }
    }
    const uint64_t ph = r.u64v(), ps = r.u64v(), pdh = r.u64v();
    if (ph != expect_heads || ps != expect_S || pdh != expect_D) good = false;
    const uint8_t opt = r.u8v();
    if (opt == 1) { r.u32v(); r.u32v(); r.u8v(); }                  // seq1_consistency: Some(..) is not read at seq_len >= 2
    else if (opt != 0) return false;
    out.reject = !good;
    return r.ok && r.at == len;
}

// ---- device -------------------------------------------------------------------------------------------------------
__device__ __forceinline__ u32 av_quadratic(u32 s0, u32 s1, u32 s2, u32 r) {               // sumcheck.rs:1122-1136
    const u32 inv2 = (ZKB_P + 1) / 2;
    const u32 r1 = sub31(r, 1), r2 = sub31(r, 2);
    const u32 l0 = mul31(mul31(r1, r2), inv2), l1 = neg31(mul31(r, r2)), l2 = mul31(mul31(r, r1), inv2);
    return add31(add31(mul31(s0, l0), mul31(s1, l1)), mul31(s2, l2));
}
__device__ __forceinline__ u32 av_cubic(const u32* s, u32 r) {                              // sumcheck.rs:1139-1157 on the points 0, 1, 2, 3
    const u32 inv6 = inv31(6), inv2 = (ZKB_P + 1) / 2;
    const u32 r0 = r, r1 = sub31(r, 1), r2 = sub31(r, 2), r3 = sub31(r, 3);
    const u32 l0 = neg31(mul31(mul31(mul31(r1, r2), r3), inv6));
    const u32 l1 = mul31(mul31(mul31(r0, r2), r3), inv2);
    const u32 l2 = neg31(mul31(mul31(mul31(r0, r1), r3), inv2));
    const u32 l3 = mul31(mul31(mul31(r0, r1), r2), inv6);
    return add31(add31(mul31(s[0], l0), mul31(s[1], l1)), add31(mul31(s[2], l2), mul31(s[3], l3)));
}
// verify_product / verify_triple on thread 0 (sumcheck.rs:981-1014, 1054-1119); per = 2: [s0, s2] with s1 = claim - s0.
__device__ inline bool av_sumcheck(Tr& tr, const u32* polys, u32 rounds, u32 per, u32 claim, u32 final_product, u32* chal_out) {
    for (u32 rd = 0; rd < rounds; rd++) {
        const u32* p = polys + rd * per;
        u32 s[4];
        if (per == 2) { s[0] = p[0] % ZKB_P; s[1] = sub31(claim, s[0]); s[2] = p[1] % ZKB_P; }
        else { for (u32 i = 0; i < per; i++) s[i] = p[i] % ZKB_P; }
        if (add31(s[0], s[1]) != claim) return false;
        const u32 nabs = per == 4 ? 4u : 3u;
        for (u32 i = 0; i < nabs; i++) att_absorb_u32(tr, s[i]);
        const u32 r = tr_squeeze(tr);
        if (chal_out) chal_out[rd] = r;
        claim = per == 4 ? av_cubic(s, r) : av_quadratic(s[0], s[1], s[2], r);
    }
    return claim == final_product;
}
// sum_j eq(point)[j] v[j], j < n (values beyond n are zero); result in thread 0
__device__ inline u32 av_mle(const u32* point, u32 k, const u32* v, u32 n, u32* eq_scratch, u32* red) {
    att_eq(point, k, eq_scratch);
    __syncthreads();
    u64 acc = 0;
    for (u32 j = threadIdx.x; j < n; j += blockDim.x) acc += (u64)mul31(eq_scratch[j], v[j] % ZKB_P);
    u32 a = red64(acc);
    block_sum_words<1>(&a, red);
    return a;
}

struct AvArgs {
    const u32* k; const u32* v;                          // (num_kv_heads or num_heads, S, D)
    const u32* rec; const u32* bind; u32* result;        // result[row] = 1 when the row's proof holds
    u32 hpg; int gqa;
};

__global__ void __launch_bounds__(ATT_THREADS) attention_verify_kernel(AvArgs A, AvLayout L, B3Prefix pre_dig) {
    extern __shared__ __align__(16) u32 av_sm[];
    const u32 S = L.S, D = L.D, s_pad = L.s_pad, d_pad = L.d_pad;
    const u32 m_pad = s_pad > d_pad ? s_pad : d_pad;
    u32* tA = av_sm;                         // m_pad: eq table of the row point
    u32* tB = tA + m_pad;                    // m_pad: eq table of the column point / partial products
    u32* cat = tB + m_pad;                   // max(2 S + 2, D) + 16: the digest stream / matrix-vector products
    u32* part = cat + (2 * S + 2 > D ? 2 * S + 2 : D) + 16;                 // max(blockDim, d_pad)
    u32* red = part + (d_pad > (u32)ATT_THREADS ? d_pad : (u32)ATT_THREADS); // 128
    u32* misc = red + 128;                   // 64: [0] flag, [1] value, [8..16) digest, [16..32) squeezed point, [32..48) second point
    unsigned char* trbuf = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(misc + 64) + 15) & ~uintptr_t(15));
    const u32 row = blockIdx.x, h = row / S, i = row - h * S;
    const u32* kh = A.k + (size_t)(h / A.hpg) * S * D;
    const u32* vh = A.v + (size_t)(h / A.hpg) * S * D;
    const u32* rec = A.rec + (size_t)row * L.words;
    const u32* scores = A.bind + (size_t)row * (S + D);
    const u32* outp = scores + S;
    const u32 tid = threadIdx.x, nt = blockDim.x;
    u32* pt = misc + 16;
    u32* pt2 = misc + 32;
    bool ok = true;                                      // meaningful in thread 0
    Tr tr;
    if (tid == 0) {
        misc[0] = 1;
        tr_iv(tr.h);
        tr.buflen = 0; tr.total = 0; tr.buf = trbuf;
        const char lab[] = "row-attn-h", lab_gqa[] = "gqa-h";
        if (A.gqa) { for (int b = 0; b < 5; b++) tr_absorb_byte(tr, (unsigned char)lab_gqa[b]); }
        else { for (int b = 0; b < 10; b++) tr_absorb_byte(tr, (unsigned char)lab[b]); }
        att_absorb_decimal(tr, h);
        tr_absorb_byte(tr, '-'); tr_absorb_byte(tr, 'r');
        att_absorb_decimal(tr, i);
        // ---- verify_matmul(score_proof, K_head, scores, S, D) (matmul.rs:183-263) ----
        for (u32 j = 0; j < s_pad; j++) att_absorb_u32(tr, j < S ? scores[j] % ZKB_P : 0u);
        for (u32 b = 0; b < L.log_s; b++) { pt[b] = tr_squeeze(tr); ok = ok && pt[b] == rec[L.o_r1 + b]; }
        for (u32 b = 0; b < L.log_d; b++) pt2[b] = rec[L.o_s1 + b] % ZKB_P;
    }
    __syncthreads();
    u32 claim = av_mle(pt, L.log_s, scores, S, tA, red);                 // y(r); tA = eq(r) over rows
    __syncthreads();
    // K(r, s) = sum_j eq(r)[j] sum_l K[j, l] eq(s)[l]
    att_eq(pt2, L.log_d, tB);
    __syncthreads();
    att_rows_dot(kh, S, D, tB, cat);                                     // cat[j] = sum_l K[j, l] eq(s)[l]  (S <= 2 S + 2 words)
    __syncthreads();
    u32 w_rs;
    {
        u64 acc = 0;
        for (u32 j = tid; j < S; j += nt) acc += (u64)mul31(tA[j], cat[j]);
        w_rs = red64(acc);
        block_sum_words<1>(&w_rs, red);
    }
    if (tid == 0) {
        const u32 w_at = rec[L.o_sc1_fin] % ZKB_P, x_at = rec[L.o_sc1_fin + 1] % ZKB_P;
        ok = ok && av_sumcheck(tr, rec + L.o_sc1_polys, L.log_d, 3, claim, mul31(w_at, x_at), nullptr);
        ok = ok && w_rs == w_at;
        // ---- verify_softmax (softmax.rs:139-238): verify_lookup first (lookup.rs:803-874) ----
        u32 nz = 0;
        for (int b = 0; b < 8; b++) nz |= rec[L.o_digest + b];
        misc[1] = nz;
    }
    __syncthreads();
    if (misc[1]) {                                                       // external_data_digest present: it must be the digest of (inputs, outputs)
        for (u32 t = tid; t < 2 * S + 2; t += nt) cat[t] = t < S ? rec[L.o_lk_in + t] : (t == S ? S : (t == S + 1 ? 0u : rec[L.o_lk_out + t - S - 2]));
        __syncthreads();
        b3_hash_block(pre_dig, cat, 2 * S + 2, misc + 8);
        if (tid == 0) for (int b = 0; b < 8; b++) ok = ok && misc[8 + b] == rec[L.o_digest + b];
        __syncthreads();
    }
    if (tid == 0) {
        for (int b = 0; b < 8; b++) att_absorb_u32(tr, 0u);
        att_absorb_u32(tr, S);
        for (u32 j = 0; j < S; j++) { att_absorb_u32(tr, rec[L.o_lk_in + j] % ZKB_P); att_absorb_u32(tr, rec[L.o_lk_out + j] % ZKB_P); }
        const u32 beta = tr_squeeze(tr), alpha = tr_squeeze(tr);
        ok = ok && alpha == rec[L.o_alpha_beta] && beta == rec[L.o_alpha_beta + 1];
        for (int b = 0; b < 8; b++) att_absorb_u32(tr, rec[L.o_root_t + b]);
        for (int b = 0; b < 8; b++) att_absorb_u32(tr, rec[L.o_root_m + b]);
        const u32 fin_ones = rec[L.o_lk_fin] % ZKB_P, fin_h = rec[L.o_lk_fin + 1] % ZKB_P;
        ok = ok && av_sumcheck(tr, rec + L.o_lk_polys, rec[L.o_hdr + 1], 2, 0u, mul31(fin_ones, fin_h), nullptr);
        ok = ok && fin_ones == 1u;
        for (u32 j = 0; j < S; j++) ok = ok && rec[L.o_e + j] == rec[L.o_lk_out + j];                 // softmax.rs:157-166
        const u32 sum = rec[L.o_sum] % ZKB_P, inv_s = rec[L.o_inv_s] % ZKB_P;
        ok = ok && mul31(inv_s, sum) == 1u;
        att_absorb_u32(tr, rec[L.o_sum]);
        const u32 ones_at = rec[L.o_sc2_fin] % ZKB_P, e_at = rec[L.o_sc2_fin + 1] % ZKB_P;
        ok = ok && av_sumcheck(tr, rec + L.o_sc2_polys, L.log_s, 3, sum, mul31(ones_at, e_at), nullptr);
        ok = ok && ones_at == 1u;
        for (u32 b = 0; b < L.log_s; b++) pt[b] = tr_squeeze(tr);
    }
    __syncthreads();
    claim = av_mle(pt, L.log_s, rec + L.o_e, S, tA, red);                // e(r)
    if (tid == 0) {
        const u32 eq_at = rec[L.o_sc3_fin] % ZKB_P, y_at = rec[L.o_sc3_fin + 1] % ZKB_P, s_at = rec[L.o_sc3_fin + 2] % ZKB_P;
        ok = ok && av_sumcheck(tr, rec + L.o_sc3_polys, L.log_s, 4, claim, mul31(mul31(eq_at, y_at), s_at), nullptr);
        u32 eq = 1;                                                      // compute_eq_at_point(r_point, output_proof.challenges)
        for (u32 b = 0; b < L.log_s; b++) {
            const u32 a = pt[b], c = rec[L.o_sc3_chal + b] % ZKB_P;
            eq = mul31(eq, add31(mul31(a, c), mul31(sub31(1, a), sub31(1, c))));
        }
        ok = ok && eq == eq_at && s_at == rec[L.o_sum] % ZKB_P;
        // ---- verify_matmul(output_proof, V_head^T, output, D, S) ----
        for (u32 l = 0; l < d_pad; l++) att_absorb_u32(tr, l < D ? outp[l] % ZKB_P : 0u);
        for (u32 b = 0; b < L.log_d; b++) { pt[b] = tr_squeeze(tr); ok = ok && pt[b] == rec[L.o_r4 + b]; }
        for (u32 b = 0; b < L.log_s; b++) pt2[b] = rec[L.o_s4 + b] % ZKB_P;
    }
    __syncthreads();
    claim = av_mle(pt, L.log_d, outp, D, tA, red);                       // out(r); tA = eq(r) over d_head
    __syncthreads();
    // V^T(r, s) = sum_c eq(r)[c] sum_l V[l, c] eq(s)[l]
    att_eq(pt2, L.log_s, tB);
    __syncthreads();
    att_cols_dot(vh, S, D, tB, cat, part);                               // cat[c] = sum_l V[l, c] eq(s)[l]
    u32 v_rs;
    {
        u64 acc = 0;
        for (u32 c = tid; c < D; c += nt) acc += (u64)mul31(tA[c], cat[c]);
        v_rs = red64(acc);
        block_sum_words<1>(&v_rs, red);
    }
    if (tid == 0) {
        const u32 w_at = rec[L.o_sc4_fin] % ZKB_P, x_at = rec[L.o_sc4_fin + 1] % ZKB_P;
        ok = ok && av_sumcheck(tr, rec + L.o_sc4_polys, L.log_s, 3, claim, mul31(w_at, x_at), nullptr);
        ok = ok && v_rs == w_at;
        A.result[row] = ok ? 1u : 0u;
    }
}

// ---- host ---------------------------------------------------------------------------------------------------------
struct AvRun { u32 rows = 0; u32* result_dev = nullptr; };
// k, v: device pointers.  The caller's transcript absorbs the dimensions and every row's scores and outputs (attention.rs:288-291, 371-383).
inline AvRun attention_verify_enqueue(zkb_ctx* c, TrState* tr, const AvParsed& pr, const u32* k, const u32* v, u32 num_kv_heads) {
    const AvLayout& L = pr.L;
    AvRun run;
    run.rows = pr.num_heads * pr.S;
    u32* rec = (u32*)c->scratch(pr.rec.size() * 4 + 16);
    u32* bind = (u32*)c->scratch(pr.bind.size() * 4 + 16);
    run.result_dev = (u32*)c->scratch((size_t)run.rows * 4 + 16);
    ZKB_CUDA(cudaMemcpyAsync(rec, pr.rec.data(), pr.rec.size() * 4, cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemcpyAsync(bind, pr.bind.data(), pr.bind.size() * 4, cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemsetAsync(run.result_dev, 0, (size_t)run.rows * 4, c->stream));
    const size_t smem = av_smem_bytes(L);
    static std::mutex mu;
    static size_t allowed[64] = {0};
    {
        std::lock_guard<std::mutex> g(mu);
        if (c->device < 64 && smem + 8192 > 48 * 1024 && allowed[c->device] < smem) {
            ZKB_CUDA(cudaFuncSetAttribute(attention_verify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            allowed[c->device] = smem;
        }
    }
    unsigned char pre[31];
    memcpy(pre, "lookup-external-data-v1", 23);
    u64 n64 = L.S;
    memcpy(pre + 23, &n64, 8);
    const bool in_order = c->opt_bf_in_order || c->capturing || !tr;       // without a transcript to advance there is nothing to overlap
    cudaStream_t rows_stream = in_order ? c->stream : c->side_stream();
    if (!in_order) {
        ZKB_CUDA(cudaEventRecord(c->side_event(0), c->stream));
        ZKB_CUDA(cudaStreamWaitEvent(rows_stream, c->side_event(0), 0));
    }
    AvArgs A{k, v, rec, bind, run.result_dev, att_heads_per_group(pr.num_heads, num_kv_heads), num_kv_heads != 0};
    const int threads = c->opt_att_threads ? c->opt_att_threads : ((L.s_pad >= 512 || L.d_pad > 128) ? 256 : 128);
    attention_verify_kernel<<<run.rows, threads, smem, rows_stream>>>(A, L, b3_prefix(pre, 31));
    ZKB_LAUNCHED(c);
    if (!in_order) ZKB_CUDA(cudaEventRecord(c->side_event(1), rows_stream));
    if (tr) {
        ScriptBuilder sb;
        sb.word(pr.num_heads);
        if (num_kv_heads) sb.word(num_kv_heads);
        sb.word(pr.S); sb.word(pr.D);
        sb.words_dev(bind, (u32)pr.bind.size());
        sb.run(c, tr);
    }
    if (!in_order) ZKB_CUDA(cudaStreamWaitEvent(c->stream, c->side_event(1), 0));
    ZKB_CUDA(cudaGetLastError());
    return run;
}

}  // namespace zkb
