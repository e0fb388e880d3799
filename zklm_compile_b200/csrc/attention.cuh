// Row-decomposed attention for seq_len >= 2: one CTA proves one (head, row).
//
//   prove_row_attention   rust/zk_ml_prover/src/proving/attention.rs:116-276
//   prove_softmax         rust/zk_ml_prover/src/proving/softmax.rs:56-131
//   prove_matmul          rust/zk_ml_prover/src/proving/matmul.rs:134-180
//   prove_lookup (base)   rust/zk_ml_prover/src/proving/lookup.rs:432-604
//   forward pass          rust/zk_ml_prover/src/pipeline/forward.rs:233-276
//
// Every row has a transcript of its own ("row-attn-h{h}-r{i}"), so the num_heads * seq_len row proofs
// are independent hash chains.  The reference spreads them over CPU threads; here each is one CTA that
// keeps the row's vectors (scores, exp values, weights, the sumcheck tables, the LogUp subtable) in
// shared memory for the whole proof and runs its SHA-256 chain on thread 0, so a launch keeps hundreds
// of chains in flight (several CTAs per SM).  K and V of a head are read from L2 by all of its rows.
// What a row stores (round polynomials, challenges, roots, final evaluations, e, y) goes into a
// fixed-layout record that the host turns into the reference's bincode; scores and outputs go into a
// contiguous buffer whose word order is the stream the caller's transcript absorbs after the rows.
#pragma once
#include "engine.cuh"
#include "logup.cuh"

namespace zkb {

constexpr int ATT_THREADS = 256;
constexpr u32 ATT_MAX_SEQ = 1024, ATT_MAX_DHEAD = 256;
constexpr u32 ST_ATT_ZERO_SUM = 11;

ZKB_HD u32 att_log2_ceil(u32 n) {                       // common.rs:16-21, minimum 1
    if (n <= 1) return 1;
    u32 k = 0;
    while ((1u << k) < n) k++;
    return k;
}

// Word offsets inside one row's record.
struct AttLayout {
    u32 S, D, log_s, log_d, s_pad, d_pad, nv_max;
    u32 o_hdr;                                            // n_active, nv
    u32 o_sc1_polys, o_sc1_chal, o_sc1_fin, o_r1;         // score matmul: log_d rounds of 3, finals (w, x), r (log_s)
    u32 o_root_t, o_root_m, o_lk_polys, o_lk_chal, o_lk_fin, o_alpha_beta, o_digest;
    u32 o_sum, o_sc2_polys, o_sc2_chal, o_sc2_fin;        // sum of e: log_s rounds of 3, finals (ones, e)
    u32 o_sc3_polys, o_sc3_chal, o_sc3_fin, o_inv_s;      // y * S = e: log_s rounds of 4, finals (eq, y, S)
    u32 o_sc4_polys, o_sc4_chal, o_sc4_fin, o_r4;         // output matmul: log_s rounds of 3, finals (w, x), r (log_d)
    u32 o_e, o_y;
    u32 words;
};
inline AttLayout att_layout(u32 S, u32 D) {
    AttLayout L{};
    L.S = S; L.D = D;
    L.log_s = att_log2_ceil(S); L.log_d = att_log2_ceil(D);
    L.s_pad = 1u << L.log_s; L.d_pad = 1u << L.log_d;
    L.nv_max = att_log2_ceil(2 * S);
    u32 o = 0;
    auto take = [&](u32 n) { u32 at = o; o += n; return at; };
    L.o_hdr = take(2);
    L.o_sc1_polys = take(3 * L.log_d); L.o_sc1_chal = take(L.log_d); L.o_sc1_fin = take(2); L.o_r1 = take(L.log_s);
    L.o_root_t = take(8); L.o_root_m = take(8); L.o_lk_polys = take(2 * L.nv_max); L.o_lk_chal = take(L.nv_max); L.o_lk_fin = take(1);
    L.o_alpha_beta = take(2); L.o_digest = take(8);
    L.o_sum = take(1); L.o_sc2_polys = take(3 * L.log_s); L.o_sc2_chal = take(L.log_s); L.o_sc2_fin = take(2);
    L.o_sc3_polys = take(4 * L.log_s); L.o_sc3_chal = take(L.log_s); L.o_sc3_fin = take(3); L.o_inv_s = take(1);
    L.o_sc4_polys = take(3 * L.log_s); L.o_sc4_chal = take(L.log_s); L.o_sc4_fin = take(2); L.o_r4 = take(L.log_d);
    L.o_e = take(S); L.o_y = take(S);
    L.words = (o + 3) & ~3u;
    return L;
}
// Shared-memory words of one CTA (the arrays listed at the top of the kernel, in order).
inline size_t att_smem_bytes(const AttLayout& L) {
    const u32 m_pad = L.s_pad > L.d_pad ? L.s_pad : L.d_pad;
    const u32 part = L.d_pad > (u32)ATT_THREADS ? L.d_pad : (u32)ATT_THREADS;
    const u32 a_pad = 2 * L.s_pad > m_pad ? 2 * L.s_pad : m_pad;
    size_t w = 3 * (size_t)L.s_pad + ((size_t)a_pad + 16) + 2 * (size_t)m_pad + 4 * (size_t)L.s_pad + 2 * (size_t)L.d_pad + part + 128 + 64;
    return w * 4 + TR_SCRATCH_BYTES + 16;
}

// One word into the stream at any byte offset (the row label's length is arbitrary, so the stream is
// rarely word-aligned): two shifted word stores instead of four byte stores.
__device__ __forceinline__ void att_absorb_u32(Tr& t, u32 v) {
    const u32 s = t.buflen & 3;
    u32* bw = reinterpret_cast<u32*>(t.buf);
    if (s == 0) {
        bw[t.buflen >> 2] = v;
        t.buflen += 4;
        t.total += 4;
        if (t.buflen == 64) tr_flush_block(t);
    } else {
        const u32 wi = t.buflen >> 2, sh = 8 * s;
        bw[wi] = (bw[wi] & ((1u << sh) - 1u)) | (v << sh);
        t.total += 4;
        if (wi == 15) {
            t.buflen = 64;
            tr_flush_block(t);
            bw[0] = v >> (32 - sh);
            t.buflen = s;
        } else {
            bw[wi + 1] = v >> (32 - sh);
            t.buflen += 4;
        }
    }
}
__device__ inline void att_absorb_decimal(Tr& t, u32 x) {
    unsigned char d[10];
    int n = 0;
    do { d[n++] = (unsigned char)('0' + x % 10); x /= 10; } while (x);
    while (n) tr_absorb_byte(t, d[--n]);
}

// out[j] = sum_l M[j, l] x[l], j < rows; a warp per row.
__device__ inline void att_rows_dot(const u32* __restrict__ M, u32 rows, u32 cols, const u32* x, u32* out) {
    const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (u32 j = warp; j < rows; j += nwarps) {
        u64 acc = 0;
        for (u32 l = lane; l < cols; l += 32) acc += (u64)mul31(M[(size_t)j * cols + l], x[l]);
        u32 a = red64(acc);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a = add31(a, __shfl_down_sync(0xffffffffu, a, off));
        if (lane == 0) out[j] = a;
    }
}
// out[l] = sum_j x[j] M[j, l], l < cols; `part` holds max(blockDim, cols) words.  Ends with a barrier.
__device__ inline void att_cols_dot(const u32* __restrict__ M, u32 rows, u32 cols, const u32* x, u32* out, u32* part) {
    const u32 G = cols >= blockDim.x ? 1u : blockDim.x / cols;
    for (u32 p = threadIdx.x; p < G * cols; p += blockDim.x) {
        const u32 g = p / cols, l = p - g * cols;
        u64 acc = 0;
        for (u32 j = g; j < rows; j += G) acc += (u64)mul31(x[j], M[(size_t)j * cols + l]);
        part[p] = red64(acc);
    }
    __syncthreads();
    for (u32 l = threadIdx.x; l < cols; l += blockDim.x) {
        u32 a = 0;
        for (u32 g = 0; g < G; g++) a = add31(a, part[g * cols + l]);
        out[l] = a;
    }
    __syncthreads();
}
// eq table of a base-field point, r[0] the most significant variable (m31_ops.rs:30-50).
__device__ inline void att_eq(const u32* r, u32 k, u32* out) {
    for (u32 x = threadIdx.x; x < (1u << k); x += blockDim.x) {
        u32 prod = 1;
        for (u32 i = 0; i < k; i++) {
            const u32 ri = r[i];
            prod = mul31(prod, ((x >> (k - 1 - i)) & 1u) ? ri : sub31(1u, ri));
        }
        out[x] = prod;
    }
}

// Sumcheck over tables in shared memory (sumcheck.rs:211-272 product, :277-354 triple, :857-902 all-ones);
// thread 0 owns the transcript.  Stored per round: 3 / 4 / 2 ([s0, s2]) words.  Tables are folded in
// place; t?[0] hold the final evaluations afterwards.  All threads of the CTA must call.
template <int KIND>
__device__ inline void att_sumcheck(u32* t0, u32* t1, u32* t2, u32 nv, Tr& tr, u32* polys, u32* chal, u32* red, u32* r_sh, u32* status) {
    constexpr int NACC = KIND == SC_PRODUCT ? 3 : (KIND == SC_TRIPLE ? 4 : 2);
    u32 size = 1u << nv;
    for (u32 rd = 0; rd < nv; rd++) {
        const u32 half = size >> 1;
        u64 a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        for (u32 j = threadIdx.x; j < half; j += blockDim.x) {
            const u32 f0 = t0[j], f1 = t0[j + half];
            if constexpr (KIND == SC_ONES) {
                a0 += f0; a1 += f1;
            } else {
                const u32 g0 = t1[j], g1 = t1[j + half];
                const u32 f2 = sub31(add31(f1, f1), f0), g2 = sub31(add31(g1, g1), g0);
                if constexpr (KIND == SC_PRODUCT) {
                    a0 += mul31(f0, g0); a1 += mul31(f1, g1); a2 += mul31(f2, g2);
                } else {
                    const u32 h0 = t2[j], h1 = t2[j + half];
                    const u32 h2 = sub31(add31(h1, h1), h0);
                    const u32 f3 = sub31(mul31(3u, f1), mul31(2u, f0)), g3 = sub31(mul31(3u, g1), mul31(2u, g0)),
                              h3 = sub31(mul31(3u, h1), mul31(2u, h0));
                    a0 += mul31(mul31(f0, g0), h0); a1 += mul31(mul31(f1, g1), h1);
                    a2 += mul31(mul31(f2, g2), h2); a3 += mul31(mul31(f3, g3), h3);
                }
            }
        }
        u32 w[NACC];
        w[0] = red64(a0); w[1] = red64(a1);
        if constexpr (NACC > 2) w[2] = red64(a2);
        if constexpr (NACC > 3) w[3] = red64(a3);
        block_sum_words<NACC>(w, red);
        if (threadIdx.x == 0) {
            if constexpr (KIND == SC_ONES) {
                const u32 s2 = sub31(add31(w[1], w[1]), w[0]);
                if (rd == 0 && add31(w[0], w[1]) != 0) atomicExch(status, ST_LOGUP_IDENTITY);
                att_absorb_u32(tr, w[0]); att_absorb_u32(tr, w[1]); att_absorb_u32(tr, s2);
                polys[2 * rd] = w[0]; polys[2 * rd + 1] = s2;
            } else {
#pragma unroll
                for (int k = 0; k < NACC; k++) { att_absorb_u32(tr, w[k]); polys[NACC * rd + k] = w[k]; }
            }
            const u32 r = tr_squeeze(tr);
            chal[rd] = r;
            r_sh[0] = r;
        }
        __syncthreads();
        const u32 r = r_sh[0];
        for (u32 j = threadIdx.x; j < half; j += blockDim.x) {
            { const u32 a = t0[j]; t0[j] = add31(a, mul31(r, sub31(t0[j + half], a))); }
            if constexpr (KIND != SC_ONES) { const u32 a = t1[j]; t1[j] = add31(a, mul31(r, sub31(t1[j + half], a))); }
            if constexpr (KIND == SC_TRIPLE) { const u32 a = t2[j]; t2[j] = add31(a, mul31(r, sub31(t2[j + half], a))); }
        }
        __syncthreads();
        size = half;
    }
}

struct AttArgs {
    const u32* q; const u32* k; const u32* v;           // (num_heads, S, D)
    const u32* table_out; u32 n_table;
    u32* attn_out;                                       // (num_heads, S, D)
    u32* bind;                                           // per row: scores (S) | output (D)
    u32* rec;                                            // per row: L.words
    u32* status;
    int prove;                                           // 0: forward pass only
    u32 hpg;                                             // query heads per K/V head (1 unless GQA)
    int gqa;                                             // rows are labelled "gqa-h{h}-r{i}" (attention.rs:427) instead of "row-attn-h{h}-r{i}"
};

__global__ void __launch_bounds__(ATT_THREADS) attention_row_kernel(AttArgs A, AttLayout L, B3Prefix pre_w, B3Prefix pre_dig) {
    extern __shared__ __align__(16) u32 att_sm[];
    const u32 S = L.S, D = L.D, s_pad = L.s_pad, d_pad = L.d_pad;
    const u32 m_pad = s_pad > d_pad ? s_pad : d_pad;
    const u32 part_n = d_pad > (u32)ATT_THREADS ? d_pad : (u32)ATT_THREADS;
    u32* sc = att_sm;                         // scores, zero-padded
    u32* ev = sc + s_pad;                     // exp values
    u32* yv = ev + s_pad;                     // softmax weights
    u32* tA = yv + s_pad;                     // max(2 s_pad, m_pad) + 16: sumcheck table / LogUp h / digest stream
    u32* tB = tA + (2 * s_pad > m_pad ? 2 * s_pad : m_pad) + 16;   // m_pad
    u32* tC = tB + m_pad;                     // m_pad
    u32* idx = tC + m_pad;                    // table index of each score
    u32* mlt = idx + s_pad;                   // multiplicity at the first occurrence of an index, else 0
    u32* act_enc = mlt + s_pad;               // active subtable, encoded
    u32* act_mult = act_enc + s_pad;
    u32* qv = act_mult + s_pad;               // d_pad
    u32* outv = qv + d_pad;                   // d_pad
    u32* part = outv + d_pad;                 // part_n
    u32* red = part + part_n;                 // 128
    u32* misc = red + 128;                    // 64: [0] r, [1] flags, [2] sum, [3] n_active, [4] beta, [5] alpha, [8..24) roots, [24..32) digest, [32..48) point
    unsigned char* trbuf = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(misc + 64) + 15) & ~uintptr_t(15));

    const u32 row = blockIdx.x, h = row / S, i = row - h * S;
    const u32* kh = A.k + (size_t)(h / A.hpg) * S * D;
    const u32* vh = A.v + (size_t)(h / A.hpg) * S * D;
    const u32* qrow = A.q + ((size_t)h * S + i) * D;
    u32* rec = A.rec ? A.rec + (size_t)row * L.words : nullptr;
    u32* bind = A.bind ? A.bind + (size_t)row * (S + D) : nullptr;
    const u32 tid = threadIdx.x, nt = blockDim.x;

    // ---- forward pass of the row (forward.rs:250-274) ----------------------------------------
    for (u32 l = tid; l < d_pad; l += nt) qv[l] = l < D ? qrow[l] : 0u;
    if (tid == 0) misc[1] = 0;
    __syncthreads();
    att_rows_dot(kh, S, D, qv, sc);
    for (u32 j = S + tid; j < s_pad; j += nt) sc[j] = 0;
    __syncthreads();
    u32 esum = 0;
    for (u32 j = tid; j < s_pad; j += nt) {
        u32 e = 0, ix = 0xffffffffu;
        if (j < S) {
            ix = field_to_table_index(sc[j], A.n_table);
            if (ix < A.n_table) e = A.table_out[ix];
            else misc[1] = 1;                              // the reference's map lookup panics (attention.rs:105)
        }
        idx[j] = ix; ev[j] = e;
        esum = add31(esum, e);
    }
    block_sum_words<1>(&esum, red);
    if (tid == 0) misc[2] = esum;
    __syncthreads();
    const u32 sum = misc[2];
    if (misc[1] || sum == 0) {
        if (tid == 0) atomicExch(A.status, misc[1] ? (u32)ST_LOOKUP_KEY : ST_ATT_ZERO_SUM);
        return;
    }
    const u32 inv_s = inv31(sum);
    for (u32 j = tid; j < s_pad; j += nt) yv[j] = mul31(ev[j], inv_s);
    __syncthreads();
    att_cols_dot(vh, S, D, yv, outv, part);
    for (u32 l = D + tid; l < d_pad; l += nt) outv[l] = 0;
    __syncthreads();
    if (A.attn_out) for (u32 l = tid; l < D; l += nt) A.attn_out[((size_t)h * S + i) * D + l] = outv[l];
    if (bind) {
        for (u32 j = tid; j < S; j += nt) bind[j] = sc[j];
        for (u32 l = tid; l < D; l += nt) bind[S + l] = outv[l];
    }
    if (!A.prove) return;
    for (u32 j = tid; j < S; j += nt) { rec[L.o_e + j] = ev[j]; rec[L.o_y + j] = yv[j]; }

    Tr tr;
    if (tid == 0) {
        tr_iv(tr.h);
        tr.buflen = 0; tr.total = 0; tr.buf = trbuf;
        const char lab[] = "row-attn-h", lab_gqa[] = "gqa-h";
        if (A.gqa) { for (int b = 0; b < 5; b++) tr_absorb_byte(tr, (unsigned char)lab_gqa[b]); }
        else { for (int b = 0; b < 10; b++) tr_absorb_byte(tr, (unsigned char)lab[b]); }
        att_absorb_decimal(tr, h);
        tr_absorb_byte(tr, '-'); tr_absorb_byte(tr, 'r');
        att_absorb_decimal(tr, i);
    }
    u32* pt = misc + 32;

    // ---- scores = K_head q (matmul.rs:134-180 with W = K_head, m = S, n = D) ----------------------
    if (tid == 0) {
        for (u32 j = 0; j < s_pad; j++) att_absorb_u32(tr, sc[j]);
        for (u32 b = 0; b < L.log_s; b++) { const u32 r = tr_squeeze(tr); pt[b] = r; rec[L.o_r1 + b] = r; }
    }
    __syncthreads();
    att_eq(pt, L.log_s, tC);
    __syncthreads();
    att_cols_dot(kh, S, D, tC, tA, part);
    for (u32 l = D + tid; l < d_pad; l += nt) tA[l] = 0;
    for (u32 l = tid; l < d_pad; l += nt) tB[l] = qv[l];
    __syncthreads();
    att_sumcheck<SC_PRODUCT>(tA, tB, nullptr, L.log_d, tr, rec + L.o_sc1_polys, rec + L.o_sc1_chal, red, misc, A.status);
    if (tid == 0) { rec[L.o_sc1_fin] = tA[0]; rec[L.o_sc1_fin + 1] = tB[0]; }
    __syncthreads();

    // ---- e = exp_table(scores) by LogUp (lookup.rs:432-604) -------------------------------------
    if (tid == 0) {
        for (int b = 0; b < 8; b++) att_absorb_u32(tr, 0u);          // the zero table root
        att_absorb_u32(tr, S);
        for (u32 j = 0; j < S; j++) { att_absorb_u32(tr, sc[j]); att_absorb_u32(tr, ev[j]); }
        const u32 beta = tr_squeeze(tr), alpha = tr_squeeze(tr);
        misc[4] = beta; misc[5] = alpha;
        rec[L.o_alpha_beta] = alpha; rec[L.o_alpha_beta + 1] = beta;
    }
    // multiplicities: the active entries in table order, without a 65536-entry histogram
    u32 n_first = 0;
    for (u32 j = tid; j < S; j += nt) {
        const u32 me = idx[j];
        u32 m = 0; bool first = true;
        for (u32 l = 0; l < S; l++) if (idx[l] == me) { m++; if (l < j) first = false; }
        mlt[j] = first ? m : 0u;
        n_first += first ? 1u : 0u;
    }
    block_sum_words<1>(&n_first, red);                                   // counts stay far below p
    if (tid == 0) misc[3] = n_first;
    __syncthreads();
    const u32 n_active = misc[3], beta = misc[4], alpha = misc[5];
    for (u32 j = tid; j < S; j += nt) {
        if (!mlt[j]) continue;
        const u32 me = idx[j];
        u32 rank = 0;
        for (u32 l = 0; l < S; l++) rank += (mlt[l] != 0 && idx[l] < me) ? 1u : 0u;
        act_enc[rank] = add31(table_input_at(me, A.n_table), mul31(beta, A.table_out[me]));
        act_mult[rank] = mlt[j];
    }
    __syncthreads();
    b3_hash_block(pre_w, act_enc, n_active, misc + 8);
    b3_hash_block(pre_w, act_mult, n_active, misc + 16);
    const u32 nv = att_log2_ceil(S + n_active);
    for (u32 t = tid; t < (1u << nv); t += nt) {
        u32 hv = 0;
        if (t < S) {
            const u32 d = sub31(alpha, add31(sc[t], mul31(beta, ev[t])));
            if (d == 0) atomicExch(A.status, ST_ALPHA_COLLISION);
            hv = inv31(d);
        } else if (t < S + n_active) {
            const u32 d = sub31(alpha, act_enc[t - S]);
            if (d == 0) atomicExch(A.status, ST_ALPHA_COLLISION);
            hv = neg31(mul31(act_mult[t - S], inv31(d)));
        }
        tA[t] = hv;
    }
    if (tid == 0) {
        rec[L.o_hdr] = n_active; rec[L.o_hdr + 1] = nv;
        for (int b = 0; b < 8; b++) { att_absorb_u32(tr, misc[8 + b]); rec[L.o_root_t + b] = misc[8 + b]; }
        for (int b = 0; b < 8; b++) { att_absorb_u32(tr, misc[16 + b]); rec[L.o_root_m + b] = misc[16 + b]; }
    }
    __syncthreads();
    att_sumcheck<SC_ONES>(tA, nullptr, nullptr, nv, tr, rec + L.o_lk_polys, rec + L.o_lk_chal, red, misc, A.status);
    if (tid == 0) rec[L.o_lk_fin] = tA[0];
    __syncthreads();
    for (u32 t = tid; t < 2 * S + 2; t += nt) tA[t] = t < S ? sc[t] : (t == S ? S : (t == S + 1 ? 0u : ev[t - S - 2]));
    __syncthreads();
    b3_hash_block(pre_dig, tA, 2 * S + 2, misc + 24);
    if (tid < 8) rec[L.o_digest + tid] = misc[24 + tid];
    __syncthreads();

    // ---- S = sum e (softmax.rs:78-96) --------------------------------------------------------
    if (tid == 0) { att_absorb_u32(tr, sum); rec[L.o_sum] = sum; rec[L.o_inv_s] = inv_s; }
    for (u32 j = tid; j < s_pad; j += nt) { tA[j] = 1u; tB[j] = ev[j]; }
    __syncthreads();
    att_sumcheck<SC_PRODUCT>(tA, tB, nullptr, L.log_s, tr, rec + L.o_sc2_polys, rec + L.o_sc2_chal, red, misc, A.status);
    if (tid == 0) {
        rec[L.o_sc2_fin] = tA[0]; rec[L.o_sc2_fin + 1] = tB[0];
        for (u32 b = 0; b < L.log_s; b++) pt[b] = tr_squeeze(tr);
    }
    __syncthreads();
    // ---- y[i] * S = e[i] at a random point (softmax.rs:98-118) ------------------------------------
    att_eq(pt, L.log_s, tA);
    for (u32 j = tid; j < s_pad; j += nt) { tB[j] = yv[j]; tC[j] = sum; }
    __syncthreads();
    att_sumcheck<SC_TRIPLE>(tA, tB, tC, L.log_s, tr, rec + L.o_sc3_polys, rec + L.o_sc3_chal, red, misc, A.status);
    if (tid == 0) { rec[L.o_sc3_fin] = tA[0]; rec[L.o_sc3_fin + 1] = tB[0]; rec[L.o_sc3_fin + 2] = tC[0]; }
    __syncthreads();

    // ---- out = V_head^T y (matmul.rs:134-180 with W = V_head^T, m = D, n = S) ----------------------
    if (tid == 0) {
        for (u32 l = 0; l < d_pad; l++) att_absorb_u32(tr, outv[l]);
        for (u32 b = 0; b < L.log_d; b++) { const u32 r = tr_squeeze(tr); pt[b] = r; rec[L.o_r4 + b] = r; }
    }
    __syncthreads();
    att_eq(pt, L.log_d, tC);
    __syncthreads();
    att_rows_dot(vh, S, D, tC, tA);
    for (u32 j = S + tid; j < s_pad; j += nt) tA[j] = 0;
    for (u32 j = tid; j < s_pad; j += nt) tB[j] = yv[j];
    __syncthreads();
    att_sumcheck<SC_PRODUCT>(tA, tB, nullptr, L.log_s, tr, rec + L.o_sc4_polys, rec + L.o_sc4_chal, red, misc, A.status);
    if (tid == 0) { rec[L.o_sc4_fin] = tA[0]; rec[L.o_sc4_fin + 1] = tB[0]; }
}

// ---- host side ------------------------------------------------------------------------------
struct AttRun { AttLayout L; u32 rows; u32* rec; u32* bind; };

inline void att_check_dims(size_t num_heads, size_t S, size_t D, size_t n_table) {
    if (num_heads == 0 || S == 0 || D == 0) throw ArgFail{ZKB_E_ARG, "attention: empty dimension"};
    if (S > ATT_MAX_SEQ || D > ATT_MAX_DHEAD) throw ArgFail{ZKB_E_TOO_LARGE, "attention: seq_len above 1024 or d_head above 256"};
    if (num_heads * S > (size_t)1 << 22) throw ArgFail{ZKB_E_TOO_LARGE, "attention: more than 2^22 rows"};
    if (n_table != 256 && n_table != 65536) throw ArgFail{ZKB_E_ARG, "attention: the exp table has 256 or 65536 entries"};
}
inline void att_launch(zkb_ctx* c, cudaStream_t stream, const AttArgs& A, const AttLayout& L, u32 rows) {
    const size_t smem = att_smem_bytes(L);
    static std::mutex mu;
    static size_t allowed[64] = {0};
    {
        std::lock_guard<std::mutex> g(mu);
        if (c->device < 64 && smem + 8192 > 48 * 1024 && allowed[c->device] < smem) {   // the kernel also has 4 KB of static shared memory
            ZKB_CUDA(cudaFuncSetAttribute(attention_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            allowed[c->device] = smem;
        }
    }
    unsigned char pre[31];
    memcpy(pre, "lookup-external-data-v1", 23);
    u64 n64 = L.S;
    memcpy(pre + 23, &n64, 8);
    // A row's critical path is thread 0's hash chain; the data-parallel phases touch at most 2 * s_pad elements.
    // Fewer threads per CTA let more rows share an SM.
    const int threads = c->opt_att_threads ? c->opt_att_threads : ((L.s_pad >= 512 || L.d_pad > 128) ? 256 : 128);
    attention_row_kernel<<<rows, threads, smem, stream>>>(A, L, b3_prefix("weights", 7), b3_prefix(pre, 31));
    ZKB_LAUNCHED(c);
}
// The op's forward pass over all (head, row) pairs.  q, k, v, table_out, attn_out: device pointers.
// num_kv_heads = 0: k, v have num_heads heads; otherwise grouped-query attention (k, v have num_kv_heads heads).
inline u32 att_heads_per_group(size_t num_heads, size_t num_kv_heads) {
    if (!num_kv_heads) return 1;
    if (num_heads % num_kv_heads) throw ArgFail{ZKB_E_ARG, "attention: num_q_heads must be divisible by num_kv_heads"};
    return (u32)(num_heads / num_kv_heads);
}
inline void attention_forward_enqueue(zkb_ctx* c, const u32* q, const u32* k, const u32* v, u32 num_heads, u32 num_kv_heads, u32 S, u32 D,
                                      const u32* table_out, u32 n_table, u32* attn_out) {
    AttArgs A{q, k, v, table_out, n_table, attn_out, nullptr, nullptr, c->status, 0, att_heads_per_group(num_heads, num_kv_heads), num_kv_heads != 0};
    att_launch(c, c->stream, A, att_layout(S, D), num_heads * S);
}
// The whole proof: the forward pass writes the scores | outputs stream, after which the row proofs (every SM but
// one, for milliseconds) and the caller's transcript absorbing that stream (one thread, one SM, one SHA-256 block
// after the other) do not depend on each other, so the rows run on the context's second stream.
// host_rec / host_bind: page-locked destinations of the records and of the scores | outputs stream.
inline AttRun attention_prove_enqueue(zkb_ctx* c, TrState* tr, const u32* q, const u32* k, const u32* v, u32 num_heads, u32 num_kv_heads, u32 S, u32 D,
                                      const u32* table_out, u32 n_table, u32* attn_out, u32* host_rec, u32* host_bind) {
    AttRun R;
    R.L = att_layout(S, D);
    R.rows = num_heads * S;
    R.rec = (u32*)c->scratch((size_t)R.rows * R.L.words * 4);
    R.bind = (u32*)c->scratch((size_t)R.rows * (S + D) * 4);
    const bool in_order = c->opt_bf_in_order || c->capturing;
    const u32 hpg = att_heads_per_group(num_heads, num_kv_heads);
    const int gqa = num_kv_heads != 0;
    if (!tr) {
        // The caller keeps its transcript and absorbs the dimensions, scores and outputs itself (attention.rs:140-143, 254-265: they are
        // in the proof it gets back): one launch computes the rows' forward values and proves them, and no serial hash runs on the GPU.
        AttArgs A{q, k, v, table_out, n_table, attn_out, R.bind, R.rec, c->status, 1, hpg, gqa};
        att_launch(c, c->stream, A, R.L, R.rows);
        ZKB_CUDA(cudaMemcpyAsync(host_bind, R.bind, (size_t)R.rows * (S + D) * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaMemcpyAsync(host_rec, R.rec, (size_t)R.rows * R.L.words * 4, cudaMemcpyDeviceToHost, c->stream));
        return R;
    }
    AttArgs F{q, k, v, table_out, n_table, attn_out, R.bind, nullptr, c->status, 0, hpg, gqa};
    att_launch(c, c->stream, F, R.L, R.rows);
    ZKB_CUDA(cudaMemcpyAsync(host_bind, R.bind, (size_t)R.rows * (S + D) * 4, cudaMemcpyDeviceToHost, c->stream));
    cudaStream_t rows_stream = in_order ? c->stream : c->side_stream();
    if (!in_order) {
        ZKB_CUDA(cudaEventRecord(c->side_event(0), c->stream));
        ZKB_CUDA(cudaStreamWaitEvent(rows_stream, c->side_event(0), 0));
    }
    AttArgs A{q, k, v, table_out, n_table, nullptr, nullptr, R.rec, c->status, 1, hpg, gqa};
    att_launch(c, rows_stream, A, R.L, R.rows);
    ZKB_CUDA(cudaMemcpyAsync(host_rec, R.rec, (size_t)R.rows * R.L.words * 4, cudaMemcpyDeviceToHost, rows_stream));
    if (!in_order) ZKB_CUDA(cudaEventRecord(c->side_event(1), rows_stream));
    {   // the dimensions, then every row's scores and outputs (attention.rs:140-143, 254-265)
        ScriptBuilder sb;
        sb.word(num_heads);
        if (gqa) sb.word(num_kv_heads);                         // attention.rs:403-406
        sb.word(S); sb.word(D);
        sb.words_dev(R.bind, (u32)((size_t)R.rows * (S + D)));
        sb.run(c, tr);
    }
    if (!in_order) ZKB_CUDA(cudaStreamWaitEvent(c->stream, c->side_event(1), 0));
    return R;
}

// RowAttentionProof (attention.rs:82-98) as bincode from the fetched records.  With p == nullptr it only counts.
struct AttSer {
    uint8_t* p;
    size_t n = 0;
    void put(const void* src, size_t bytes) { if (p) memcpy(p + n, src, bytes); n += bytes; }
    void u32le(u32 v) { put(&v, 4); }
    void u64le(u64 v) { put(&v, 8); }
    void vec(const u32* src, u32 cnt) { u64le(cnt); put(src, (size_t)cnt * 4); }
    void sumcheck(const u32* polys, u32 per, const u32* chal, u32 nv) {        // sumcheck.rs:57-65
        u64le(nv);
        for (u32 r = 0; r < nv; r++) vec(polys + (size_t)r * per, per);
        vec(chal, nv);
    }
    void commitment(const u32* root, u64 cnt) {                                   // weight_commitment.rs:54-61
        put(root, 32);
        u64le(cnt); u64le(cnt <= 1 ? 1 : att_log2_ceil((u32)cnt)); u32le(0);
    }
    void matmul(const u32* polys, const u32* chal, u32 nv, const u32* fin, const u32* r, u32 nr) {   // matmul.rs:24-31
        sumcheck(polys, 3, chal, nv);
        put(fin, 8);
        vec(r, nr); vec(chal, nv);
    }
    void row(const AttLayout& L, const u32* rec, const u32* bind) {                // attention.rs:25-42
        const u32 n_active = rec[L.o_hdr], nv = rec[L.o_hdr + 1];
        matmul(rec + L.o_sc1_polys, rec + L.o_sc1_chal, L.log_d, rec + L.o_sc1_fin, rec + L.o_r1, L.log_s);
        // SoftmaxProof (softmax.rs:20-43) starting with its LookupProof (lookup.rs:39-85)
        commitment(rec + L.o_root_t, n_active);
        commitment(rec + L.o_root_m, n_active);
        sumcheck(rec + L.o_lk_polys, 2, rec + L.o_lk_chal, nv);
        u32le(1); u32le(rec[L.o_lk_fin]);
        put(rec + L.o_alpha_beta, 8);
        vec(bind, L.S); vec(rec + L.o_e, L.S); u64le(0);
        put(rec + L.o_digest, 32);
        u32le(rec[L.o_sum]);
        sumcheck(rec + L.o_sc2_polys, 3, rec + L.o_sc2_chal, L.log_s);
        put(rec + L.o_sc2_fin, 8);
        sumcheck(rec + L.o_sc3_polys, 4, rec + L.o_sc3_chal, L.log_s);
        put(rec + L.o_sc3_fin, 12);
        u32le(rec[L.o_inv_s]);
        vec(rec + L.o_e, L.S); vec(rec + L.o_y, L.S);
        matmul(rec + L.o_sc4_polys, rec + L.o_sc4_chal, L.log_s, rec + L.o_sc4_fin, rec + L.o_r4, L.log_d);
        vec(bind, L.S); vec(rec + L.o_y, L.S); vec(bind + L.S, L.D);
    }
    void proof(const AttLayout& L, size_t num_heads, const u32* rec, const u32* bind) {
        u64le(num_heads);
        for (size_t h = 0; h < num_heads; h++) {
            u64le(L.S);
            for (size_t i = 0; i < L.S; i++) {
                const size_t r = h * L.S + i;
                row(L, rec + r * L.words, bind + r * (L.S + L.D));
            }
        }
        u64le(num_heads); u64le(L.S); u64le(L.D);
        const uint8_t none = 0;                                                    // seq1_consistency: None
        put(&none, 1);
    }
};

}  // namespace zkb
