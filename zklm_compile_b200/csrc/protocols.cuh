// Protocol layer: enqueues the kernels of each sub-protocol in the reference's transcript
// order and remembers where its outputs land in the record buffer; after the record has been
// fetched, `put_*` turns them into the reference's bincode layout.
//
//   MLE-eval proofs   rust/zk_ml_prover/src/proving/weight_commitment.rs:349-374, 470-517
//   matmul            rust/zk_ml_prover/src/proving/matmul.rs:838-997, 360-453 (default features)
//   hadamard / add    rust/zk_ml_prover/src/proving/elementwise.rs:429-480, 545-595
//   RMSNorm           rust/zk_ml_prover/src/proving/rmsnorm.rs:512-667
//   LogUp             rust/zk_ml_prover/src/proving/lookup.rs:643-762
//   gates             rust/zk_ml_prover/src/proving/sigmoid_gate.rs:90-114, swiglu.rs:99-118
#pragma once
#include "basefold.cuh"

namespace zkb {

inline u32 log2_ceil_u(size_t n) { u32 k = 1; if (n <= 1) return 1; k = 0; while ((size_t(1) << k) < n) k++; return k; }

// ---- bincode writer (bincode 1.3 defaults: LE fixed ints, u64 lengths, u8 Option tags) -------
struct Ser {
    std::vector<uint8_t> b;
    const u32* rec = nullptr;     // fetched record
    void u8(uint8_t v) { b.push_back(v); }
    void u32le(u32 v) { for (int i = 0; i < 4; i++) b.push_back(uint8_t(v >> (8 * i))); }
    void u64le(u64 v) { for (int i = 0; i < 8; i++) b.push_back(uint8_t(v >> (8 * i))); }
    void words(size_t off, size_t n) { for (size_t i = 0; i < n; i++) u32le(rec[off + i]); }
    void ef(size_t off) { words(off, 4); }
    // 32-byte root stored as 8 LE words
    void root(size_t off) { words(off, 8); }
    // WeightCommitment {root, num_weights, log_height, kind = Blake3Fast}
    void commitment(size_t root_off, u64 num_weights) {
        root(root_off);
        u64le(num_weights);
        u64le(num_weights <= 1 ? 1 : log2_ceil_u(num_weights));
        u32le(0);
    }
    // SumcheckProof / SumcheckProofEF with only the stored evaluations; challenges optional.
    void sumcheck(const ScRec& r, bool with_challenges, long nv_override = -1) {
        KindInfo ki = kind_info(r.kind);
        u32 nv = nv_override >= 0 ? (u32)nv_override : r.nv;
        u64le(nv);
        for (u32 round = 0; round < nv; round++) {
            u64le(ki.nstored);
            for (u32 k = 0; k < ki.nabs; k++)
                if (ki.mask & (1u << k)) words(r.polys + ((size_t)round * ki.nabs + k) * ki.w, ki.w);
        }
        if (with_challenges) { u64le(nv); words(r.chal, (size_t)nv * ki.w); }
        else u64le(0);
    }
    // s0 + s1 of round 0 (the claimed sum), as EF words
    void claimed_sum_ef(const ScRec& r) {
        KindInfo ki = kind_info(r.kind);
        for (int k = 0; k < 4; k++) u32le(add31(rec[r.polys + k], rec[r.polys + ki.w + k]));
    }
};

// ---- MLE-eval proof ---------------------------------------------------------------------------
struct EvalRec { ScRec sc; };
// w: base-field device vector (`len` valid entries, MLE over 2^k), point: k EF challenges on device.
// Absorbs label and root (8 words on device) first when label != nullptr.
inline EvalRec prove_mle_eval_ef_base(zkb_ctx* c, TrState* tr, const u32* w, u32 len, const Fe* point, u32 k,
                                      const char* label, const u32* root_dev) {
    if (label) {
        ScriptBuilder sb;
        sb.str(label);
        sb.words_dev(root_dev, 8);
        sb.run(c, tr);
    }
    size_t n = size_t(1) << k;
    Fe* eq = (Fe*)c->scratch(n * 16);
    Fe* wef = (Fe*)c->scratch(n * 16);
    WidenEqArgs a{};
    a.src[0] = w; a.dst[0] = wef; a.len[0] = len; a.nsrc = 1; a.point = point; a.eq_out = eq; a.k = k;
    widen_eq_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(a);
    ZKB_LAUNCHED(c);
    const u32* tabs[3] = {(const u32*)eq, (const u32*)wef, nullptr};
    ScOpts o;
    o.clobber[0] = o.clobber[1] = true;
    o.post_squeezes = 24;     // derive_query_indices (pcs.rs:442-451); the indices are not used
    EvalRec r;
    r.sc = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_EF_FULL, tabs, k, o);
    return r;
}
// EF weights (w_partial of a matmul); `w_ef` is clobbered.
inline EvalRec prove_mle_eval_ef_ef(zkb_ctx* c, TrState* tr, Fe* w_ef, const Fe* point, u32 k) {
    size_t n = size_t(1) << k;
    Fe* eq = (Fe*)c->scratch(n * 16);
    eq_evals_kernel<Fe><<<grid_for(c, n), 256, 0, c->stream>>>(point, k, eq);
    ZKB_LAUNCHED(c);
    const u32* tabs[3] = {(const u32*)eq, (const u32*)w_ef, nullptr};
    ScOpts o;
    o.clobber[0] = o.clobber[1] = true;
    o.post_squeezes = 24;
    EvalRec r;
    r.sc = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_EF_FULL, tabs, k, o);
    return r;
}
// MleEvalProofEF {eval_sumcheck, eq_at_s, w_at_s}
inline void put_eval(Ser& s, const EvalRec& e, bool with_challenges) {
    s.sumcheck(e.sc, with_challenges);
    s.ef(e.sc.fin);
    s.ef(e.sc.fin + 4);
}

// ---- matmul -------------------------------------------------------------------------------------
struct MatmulRec {
    ScRec sc;            // product sumcheck over w_partial x x
    size_t r_point = 0;  // log_m EF challenges
    u32 log_m = 0, log_n = 0;
    size_t root = 0;     // commitment of w_partial (interleaved coordinates)
    u32 n_pad = 0;
    EvalRec eval;
    int bind = 0;        // BIND_*; in the PCS modes `bf` holds the Basefold opening and `root` is unused
    BfPending bf;
};
// Weight-binding modes of bind_weights_ef (matmul.rs:360-453): the default build hashes
// w_partial with blake3; feature pcs commits to w_partial with Basefold; feature pcs-full commits
// to the row-padded matrix W itself.
enum BindMode : int { BIND_BLAKE3 = 0, BIND_PCS = 1, BIND_PCS_FULL = 2 };

// W: m x n row-major on device; x: n valid of n_pad (zero padded); y: m valid.
inline MatmulRec prove_matmul_succinct_ef(zkb_ctx* c, TrState* tr, const u32* W, const u32* x, const u32* y, u32 m, u32 n,
                                          int bind = BIND_BLAKE3, int node_kind = NODE_BLAKE3) {
    MatmulRec R;
    if (bind < BIND_BLAKE3 || bind > BIND_PCS_FULL) throw ArgFail{ZKB_E_ARG, "unknown weight-binding mode"};
    R.bind = bind;
    R.log_m = log2_ceil_u(m); R.log_n = log2_ceil_u(n);
    const size_t m_pad = size_t(1) << R.log_m, n_pad = size_t(1) << R.log_n;
    R.n_pad = (u32)n_pad;
    R.r_point = c->rec_alloc(4 * (size_t)R.log_m);
    u32* r_dev = c->rec_dev + R.r_point;
    {   // absorb_many(y_padded); r = squeeze_ef_many(log_m)     (matmul.rs:857-858)
        ScriptBuilder sb;
        sb.words_dev(y, m, (u32)m_pad);
        sb.squeeze(r_dev, 4 * R.log_m);
        sb.run(c, tr);
    }
    // eq table over the rows, then the one pass over W                     (matmul.rs:743-835)
    Fe* eq_r = (Fe*)c->scratch(m_pad * 16);
    eq_evals_kernel<Fe><<<grid_for(c, m_pad), 256, 0, c->stream>>>((const Fe*)r_dev, R.log_m, eq_r);
    ZKB_LAUNCHED(c);
    Fe* w_partial = (Fe*)c->scratch(n_pad * 16);
    {
        size_t rows_per = 0;
        dim3 grid = fold_launch_dims(c->sm_count, m, n, &rows_per);
        int rg = c->range_begin(ZKB_RANGE_FOLD_EQ_MATVEC, 4.0 * m * n);
        u32* slabs = (u32*)c->scratch((size_t)grid.y * n * 4 * 4 + 16);
        fold_eq_matvec_kernel<4, false><<<fold_grid(grid, c->sm_count, c->polite), FOLD_THREADS, 0, c->stream>>>(W, m, n, (const u32*)eq_r, rows_per, nullptr, slabs);
        c->range_end(rg);
        ZKB_LAUNCHED(c);
        fold_finalize_partials_kernel<4><<<grid_for(c, n_pad * 4), 256, 0, c->stream>>>(slabs, grid.y, n, n_pad, (u32*)w_partial);
        ZKB_LAUNCHED(c);
    }
    // product sumcheck, full messages                                     (matmul.rs:889-944)
    const u32* tabs[3] = {(const u32*)w_partial, x, nullptr};
    R.sc = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_EF_MIXED, tabs, R.log_n);
    if (bind == BIND_BLAKE3) {
        // default binding: blake3 of the interleaved coordinates, absorbed; then the EF MLE-eval
        R.root = commit_small(c, (const u32*)w_partial, (u32)(4 * n_pad), nullptr, (u32)(4 * n_pad), tr);
    } else {
        // Basefold at a base-field point squeezed from the transcript (matmul.rs:372-438), then the
        // 32-byte commitment root (16-byte Merkle root, zero-padded) is absorbed (matmul.rs:446)
        CoefSrc src = bind == BIND_PCS_FULL ? CoefSrc{W, m, n, R.log_n} : CoefSrc{(const u32*)w_partial, 1, (u32)(4 * n_pad), R.log_n + 2};
        const u32 bf_log = bind == BIND_PCS_FULL ? R.log_m + R.log_n : R.log_n + 2;
        const size_t num_coeffs = bind == BIND_PCS_FULL ? (size_t)m * n : 4 * n_pad;
        // codeword, trees and evaluation buffer (about 60 bytes per coefficient) are dead once the opening is
        // enqueued: everything the proof keeps goes to the record, so the next protocol step reuses the memory
        const auto mark = c->scratch_mark();
        u32* bf_point = (u32*)c->scratch((bf_log + 1) * 4);
        ScriptBuilder sb;
        sb.squeeze(bf_point, bf_log);
        sb.run(c, tr);
        R.bf = basefold_enqueue(c, tr, src, num_coeffs, bf_log, bf_point, bf_log, node_kind);
        sb.words_dev(c->rec_dev + R.bf.root_off, 4, 8);
        sb.run(c, tr);
        c->scratch_release(mark);
    }
    R.eval = prove_mle_eval_ef_ef(c, tr, w_partial, (const Fe*)(c->rec_dev + R.sc.chal), R.log_n);
    return R;
}
// SuccinctMatmulProofEF after strip_redundant (qwen.rs:745-750) when stripped = true.
inline void put_matmul(Ser& s, const MatmulRec& R, bool stripped) {
    // MatmulProofEF {sumcheck_proof, w_at_rs, x_at_s, r_point, s_point}
    s.sumcheck(R.sc, !stripped);
    s.ef(R.sc.fin); s.ef(R.sc.fin + 4);
    if (stripped) { s.u64le(0); s.u64le(0); }
    else {
        s.u64le(R.log_m); s.words(R.r_point, 4 * (size_t)R.log_m);
        s.u64le(R.log_n); s.words(R.sc.chal, 4 * (size_t)R.log_n);
    }
    put_eval(s, R.eval, !stripped);
    for (int i = 0; i < 4; i++) s.u32le(0);                 // w_claimed_value
    if (R.bind == BIND_BLAKE3) {
        s.commitment(R.root, 4 * (u64)R.n_pad);             // w_partial_commitment
        s.u8(0);                                            // bound
        s.u8(0);                                            // basefold_proof: None
    } else {
        // WeightCommitment {root = Merkle root || 16 zero bytes, num_weights, log_height, Blake3Fast} (matmul.rs:393-401)
        s.words(R.bf.root_off, 4);
        for (int i = 0; i < 4; i++) s.u32le(0);
        s.u64le(R.bf.num_coeffs);
        s.u64le(R.bf.log_n);
        s.u32le(0);
        s.u8(0);                                            // bound
        s.u8(1);                                            // basefold_proof: Some
        put_basefold_proof(s, s.rec, R.bf);
    }
}

// ---- base-field twins: matmul with base-field challenges (MLP / GPT-2 op lists) --------------------
// prove_mle_eval_no_merkle (weight_commitment.rs:177-206): eq table at a base-field point, the
// full-message product sumcheck of (eq, w), then the 24 discarded query squeezes.  w: 2^k values
// on device (already zero-padded); point: k base-field challenges on device.
inline EvalRec prove_mle_eval_base(zkb_ctx* c, TrState* tr, const u32* w, const u32* point, u32 k, const char* label = nullptr,
                                   const u32* root_dev = nullptr) {
    if (label) {                       // prove_mle_eval_bound (weight_commitment.rs:437-447)
        ScriptBuilder sb;
        sb.str(label);
        sb.words_dev(root_dev, 8);
        sb.run(c, tr);
    }
    size_t n = size_t(1) << k;
    Fp* eq = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)point, k, eq);
    ZKB_LAUNCHED(c);
    const u32* tabs[3] = {(const u32*)eq, w, nullptr};
    ScOpts o;
    o.post_squeezes = 24;
    EvalRec r;
    r.sc = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tabs, k, o);
    return r;
}
// MleEvalProof {eval_sumcheck, eq_at_s, w_at_s, merkle_opening: None} (weight_commitment.rs:65-73)
inline void put_eval_base(Ser& s, const EvalRec& e) {
    s.sumcheck(e.sc, true);
    s.words(e.sc.fin, 1);
    s.words(e.sc.fin + 1, 1);
    s.u8(0);
}
// prove_matmul_succinct (matmul.rs:482-511) over prove_matmul (matmul.rs:134-180) with the
// default weight binding (matmul.rs:346-355).
inline MatmulRec prove_matmul_succinct_base(zkb_ctx* c, TrState* tr, const u32* W, const u32* x, const u32* y, u32 m, u32 n) {
    MatmulRec R;
    R.log_m = log2_ceil_u(m); R.log_n = log2_ceil_u(n);
    const size_t m_pad = size_t(1) << R.log_m, n_pad = size_t(1) << R.log_n;
    R.n_pad = (u32)n_pad;
    R.r_point = c->rec_alloc(R.log_m);
    u32* r_dev = c->rec_dev + R.r_point;
    {
        ScriptBuilder sb;
        sb.words_dev(y, m, (u32)m_pad);
        sb.squeeze(r_dev, R.log_m);
        sb.run(c, tr);
    }
    Fp* eq_r = (Fp*)c->scratch(m_pad * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, m_pad), 256, 0, c->stream>>>((const Fp*)r_dev, R.log_m, eq_r);
    ZKB_LAUNCHED(c);
    u32* w_partial = (u32*)c->scratch(n_pad * 4 + 16);
    {
        size_t rows_per = 0;
        dim3 grid = fold_launch_dims(c->sm_count, m, n, &rows_per);
        int rg = c->range_begin(ZKB_RANGE_FOLD_EQ_MATVEC, 4.0 * m * n);
        u32* slabs = (u32*)c->scratch((size_t)grid.y * n * 4 + 16);
        fold_eq_matvec_kernel<1, false><<<fold_grid(grid, c->sm_count, c->polite), FOLD_THREADS, 0, c->stream>>>(W, m, n, (const u32*)eq_r, rows_per, nullptr, slabs);
        c->range_end(rg);
        ZKB_LAUNCHED(c);
        fold_finalize_partials_kernel<1><<<grid_for(c, n_pad), 256, 0, c->stream>>>(slabs, grid.y, n, n_pad, w_partial);
        ZKB_LAUNCHED(c);
    }
    const u32* tabs[3] = {w_partial, x, nullptr};
    R.sc = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tabs, R.log_n);
    R.root = commit_small(c, w_partial, (u32)n_pad, nullptr, (u32)n_pad, tr);
    R.eval = prove_mle_eval_base(c, tr, w_partial, c->rec_dev + R.sc.chal, R.log_n);
    return R;
}
// SuccinctMatmulProof (matmul.rs:458-474)
inline void put_matmul_base(Ser& s, const MatmulRec& R) {
    s.sumcheck(R.sc, true);
    s.words(R.sc.fin, 1); s.words(R.sc.fin + 1, 1);
    s.u64le(R.log_m); s.words(R.r_point, R.log_m);
    s.u64le(R.log_n); s.words(R.sc.chal, R.log_n);
    put_eval_base(s, R.eval);
    s.u32le(0);                                             // w_claimed_value
    s.commitment(R.root, (u64)R.n_pad);
    s.u8(0);                                                // bound
    s.u8(0);                                                // basefold_proof: None
}

// ---- hadamard / add -------------------------------------------------------------------------------
struct HadamardRec { ScRec sc; size_t root = 0; EvalRec eval; u32 k = 0; };
// a, b, c: base vectors with `len` valid entries, c zero-padded to 2^k on device; point: k EF on device.
inline HadamardRec prove_hadamard_ef(zkb_ctx* c, TrState* tr, const u32* a, const u32* b, const u32* cvec, u32 len, const Fe* point, u32 k) {
    HadamardRec R;
    R.k = k;
    size_t n = size_t(1) << k;
    R.root = commit_small(c, cvec, (u32)n, nullptr, (u32)n, tr);
    Fe* eq = (Fe*)c->scratch(n * 16);
    Fe* aef = (Fe*)c->scratch(n * 16);
    Fe* bef = (Fe*)c->scratch(n * 16);
    WidenEqArgs w{};
    w.src[0] = a; w.dst[0] = aef; w.len[0] = len; w.src[1] = b; w.dst[1] = bef; w.len[1] = len; w.nsrc = 2;
    w.point = point; w.eq_out = eq; w.k = k;
    widen_eq_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(w);
    ZKB_LAUNCHED(c);
    const u32* tabs[3] = {(const u32*)eq, (const u32*)aef, (const u32*)bef};
    ScOpts o;
    o.clobber[0] = o.clobber[1] = o.clobber[2] = true;
    R.sc = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE_EF_FULL, tabs, k, o);
    R.eval = prove_mle_eval_ef_base(c, tr, cvec, (u32)n, point, k, "hadamard-c-eval-ef", c->rec_dev + R.root);
    return R;
}
// HadamardProofEF {product_sumcheck, product_finals(3), c_eval, c_eval_proof, c_commitment}
inline void put_hadamard(Ser& s, const HadamardRec& R, bool stripped) {
    s.sumcheck(R.sc, !stripped);
    s.ef(R.sc.fin); s.ef(R.sc.fin + 4); s.ef(R.sc.fin + 8);
    s.claimed_sum_ef(R.eval.sc);      // c_eval = MLE of c at the point = sum eq . c = s0 + s1 of the eval sumcheck
    put_eval(s, R.eval, true);
    s.commitment(R.root, u64(1) << R.k);
}

struct AddRec { ScRec sa, sb; size_t root = 0; EvalRec eval; u32 k = 0; };
inline AddRec prove_add_ef(zkb_ctx* c, TrState* tr, const u32* a, const u32* b, const u32* cvec, u32 len, const Fe* point, u32 k) {
    AddRec R;
    R.k = k;
    size_t n = size_t(1) << k;
    R.root = commit_small(c, cvec, (u32)n, nullptr, (u32)n, tr);
    Fe* eq = (Fe*)c->scratch(n * 16);
    Fe* aef = (Fe*)c->scratch(n * 16);
    Fe* bef = (Fe*)c->scratch(n * 16);
    WidenEqArgs w{};
    w.src[0] = a; w.dst[0] = aef; w.len[0] = len; w.src[1] = b; w.dst[1] = bef; w.len[1] = len; w.nsrc = 2;
    w.point = point; w.eq_out = eq; w.k = k;
    widen_eq_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(w);
    ZKB_LAUNCHED(c);
    const u32* ta[3] = {(const u32*)eq, (const u32*)aef, nullptr};
    ScOpts oa;
    oa.clobber[1] = true;             // eq is needed again by the second sumcheck
    R.sa = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_EF_FULL, ta, k, oa);
    const u32* tb[3] = {(const u32*)eq, (const u32*)bef, nullptr};
    ScOpts ob;
    ob.clobber[0] = ob.clobber[1] = true;
    R.sb = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT_EF_FULL, tb, k, ob);
    R.eval = prove_mle_eval_ef_base(c, tr, cvec, (u32)n, point, k, "add-c-eval-ef", c->rec_dev + R.root);
    return R;
}
// AddProofEF {a_sumcheck, a_finals(2), b_sumcheck, b_finals(2), c_eval, c_eval_proof, c_commitment}
inline void put_add(Ser& s, const AddRec& R, bool stripped) {
    s.sumcheck(R.sa, !stripped); s.ef(R.sa.fin); s.ef(R.sa.fin + 4);
    s.sumcheck(R.sb, !stripped); s.ef(R.sb.fin); s.ef(R.sb.fin + 4);
    s.claimed_sum_ef(R.eval.sc);
    put_eval(s, R.eval, true);
    s.commitment(R.root, u64(1) << R.k);
}

// ---- base-field twins of hadamard / add (elementwise.rs:50-98, 189-235) ---------------------------
// a, b, cvec: device vectors zero-padded to 2^k; point: k base-field challenges on device.
inline HadamardRec prove_hadamard_base(zkb_ctx* c, TrState* tr, const u32* a, const u32* b, const u32* cvec, const u32* point, u32 k) {
    HadamardRec R;
    R.k = k;
    size_t n = size_t(1) << k;
    R.root = commit_small(c, cvec, (u32)n, nullptr, (u32)n, tr);
    Fp* eq = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)point, k, eq);
    ZKB_LAUNCHED(c);
    const u32* tabs[3] = {(const u32*)eq, a, b};
    R.sc = sumcheck_enqueue(c, tr, ZKB_SC_TRIPLE, tabs, k);
    R.eval = prove_mle_eval_base(c, tr, cvec, point, k, "hadamard-c-eval", c->rec_dev + R.root);
    return R;
}
// c_eval = MLE of c at the point = s0 + s1 of round 0 of the eval sumcheck (sum of eq . c)
inline void put_claimed_sum_base(Ser& s, const ScRec& r) { s.u32le(add31(s.rec[r.polys], s.rec[r.polys + 1])); }
// HadamardProof {product_sumcheck, product_finals(3), c_eval, c_eval_proof, c_commitment} (elementwise.rs:31-44)
inline void put_hadamard_base(Ser& s, const HadamardRec& R) {
    s.sumcheck(R.sc, true);
    s.words(R.sc.fin, 3);
    put_claimed_sum_base(s, R.eval.sc);
    put_eval_base(s, R.eval);
    s.commitment(R.root, u64(1) << R.k);
}
inline AddRec prove_add_base(zkb_ctx* c, TrState* tr, const u32* a, const u32* b, const u32* cvec, const u32* point, u32 k) {
    AddRec R;
    R.k = k;
    size_t n = size_t(1) << k;
    R.root = commit_small(c, cvec, (u32)n, nullptr, (u32)n, tr);
    Fp* eq = (Fp*)c->scratch(n * 4 + 16);
    eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)point, k, eq);
    ZKB_LAUNCHED(c);
    const u32* ta[3] = {(const u32*)eq, a, nullptr};
    R.sa = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, ta, k);
    const u32* tb[3] = {(const u32*)eq, b, nullptr};
    R.sb = sumcheck_enqueue(c, tr, ZKB_SC_PRODUCT, tb, k);
    R.eval = prove_mle_eval_base(c, tr, cvec, point, k, "add-c-eval", c->rec_dev + R.root);
    return R;
}
// AddProof (elementwise.rs:165-181)
inline void put_add_base(Ser& s, const AddRec& R) {
    s.sumcheck(R.sa, true); s.words(R.sa.fin, 2);
    s.sumcheck(R.sb, true); s.words(R.sb.fin, 2);
    put_claimed_sum_base(s, R.eval.sc);
    put_eval_base(s, R.eval);
    s.commitment(R.root, u64(1) << R.k);
}

}  // namespace zkb
