// C ABI, part 9: batch Basefold - k polynomials of possibly different sizes opened with one fold chain
// (rust/zk_ml_prover/src/proving/basefold.rs:769-1590).  Included by zkb200.cu.
//
//   zkb_basefold_batch_precommit   batch_precommit_multi_height (:1183-1216): encodings and trees, transcript-independent,
//                                  kept in device memory for the life of the object (the reference's "load time" half)
//   zkb_basefold_batch_prove       batch_prove_with_precommit (:1221-1378); with individual openings and equal sizes it is
//                                  batch_commit_and_prove (:801-956)
//
// Every fold challenge is squeezed before the first fold (:1284), so once the batched root has been absorbed the folds,
// the additions of the smaller codewords and the trees of all rounds run ahead on the context's second stream while its
// main stream runs the hash chain (per round: root absorb, 24 query squeezes) and gathers the paths behind them.

namespace zkb {

__global__ void bfb_coeffs_kernel(const u32* __restrict__ rho, u32 k, u32* coef) {        // [1, rho, rho^2, ...] (:1239-1242)
    for (u32 i = blockIdx.x * blockDim.x + threadIdx.x; i < k; i += gridDim.x * blockDim.x) coef[i] = pow31(rho[0], i);
}
// out[j] = sum_{i in [first, first + count)} coef[i] * cws[i][j], j < len.  Codewords and out are cudaMalloc'd and len is a power of
// two >= 4 (a codeword has 2 * 2^log_n >= 4 words), so every thread moves 16-byte vectors; the codewords are read once (evict first).
__global__ void __launch_bounds__(256) bfb_lincomb_kernel(const u32* const* __restrict__ cws, const u32* __restrict__ coef, u32 first, u32 count,
                                                          size_t len, u32* __restrict__ out) {
    const size_t n4 = len >> 2;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n4; j += (size_t)gridDim.x * blockDim.x) {
        u64 a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        for (u32 i = first; i < first + count; i++) {
            const u32 c = coef[i];
            const uint4 v = __ldcs(reinterpret_cast<const uint4*>(cws[i]) + j);
            a0 += (u64)mul31(c, v.x); a1 += (u64)mul31(c, v.y); a2 += (u64)mul31(c, v.z); a3 += (u64)mul31(c, v.w);
        }
        reinterpret_cast<uint4*>(out)[j] = make_uint4(red64(a0), red64(a1), red64(a2), red64(a3));
    }
}
// Absorb the batched root, squeeze the whole fold point, absorb its first coordinate (:1277-1291).
__global__ void bfb_begin_kernel(TrState* st, const uint4* root, u32 log_n, u32* fold_point, u32* rec_root) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    Tr tr;
    tr_load(tr, st, trbuf);
    uint4 r = *root;
    u32 rw[4] = {r.x, r.y, r.z, r.w};
    tr_absorb_words<4>(tr, rw);
    rec_root[0] = r.x; rec_root[1] = r.y; rec_root[2] = r.z; rec_root[3] = r.w;
    for (u32 b = 0; b < log_n; b++) fold_point[b] = tr_squeeze(tr);
    tr_absorb_u32(tr, fold_point[0]);
    tr_store(tr, st);
}
// derive_query_indices(transcript, max_log_n + 1) after the last round (:1366), reduced mod 2^max_log_n as the
// individual openings use them (:917-923).
__global__ void bfb_final_kernel(TrState* st, u32 mask, u32* idx) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    Tr tr;
    tr_load(tr, st, trbuf);
    for (u32 q = 0; q < BF_QUERIES; q++) idx[q] = tr_squeeze(tr) & mask;
    tr_store(tr, st);
}
// 48 raw paths of an individual tree: positions (idx[q] mod tree_half) and that + tree_half (:1330-1340, :917-927).
__global__ void __launch_bounds__(256) bfb_open_kernel(const u32* __restrict__ values, const uint4* __restrict__ nodes, u32 h, const u32* __restrict__ idx,
                                                       u32 tree_half, u32* out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const size_t pw = 2 + 4 * (size_t)(h - 1);
    for (u32 item = warp; item < 2 * BF_QUERIES; item += nwarps) {
        const size_t pos = (size_t)(idx[item >> 1] & (tree_half - 1)) + ((item & 1) ? tree_half : 0);
        mk_gather_path(values, size_t(1) << h, nodes, h, pos, out + item * pw, lane, 32);
    }
}
__global__ void bfb_final_value_kernel(const u32* __restrict__ coef, const u32* __restrict__ evals, u32 k, u32* out) {
    u32 acc = 0;
    for (u32 i = 0; i < k; i++) acc = add31(acc, mul31(coef[i], evals[i]));
    *out = acc;
}

}  // namespace zkb

struct zkb_bf_batch {
    zkb_ctx* ctx = nullptr;
    int kind = 0;
    zkb::u32 max_log_n = 0;
    struct Entry {
        const zkb::u32* coeffs; size_t n; zkb::u32 log_n; size_t orig;
        zkb::u32* cw; uint4* tree; zkb::u32 root[4];
    };
    std::vector<Entry> e;                     // by log_n descending, ties in input order
    std::vector<void*> owned;
    const zkb::u32** cw_ptrs_dev = nullptr;
};

namespace {

struct BfbPending {
    size_t batched_root_off = 0, final_off = 0, final_idx_off = 0;
    std::vector<size_t> round_off;
    struct Open { zkb::u32 round; zkb::u32 poly; size_t off; };
    std::vector<Open> add_opens, final_opens;
};

BfbPending bfb_enqueue(zkb_bf_batch* B, TrState* tr, bool individual) {
    zkb_ctx* c = B->ctx;
    const u32 k = (u32)B->e.size(), log_n = B->max_log_n;
    const int kind = B->kind;
    BfTables tb = bf_tables(c, log_n);
    BfbPending pd;
    // roots in sorted order, then rho (:1233-1239)
    u32* rho = (u32*)c->scratch(16);
    u32* coef = (u32*)c->scratch((size_t)k * 4 + 16);
    {
        ScriptBuilder sb;
        for (u32 i = 0; i < k; i++) {
            sb.bytes(B->e[i].root, 16);
            if (sb.s.nops + 2 >= TRSCRIPT_MAX_OPS || sb.inl_used + 32 > TRSCRIPT_INLINE) sb.run(c, tr);
        }
        sb.squeeze(rho, 1);
        sb.run(c, tr);
    }
    bfb_coeffs_kernel<<<grid_for(c, k), 256, 0, c->stream>>>(rho, k, coef);
    ZKB_LAUNCHED(c);
    // groups of equal size
    struct Group { u32 log_n, s, e; };
    std::vector<Group> groups;
    for (u32 gs = 0; gs < k;) {
        u32 ge = gs + 1;
        while (ge < k && B->e[ge].log_n == B->e[gs].log_n) ge++;
        groups.push_back(Group{B->e[gs].log_n, gs, ge});
        gs = ge;
    }
    const size_t cw_len0 = size_t(2) << log_n;
    u32* cw0 = (u32*)c->scratch(cw_len0 * 4);
    uint4* tree0 = (uint4*)c->scratch(mk_node_count(log_n + 1) * 16 + 16);
    bfb_lincomb_kernel<<<grid_for(c, cw_len0 / 4), 256, 0, c->stream>>>(B->cw_ptrs_dev, coef, groups[0].s, groups[0].e - groups[0].s, cw_len0, cw0);
    ZKB_LAUNCHED(c);
    MkFold none{};
    mk_build(c, kind, MK_VALUES, cw0, cw_len0, log_n + 1, tree0, none);
    u32* fold_point = (u32*)c->scratch(((size_t)log_n + 1) * 4);
    pd.batched_root_off = c->rec_alloc(4);
    bfb_begin_kernel<<<1, 1, 0, c->stream>>>(tr, tree0 + mk_layer_offset(log_n + 1, log_n + 1), log_n, fold_point, c->rec_dev + pd.batched_root_off);
    ZKB_LAUNCHED(c);

    const bool in_order = c->opt_bf_in_order || c->capturing;
    cudaStream_t main_stream = c->stream, work = in_order ? main_stream : c->side_stream();
    if (!in_order) {
        cudaEvent_t fork = c->side_event(log_n);
        ZKB_CUDA(cudaEventRecord(fork, main_stream));
        ZKB_CUDA(cudaStreamWaitEvent(work, fork, 0));
    }
    // final value: sum_i rho^i MLE_i(fold_point[..log_n_i]) (:1357-1362).  It needs only the fold point, so it goes in front of the rounds on
    // the main stream, where it runs while the second stream folds and hashes the first (largest) rounds.
    u32* evals = (u32*)c->scratch((size_t)k * 4 + 16);
    for (u32 i = 0; i < k; i++)
        mle_eval_enqueue<Fp, Fp>(c, (const Fp*)B->e[i].coeffs, B->e[i].n, (const Fp*)fold_point, B->e[i].log_n, (Fp*)(evals + i));
    pd.final_off = c->rec_alloc(1);
    bfb_final_value_kernel<<<1, 1, 0, c->stream>>>(coef, evals, k, c->rec_dev + pd.final_off);
    ZKB_LAUNCHED(c);
    u32* prev_cw = cw0;
    uint4* prev_tree = tree0;
    size_t next_group = 1;
    for (u32 round = 0; round < log_n; round++) {
        const u32 h_prev = log_n + 1 - round;
        const size_t half = size_t(1) << (h_prev - 1);           // length of the folded codeword
        const u32 fold_level = log_n - 1 - round, target = log_n - 1 - round;
        u32* next_cw = (u32*)c->scratch(half * 4 + 16);
        uint4* next_tree = (uint4*)c->scratch(mk_node_count(h_prev - 1) * 16 + 16);
        MkFold f{};
        f.prev = prev_cw; f.out = next_cw;
        f.weights = tb.w_flat + ((size_t(1) << fold_level) - 1);
        f.w_len = size_t(1) << fold_level;
        f.alpha = fold_point + round;
        c->stream = work;
        try {
            // codewords that reach their own length at this round join the chain (:1304-1314); a codeword of 2 * 2^target values
            // is exactly as long as the folded one
            u32 first = 0, count = 0;
            while (next_group < groups.size() && groups[next_group].log_n == target) {
                if (!count) first = groups[next_group].s;
                count += groups[next_group].e - groups[next_group].s;
                next_group++;
            }
            if (count) {
                u32* add = (u32*)c->scratch(half * 4 + 16);
                bfb_lincomb_kernel<<<grid_for(c, half / 4 ? half / 4 : 1), 256, 0, c->stream>>>(B->cw_ptrs_dev, coef, first, count, half, add);
                ZKB_LAUNCHED(c);
                f.add = add;
            }
            mk_build(c, kind, MK_FOLD, nullptr, half, h_prev - 1, next_tree, f);
            c->stream = main_stream;
            if (!in_order) {
                ZKB_CUDA(cudaEventRecord(c->side_event(round), work));
                ZKB_CUDA(cudaStreamWaitEvent(main_stream, c->side_event(round), 0));
            }
            BfRound rp{};
            rp.tr = tr; rp.point = fold_point; rp.n_point = log_n; rp.round = round; rp.log_n = log_n;
            rp.alpha_next = round + 1 < log_n ? fold_point + log_n : nullptr;    // the value is already in fold_point; the slot behind it takes the copy
            rp.prev_values = prev_cw; rp.prev_nodes = prev_tree; rp.fold_values = next_cw; rp.fold_nodes = next_tree;
            rp.h_prev = h_prev;
            const size_t off = c->rec_alloc(bf_round_words(h_prev));
            rp.rec = c->rec_dev + off;
            pd.round_off.push_back(off);
            bf_round_kernel<<<1, 256, exclusive_smem(bf_round_kernel, c), c->stream>>>(rp);
            ZKB_LAUNCHED(c);
            // the joined polynomials' own trees, opened at this round's positions (:1330-1345)
            for (u32 i = first; i < first + count; i++) {
                const u32 h = B->e[i].log_n + 1;
                const size_t o = c->rec_alloc(2 * (size_t)BF_QUERIES * (2 + 4 * (size_t)(h - 1)));
                bfb_open_kernel<<<1, 256, 0, c->stream>>>(B->e[i].cw, B->e[i].tree, h, c->rec_dev + off + 4, u32(1) << B->e[i].log_n, c->rec_dev + o);
                ZKB_LAUNCHED(c);
                pd.add_opens.push_back(BfbPending::Open{round, i, o});
            }
        } catch (...) { c->stream = main_stream; throw; }
        prev_cw = next_cw; prev_tree = next_tree;
    }
    pd.final_idx_off = c->rec_alloc(BF_QUERIES);
    bfb_final_kernel<<<1, 1, 0, c->stream>>>(tr, (u32(1) << log_n) - 1, c->rec_dev + pd.final_idx_off);
    ZKB_LAUNCHED(c);
    if (individual) {
        for (u32 i = 0; i < k; i++) {
            const u32 h = log_n + 1;
            const size_t o = c->rec_alloc(2 * (size_t)BF_QUERIES * (2 + 4 * (size_t)(h - 1)));
            bfb_open_kernel<<<1, 256, 0, c->stream>>>(B->e[i].cw, B->e[i].tree, h, c->rec_dev + pd.final_idx_off, u32(1) << log_n, c->rec_dev + o);
            ZKB_LAUNCHED(c);
            pd.final_opens.push_back(BfbPending::Open{0, i, o});
        }
    }
    return pd;
}

// 48 opened positions of an individual tree as a BatchMerkleProof
void bfb_put_open(Ser& s, const u32* rec_host, const u32* idx, size_t off, u32 tree_half, u32 h) {
    const size_t pw = 2 + 4 * (size_t)(h - 1);
    std::vector<size_t> pos;
    std::vector<const u32*> raw;
    for (u32 q = 0; q < BF_QUERIES; q++) {
        const size_t li = idx[q] & (tree_half - 1);
        pos.push_back(li); raw.push_back(rec_host + off + (2 * q) * pw);
        pos.push_back(li + tree_half); raw.push_back(rec_host + off + (2 * q + 1) * pw);
    }
    put_batch_proof(s, pos, raw, h);
}

}  // namespace

extern "C" {

int32_t zkb_basefold_batch_precommit(zkb_ctx* c, const uint32_t* const* coeffs, const size_t* n_coeffs, const uint32_t* log_ns, size_t k,
                                     int32_t on_device, int32_t node_hash, zkb_bf_batch** out) {
    if (!c || !coeffs || !n_coeffs || !log_ns || !out || k == 0 || k > 4096) return ZKB_E_ARG;
    *out = nullptr;
    zkb_bf_batch* B = new (std::nothrow) zkb_bf_batch();
    if (!B) return ZKB_E_CUDA;
    B->ctx = c;
    auto body = [&]() -> int32_t {
        ZKB_TRY(c, {
            c->use();
            if (node_hash != NODE_BLAKE3 && node_hash != NODE_AES_MMO) throw ArgFail{ZKB_E_ARG, "unknown node hash"};
            if (node_hash == NODE_AES_MMO) aes_tables_upload();
            B->kind = node_hash;
            std::vector<size_t> order(k);
            for (size_t i = 0; i < k; i++) {
                order[i] = i;
                if (!coeffs[i] && n_coeffs[i]) throw ArgFail{ZKB_E_ARG, "batch basefold: null polynomial"};
                if (log_ns[i] < 1 || log_ns[i] > 28) throw ArgFail{ZKB_E_TOO_LARGE, "basefold: log_n out of range"};
                if (n_coeffs[i] > (size_t(1) << log_ns[i])) throw ArgFail{ZKB_E_LENGTH, "batch basefold: more coefficients than 2^log_n"};
            }
            std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return log_ns[a] > log_ns[b]; });
            B->max_log_n = log_ns[order[0]];
            BfTables tb = bf_tables(c, B->max_log_n);      // every polynomial is encoded with the largest one's tables (:1191-1199)
            std::vector<const u32*> ptrs;
            for (size_t idx : order) {
                zkb_bf_batch::Entry e{};
                e.n = n_coeffs[idx]; e.log_n = log_ns[idx]; e.orig = idx;
                const size_t n_pad = size_t(1) << e.log_n;
                if (on_device) e.coeffs = coeffs[idx];
                else {
                    u32* d = nullptr;
                    ZKB_CUDA(cudaMalloc(&d, (e.n ? e.n : 1) * 4));
                    B->owned.push_back(d);
                    if (e.n) ZKB_CUDA(cudaMemcpyAsync(d, coeffs[idx], e.n * 4, cudaMemcpyHostToDevice, c->stream));
                    e.coeffs = d;
                }
                ZKB_CUDA(cudaMalloc(&e.cw, 2 * n_pad * 4));
                B->owned.push_back(e.cw);
                ZKB_CUDA(cudaMalloc(&e.tree, mk_node_count(e.log_n + 1) * 16 + 16));
                B->owned.push_back(e.tree);
                bf_encode(c, CoefSrc{e.coeffs, 1, (u32)e.n, e.log_n}, e.log_n, tb, e.cw);
                MkFold none{};
                mk_build(c, node_hash, MK_VALUES, e.cw, 2 * n_pad, e.log_n + 1, e.tree, none);
                ZKB_CUDA(cudaMemcpyAsync(e.root, e.tree + mk_layer_offset(e.log_n + 1, e.log_n + 1), 16, cudaMemcpyDeviceToHost, c->stream));
                B->e.push_back(e);
                ptrs.push_back(e.cw);
            }
            void* pd = nullptr;
            ZKB_CUDA(cudaMalloc(&pd, k * sizeof(u32*)));
            B->owned.push_back(pd);
            B->cw_ptrs_dev = (const u32**)pd;
            ZKB_CUDA(cudaMemcpyAsync(pd, ptrs.data(), k * sizeof(u32*), cudaMemcpyHostToDevice, c->stream));
            ZKB_CUDA(cudaStreamSynchronize(c->stream));
            ZKB_CUDA(cudaGetLastError());
        });
    };
    int32_t rc = body();
    if (rc != ZKB_OK) {
        cudaStreamSynchronize(c->stream);
        for (void* p : B->owned) cudaFree(p);
        delete B;
        return rc;
    }
    *out = B;
    return ZKB_OK;
}

void zkb_basefold_batch_destroy(zkb_bf_batch* B) {
    if (!B) return;
    if (B->ctx) { cudaSetDevice(B->ctx->device); cudaStreamSynchronize(B->ctx->stream); }
    for (void* p : B->owned) cudaFree(p);
    delete B;
}

size_t zkb_basefold_batch_count(const zkb_bf_batch* B) { return B ? B->e.size() : 0; }
uint64_t zkb_basefold_batch_device_bytes(const zkb_bf_batch* B) {
    uint64_t t = 0;
    if (B) for (auto& e : B->e) t += (uint64_t(8) << e.log_n) + (mk_node_count(e.log_n + 1) * 16 + 16);
    return t;
}

int32_t zkb_basefold_batch_commitment(const zkb_bf_batch* B, size_t index, uint8_t root[16], uint64_t* num_coeffs, uint64_t* log_n) {
    if (!B || !root) return ZKB_E_ARG;
    for (auto& e : B->e) if (e.orig == index) {
        memcpy(root, e.root, 16);
        if (num_coeffs) *num_coeffs = e.n;
        if (log_n) *log_n = e.log_n;
        return ZKB_OK;
    }
    return ZKB_E_ARG;
}

int32_t zkb_basefold_batch_prove(zkb_bf_batch* B, zkb_transcript* t, int32_t individual_openings, uint8_t* out, size_t cap, size_t* len) {
    if (!B || !t || !len) return ZKB_E_ARG;
    zkb_ctx* c = B->ctx;
    ZKB_TRY(c, {
        c->use();
        const u32 k = (u32)B->e.size(), log_n = B->max_log_n;
        if (individual_openings) for (auto& e : B->e) if (e.log_n != log_n)
            throw ArgFail{ZKB_E_ARG, "batch basefold: individual openings are defined for polynomials of one size (batch_commit_and_prove)"};
        c->rec_reset();
        BfbPending pd = bfb_enqueue(B, t->dev, individual_openings != 0);
        ZKB_CUDA(cudaGetLastError());
        c->rec_fetch();
        const u32* rec = c->rec_host;
        Ser s;
        s.rec = rec;
        // Vec<BasefoldCommitment>, input order (basefold.rs:39-47)
        s.u64le(k);
        for (size_t i = 0; i < k; i++) for (auto& e : B->e) if (e.orig == i) { put_digest(s, e.root); s.u64le(e.n); s.u64le(e.log_n); }
        // BasefoldBatchProof (basefold.rs:769-795)
        s.u64le(k);
        s.u64le(k); for (auto& e : B->e) s.u64le(e.log_n);
        s.u64le(k); for (auto& e : B->e) put_digest(s, e.root);
        put_digest(s, rec + pd.batched_root_off);
        s.u64le(log_n);
        for (u32 r = 0; r < log_n; r++) put_digest(s, rec + pd.round_off[r]);
        s.u64le(log_n);
        for (u32 r = 0; r < log_n; r++) {
            const u32 h_prev = log_n + 1 - r, h_fold = h_prev - 1;
            const u32* rr = rec + pd.round_off[r];
            const u32* idx = rr + 4;
            const size_t prev_half = size_t(1) << (h_prev - 1);
            const size_t pw_prev = 2 + 4 * (size_t)(h_prev - 1), pw_fold = h_fold >= 1 ? 2 + 4 * (size_t)(h_fold - 1) : 2;
            const u32* out_prev = rr + 4 + BF_QUERIES;
            const u32* out_fold = out_prev + 2 * BF_QUERIES * pw_prev;
            std::vector<size_t> pp, fp;
            std::vector<const u32*> pr, fr;
            for (u32 q = 0; q < BF_QUERIES; q++) {
                pp.push_back(idx[q]); pr.push_back(out_prev + (2 * q) * pw_prev);
                pp.push_back(idx[q] + prev_half); pr.push_back(out_prev + (2 * q + 1) * pw_prev);
                fp.push_back(idx[q]); fr.push_back(out_fold + q * pw_fold);
            }
            put_batch_proof(s, pp, pr, h_prev);
            put_batch_proof(s, fp, fr, h_fold);
        }
        s.u64le(pd.final_opens.size());
        for (auto& o : pd.final_opens) bfb_put_open(s, rec, rec + pd.final_idx_off, o.off, u32(1) << log_n, log_n + 1);
        s.u32le(rec[pd.final_off]);
        // add_round_openings: (round, [(poly index in sorted order, opening)]) for every round at which codewords joined
        size_t n_rounds = 0;
        for (size_t i = 0; i < pd.add_opens.size(); i++) if (i == 0 || pd.add_opens[i].round != pd.add_opens[i - 1].round) n_rounds++;
        s.u64le(n_rounds);
        for (size_t i = 0; i < pd.add_opens.size();) {
            size_t j = i;
            while (j < pd.add_opens.size() && pd.add_opens[j].round == pd.add_opens[i].round) j++;
            s.u64le(pd.add_opens[i].round);
            s.u64le(j - i);
            for (size_t a = i; a < j; a++) {
                const auto& o = pd.add_opens[a];
                s.u64le(o.poly);
                bfb_put_open(s, rec, rec + pd.round_off[o.round] + 4, o.off, u32(1) << B->e[o.poly].log_n, B->e[o.poly].log_n + 1);
            }
            i = j;
        }
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

// batch_verify_opening (basefold.rs:959-1137) on the bytes zkb_basefold_batch_prove returns.  The transcript ends where the prover's does.
int32_t zkb_basefold_batch_verify_opening(zkb_ctx* c, zkb_transcript* tr, const uint8_t* bytes, size_t len, int32_t node_hash, int32_t* accepted) {
    if (!c || !tr || !bytes || !accepted) return ZKB_E_ARG;
    *accepted = 0;
    ZKB_TRY(c, {
        c->use();
        BbvParsed pr;
        if (!bbv_parse(bytes, len, pr)) throw ArgFail{ZKB_E_ARG, "batch basefold: the bytes do not decode as commitments followed by a batch proof"};
        if (pr.too_large) throw ArgFail{ZKB_E_TOO_LARGE, "basefold: more than 256 opened positions in one batch proof"};
        if (pr.trivially_true) { *accepted = 1; return ZKB_OK; }
        if (pr.reject) return ZKB_OK;                             // decided from the shape, before the transcript is touched
        BvRun run = basefold_batch_verify_enqueue(c, tr->dev, pr, node_hash);
        std::vector<u32> res(run.n_results);
        ZKB_CUDA(cudaMemcpyAsync(res.data(), run.result_dev, (size_t)run.n_results * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
        bool ok = true;
        for (u32 v : res) ok = ok && v == 1;
        *accepted = ok ? 1 : 0;
    });
}

}  // extern "C"
