// Batch Basefold verifier (rust/zk_ml_prover/src/proving/basefold.rs:959-1137) on the bytes the batch prover emits:
// bincode(Vec<BasefoldCommitment>) || bincode(BasefoldBatchProof).
//
// The host decodes the bytes into the flat word array and the per-tree descriptors of verify.cuh; the Merkle checks of all
// trees (two per round, the joined polynomials' trees, the individual openings) are one launch of bf_verify_batch_kernel on the
// second stream, the transcript (roots, rho, batched root, fold point, per round alpha / root / 24 queries, the last 24 queries)
// one thread on the main stream, and the fold relation with the joined polynomials' contributions one warp per (round, query).
// Like the reference's verifier it reads neither the final value nor the commitments' num_coeffs.
#pragma once
#include "verify.cuh"

namespace zkb {

struct BbvAdd { u32 tree, poly, log_n, pad; };          // an opening that joins at a round: its descriptor, its index in size order

struct BbvParsed {
    std::vector<u32> words;
    std::vector<BvTree> trees;                            // [2 per round][add openings][individual openings]
    std::vector<BbvAdd> adds;                             // grouped by round through add_first / add_count
    std::vector<u32> add_first, add_count;                // per round
    u32 k = 0, log_n = 0, roots_off = 0, batched_off = 0, fold_off = 0;
    bool reject = false, too_large = false, trivially_true = false;
};

// One BatchMerkleProof (pcs.rs:43-53) appended to words; false when the bytes end early or a length is absurd.
inline bool bbv_read_tree(BvReader& r, BbvParsed& out, BvTree& t) {
    const uint64_t ni = r.u64();
    if (!r.ok || ni > (1u << 20) || !r.fits(ni, 4)) return false;
    if (ni > BV_MAX_OPENED) out.too_large = true;
    t.idx_off = (u32)out.words.size(); t.n_idx = (u32)ni;
    for (uint64_t i = 0; i < ni; i++) out.words.push_back(r.u32v());
    const uint64_t nv = r.u64();
    if (!r.ok || nv > (1u << 20) || !r.fits(nv, 4)) return false;
    t.val_off = (u32)out.words.size(); t.n_val = (u32)nv;
    for (uint64_t i = 0; i < nv; i++) out.words.push_back(r.u32v());
    const uint64_t nl = r.u64();
    if (!r.ok || nl > 64) return false;
    t.n_levels = (u32)nl;
    std::vector<u32> counts, digs;
    for (uint64_t l = 0; l < nl; l++) {
        const uint64_t cnt = r.u64();
        if (!r.ok || cnt > (1u << 20) || !r.fits(cnt, 16)) return false;
        counts.push_back((u32)cnt);
        for (uint64_t i = 0; i < cnt * 4; i++) digs.push_back(r.u32v());
    }
    t.cnt_off = (u32)out.words.size();
    out.words.insert(out.words.end(), counts.begin(), counts.end());
    while (out.words.size() % 4) out.words.push_back(0);
    t.dig_off = (u32)out.words.size();
    out.words.insert(out.words.end(), digs.begin(), digs.end());
    return r.ok;
}

inline bool bbv_parse(const uint8_t* bytes, size_t len, BbvParsed& out) {
    BvReader r{bytes, len};
    struct Commit { u32 root[4]; uint64_t log_n; };
    const uint64_t kc = r.u64();
    if (!r.ok || kc > 4096 || !r.fits(kc, 32)) return false;
    std::vector<Commit> commits(kc);
    for (auto& c : commits) { for (int i = 0; i < 4; i++) c.root[i] = r.u32v(); r.u64(); c.log_n = r.u64(); }
    const uint64_t num_polys = r.u64();
    const uint64_t n_logs = r.u64();
    if (!r.ok || n_logs > 4096 || !r.fits(n_logs, 8)) return false;
    std::vector<uint64_t> logs(n_logs);
    for (auto& l : logs) l = r.u64();
    const uint64_t n_roots = r.u64();
    if (!r.ok || n_roots > 4096 || !r.fits(n_roots, 16)) return false;
    out.roots_off = (u32)out.words.size();
    for (uint64_t i = 0; i < n_roots * 4; i++) out.words.push_back(r.u32v());
    out.batched_off = (u32)out.words.size();
    for (int i = 0; i < 4; i++) out.words.push_back(r.u32v());
    const uint64_t n_fold = r.u64();
    if (!r.ok || n_fold > 64 || !r.fits(n_fold, 16)) return false;
    out.fold_off = (u32)out.words.size();
    for (uint64_t i = 0; i < n_fold * 4; i++) out.words.push_back(r.u32v());
    const uint64_t n_q = r.u64();
    if (!r.ok || n_q > 64) return false;
    // what the verifier decides before it touches the transcript (:965-972) and what would make it index out of range
    uint64_t max_log = 1;
    for (uint64_t l : logs) max_log = l > max_log ? l : max_log;
    bool shape_ok = kc == num_polys && kc == n_roots && n_logs == kc;
    for (uint64_t l : logs) if (l < 1 || l > 28) shape_ok = false;
    if (shape_ok && kc == 0) out.trivially_true = true;
    if (n_fold < max_log || n_q < max_log) shape_ok = false;
    out.k = (u32)kc; out.log_n = (u32)max_log;
    const size_t commit_off = out.words.size();               // commitment roots by log_n descending (stable), for the individual openings
    {
        std::vector<size_t> order(kc);
        for (size_t i = 0; i < kc; i++) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return commits[a].log_n > commits[b].log_n; });
        std::vector<uint64_t> sorted_logs;
        for (size_t i : order) { for (int w = 0; w < 4; w++) out.words.push_back(commits[i].root[w]); sorted_logs.push_back(commits[i].log_n); }
        for (uint64_t round = 0; round < n_q; round++) {
            for (int tree = 0; tree < 2; tree++) {
                BvTree t{};
                if (!bbv_read_tree(r, out, t)) return false;
                if (round < max_log) {
                    t.root_off = tree == 0 ? (round == 0 ? out.batched_off : out.fold_off + 4u * (u32)(round - 1)) : out.fold_off + 4u * (u32)round;
                    t.log_height = (u32)(max_log + 1 - round) - (tree == 0 ? 0u : 1u);
                    out.trees.push_back(t);
                }
            }
        }
        const uint64_t n_open = r.u64();
        if (!r.ok || n_open > 4096) return false;
        std::vector<BvTree> individual;
        for (uint64_t i = 0; i < n_open; i++) {
            BvTree t{};
            if (!bbv_read_tree(r, out, t)) return false;
            if (i < kc) {                                       // openings beyond the number of commitments are not looked at (:1110-1112)
                if (sorted_logs[i] > 40) { shape_ok = false; continue; }
                t.root_off = (u32)(commit_off + 4 * i);
                t.log_height = (u32)sorted_logs[i] + 1;
                individual.push_back(t);
            }
        }
        r.u32v();                                               // final_value: not checked by the reference
        const uint64_t n_add = r.u64();
        if (!r.ok || n_add > 64) return false;
        out.add_first.assign(max_log, 0); out.add_count.assign(max_log, 0);
        std::vector<std::vector<BbvAdd>> by_round(max_log);
        std::vector<BvTree> add_trees;
        for (uint64_t a = 0; a < n_add; a++) {
            const uint64_t round = r.u64();
            const uint64_t cnt = r.u64();
            if (!r.ok || cnt > 4096) return false;
            std::vector<BbvAdd> lst;
            for (uint64_t j = 0; j < cnt; j++) {
                const uint64_t poly = r.u64();
                BvTree t{};
                if (!bbv_read_tree(r, out, t)) return false;
                if (!shape_ok) continue;
                if (poly >= kc) { shape_ok = false; continue; }
                t.root_off = out.roots_off + 4u * (u32)poly;
                t.log_height = (u32)logs[poly] + 1;
                lst.push_back(BbvAdd{(u32)(2 * max_log + add_trees.size()), (u32)poly, (u32)logs[poly], 0});
                add_trees.push_back(t);                         // every add opening is Merkle-checked (:1126-1135) ...
            }
            if (shape_ok && round < max_log) by_round[round] = lst;   // ... and the last entry of a round is the one the fold check uses (HashMap insert)
        }
        if (shape_ok) {
            out.trees.insert(out.trees.end(), add_trees.begin(), add_trees.end());
            out.trees.insert(out.trees.end(), individual.begin(), individual.end());
            for (uint64_t round = 0; round < max_log; round++) {
                out.add_first[round] = (u32)out.adds.size();
                out.add_count[round] = (u32)by_round[round].size();
                out.adds.insert(out.adds.end(), by_round[round].begin(), by_round[round].end());
            }
        }
    }
    out.reject = !shape_ok;
    return r.ok && r.at == len;
}

__global__ void bbv_chain_kernel(TrState* st, const u32* __restrict__ words, u32 k, u32 roots_off, u32 batched_off, u32 fold_off, u32 log_n,
                                 u32* rho_out, u32* alpha_out, u32* qidx_out) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    if (threadIdx.x) return;
    Tr tr;
    tr_load(tr, st, trbuf);
    for (u32 i = 0; i < 4 * k; i++) tr_absorb_u32(tr, words[roots_off + i]);
    rho_out[0] = tr_squeeze(tr);
    for (u32 i = 0; i < 4; i++) tr_absorb_u32(tr, words[batched_off + i]);
    for (u32 b = 0; b < log_n; b++) alpha_out[b] = tr_squeeze(tr);
    for (u32 round = 0; round < log_n; round++) {
        tr_absorb_u32(tr, alpha_out[round]);
        for (u32 i = 0; i < 4; i++) tr_absorb_u32(tr, words[fold_off + 4 * round + i]);
        const u32 prev_half_mask = (1u << (log_n - round)) - 1;
        for (u32 q = 0; q < BF_QUERIES; q++) qidx_out[round * BF_QUERIES + q] = tr_squeeze(tr) & prev_half_mask;
    }
    for (u32 q = 0; q < BF_QUERIES; q++) tr_squeeze(tr);
    tr_store(tr, st);
}

// Fold consistency of one query with the joined polynomials' contributions (basefold.rs:1014-1082): one warp per (round, query).
__global__ void bbv_fold_kernel(const u32* __restrict__ words, const BvTree* __restrict__ trees, u32 log_n, const u32* __restrict__ rho,
                                const u32* __restrict__ alpha, const u32* __restrict__ qidx, const u32* __restrict__ w_flat,
                                const BbvAdd* __restrict__ adds, const u32* __restrict__ add_first, const u32* __restrict__ add_count, u32* result) {
    const u32 item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= log_n * BF_QUERIES) return;
    const u32 round = item / BF_QUERIES;
    const BvTree bp = trees[2 * round], fbp = trees[2 * round + 1];
    const u32 prev_half = 1u << (log_n - round);
    const u32 idx = qidx[item] & (prev_half - 1);
    auto find = [&](const BvTree& t, u32 want, u32& val) -> bool {
        u32 best = 0xffffffffu;
        for (u32 i = lane; i < t.n_idx; i += 32)
            if (words[t.idx_off + i] == want) { best = i; break; }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) { const u32 o = __shfl_xor_sync(0xffffffffu, best, off); best = o < best ? o : best; }
        if (best == 0xffffffffu || best >= t.n_val) return false;
        val = words[t.val_off + best];
        return true;
    };
    u32 lv = 0, rv = 0, fv = 0;
    bool ok = find(bp, idx, lv) && find(bp, idx + prev_half, rv);
    if (ok) {
        const u32 fold_level = log_n - 1 - round;
        const u32 w = w_flat[((1u << fold_level) - 1) + (idx & ((1u << fold_level) - 1))];
        const u32 two_inv = (ZKB_P + 1) / 2;
        const u32 l = lv % ZKB_P, r = rv % ZKB_P;
        u32 expect = add31(mul31(add31(l, r), two_inv), mul31(mul31(alpha[round], sub31(l, r)), w));
        for (u32 a = 0; a < add_count[round]; a++) {
            const BbvAdd ad = adds[add_first[round] + a];
            u32 v = 0;
            if (find(trees[ad.tree], idx & ((1u << ad.log_n) - 1), v)) expect = add31(expect, mul31(pow31(rho[0], ad.poly), v % ZKB_P));
        }
        ok = find(fbp, idx, fv) && (fv % ZKB_P) == expect;
    }
    if (lane == 0) result[item] = ok ? 1u : 0u;
}

inline BvRun basefold_batch_verify_enqueue(zkb_ctx* c, TrState* tr, const BbvParsed& pr, int kind) {
    if (kind != NODE_BLAKE3 && kind != NODE_AES_MMO) throw ArgFail{ZKB_E_ARG, "unknown node hash"};
    if (kind == NODE_AES_MMO) aes_tables_upload();
    const u32 log_n = pr.log_n, n_trees = (u32)pr.trees.size();
    BfTables tb = bf_tables(c, log_n);
    u32* words = (u32*)c->scratch(pr.words.size() * 4 + 16);
    BvTree* trees = (BvTree*)c->scratch(pr.trees.size() * sizeof(BvTree) + 16);
    BbvAdd* adds = (BbvAdd*)c->scratch(pr.adds.size() * sizeof(BbvAdd) + 16);
    u32* add_first = (u32*)c->scratch((size_t)log_n * 4 + 16);
    u32* add_count = (u32*)c->scratch((size_t)log_n * 4 + 16);
    u32* rho = (u32*)c->scratch(16);
    u32* alpha = (u32*)c->scratch((size_t)log_n * 4 + 16);
    u32* qidx = (u32*)c->scratch((size_t)log_n * BF_QUERIES * 4 + 16);
    BvRun run;
    run.n_results = n_trees + log_n * BF_QUERIES;
    run.result_dev = (u32*)c->scratch((size_t)run.n_results * 4 + 16);
    ZKB_CUDA(cudaMemcpyAsync(words, pr.words.data(), pr.words.size() * 4, cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemcpyAsync(trees, pr.trees.data(), pr.trees.size() * sizeof(BvTree), cudaMemcpyHostToDevice, c->stream));
    if (!pr.adds.empty()) ZKB_CUDA(cudaMemcpyAsync(adds, pr.adds.data(), pr.adds.size() * sizeof(BbvAdd), cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemcpyAsync(add_first, pr.add_first.data(), (size_t)log_n * 4, cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemcpyAsync(add_count, pr.add_count.data(), (size_t)log_n * 4, cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemsetAsync(run.result_dev, 0, (size_t)run.n_results * 4, c->stream));
    cudaStream_t main_stream = c->stream, side = c->capturing ? main_stream : c->side_stream();
    if (side != main_stream) {
        cudaEvent_t fork = c->side_event(0);
        ZKB_CUDA(cudaEventRecord(fork, main_stream));
        ZKB_CUDA(cudaStreamWaitEvent(side, fork, 0));
    }
    if (kind == NODE_AES_MMO) bf_verify_batch_kernel<NODE_AES_MMO><<<n_trees, 128, 0, side>>>(words, trees, run.result_dev);
    else bf_verify_batch_kernel<NODE_BLAKE3><<<n_trees, 128, 0, side>>>(words, trees, run.result_dev);
    ZKB_LAUNCHED(c);
    bbv_chain_kernel<<<1, 32, exclusive_smem(bbv_chain_kernel, c), main_stream>>>(tr, words, pr.k, pr.roots_off, pr.batched_off, pr.fold_off, log_n, rho, alpha, qidx);
    ZKB_LAUNCHED(c);
    const u32 items = log_n * BF_QUERIES;
    bbv_fold_kernel<<<(items + 7) / 8, 256, 0, main_stream>>>(words, trees, log_n, rho, alpha, qidx, tb.w_flat, adds, add_first, add_count, run.result_dev + n_trees);
    ZKB_LAUNCHED(c);
    if (side != main_stream) {
        cudaEvent_t join = c->side_event(1);
        ZKB_CUDA(cudaEventRecord(join, side));
        ZKB_CUDA(cudaStreamWaitEvent(main_stream, join, 0));
    }
    ZKB_CUDA(cudaGetLastError());
    return run;
}

}  // namespace zkb
