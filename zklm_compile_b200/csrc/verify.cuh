// Basefold opening verifier (rust/zk_ml_prover/src/proving/basefold.rs:611-748) with the batched
// Merkle check it rests on (proving/pcs.rs:345-438).
//
// The host decodes bincode(BasefoldCommitment) || bincode(BasefoldOpeningProof) into one flat word
// array plus one descriptor per (round, tree).  Three kernels then run:
//
//   bf_verify_chain_kernel   the transcript of all rounds (challenge, root absorb, 24 query squeezes
//                            each): one thread, the same serial SHA-256 chain the prover runs
//   bf_verify_batch_kernel   one CTA per (round, tree): leaves sorted and de-duplicated, then level by
//                            level the missing siblings merged in from the proof and the parents
//                            hashed in parallel, up to the root; does not depend on the transcript,
//                            so it runs on the context's second stream beside the chain
//   bf_verify_fold_kernel    one warp per (round, query): the opened left / right / folded values
//                            and the fold relation  (l + r) / 2 + alpha (l - r) w[idx]
//
// Every check writes one word of a result vector; the proof is accepted when all are 1 and the final
// value equals the claimed evaluation.
#pragma once
#include "basefold.cuh"

namespace zkb {

constexpr u32 BV_MAX_OPENED = 256;      // opened positions per batch proof (an honest proof has 48 / 24)

struct BvTree {
    u32 idx_off, val_off, n_idx, n_val;         // word offsets into the flat array
    u32 n_levels, cnt_off, dig_off;             // cnt_off: n_levels counts; dig_off: all digests of all levels, 4 words each
    u32 root_off, log_height;
};

// ---- host: bincode reader -------------------------------------------------------------------------
struct BvReader {
    const uint8_t* p; size_t n, at = 0; bool ok = true;
    uint64_t u64() { if (at + 8 > n) { ok = false; return 0; } uint64_t v = 0; for (int i = 0; i < 8; i++) v |= (uint64_t)p[at + i] << (8 * i); at += 8; return v; }
    uint32_t u32v() { if (at + 4 > n) { ok = false; return 0; } uint32_t v = 0; for (int i = 0; i < 4; i++) v |= (uint32_t)p[at + i] << (8 * i); at += 4; return v; }
    // a declared element count that the remaining bytes cannot hold ends the decode (nothing is allocated for it)
    bool fits(uint64_t count, size_t bytes_each) { if (!ok || count > (n - at) / bytes_each) { ok = false; return false; } return true; }
};
struct BvParsed {
    std::vector<u32> words;            // [commitment root 4][fold roots 4 each][per tree: indices, values, counts, digests]
    std::vector<BvTree> trees;         // 2 per round: previous tree, folded tree
    u32 log_n = 0, final_value = 0;
    uint64_t num_coeffs = 0;
    bool too_large = false;
};
// With `used`, trailing bytes are allowed and the number of bytes decoded is returned there.
inline bool bv_parse(const uint8_t* bytes, size_t len, BvParsed& out, size_t* used = nullptr) {
    BvReader r{bytes, len};
    for (int i = 0; i < 4; i++) out.words.push_back(r.u32v());
    out.num_coeffs = r.u64();
    const uint64_t log_n = r.u64();
    if (!r.ok || log_n < 1 || log_n > 28) return false;
    out.log_n = (u32)log_n;
    const uint64_t n_roots = r.u64();
    if (!r.ok || n_roots > 64 || !r.fits(n_roots, 16)) return false;
    for (uint64_t i = 0; i < n_roots; i++) for (int k = 0; k < 4; k++) out.words.push_back(r.u32v());
    const uint64_t n_q = r.u64();
    if (!r.ok || n_q > 64) return false;
    if (n_roots != log_n || n_q != log_n) {      // wrong number of fold rounds: rejected, not malformed (the rest is not decoded)
        out.trees.clear();
        if (used) return false;                  // embedded in a larger proof: where it ends is unknown
        return r.ok;
    }
    for (uint64_t round = 0; round < n_q; round++) {
        for (int tree = 0; tree < 2; tree++) {
            BvTree t{};
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
            while (out.words.size() % 4) out.words.push_back(0);            // digests are read as 16-byte vectors
            t.dig_off = (u32)out.words.size();
            out.words.insert(out.words.end(), digs.begin(), digs.end());
            // tree of round `round`: the previous one hangs off the commitment root (round 0) or the last fold root
            t.root_off = tree == 0 ? (round == 0 ? 0u : 4u + 4u * (u32)(round - 1)) : 4u + 4u * (u32)round;
            t.log_height = (u32)(log_n + 1 - round) - (tree == 0 ? 0u : 1u);
            out.trees.push_back(t);
        }
    }
    out.final_value = r.u32v();
    const uint64_t n_final = r.u64();
    if (n_final > (1u << 20) || !r.fits(n_final, 4)) return false;
    for (uint64_t i = 0; i < n_final && r.ok; i++) r.u32v();
    if (used) { *used = r.at; return r.ok; }
    return r.ok && r.at == len;
}

// ---- device ------------------------------------------------------------------------------------------
__global__ void bf_verify_chain_kernel(TrState* st, const u32* __restrict__ words, u32 log_n, const u32* __restrict__ point, u32 n_point,
                                       u32* alpha_out, u32* qidx_out) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    if (threadIdx.x) return;
    Tr tr;
    tr_load(tr, st, trbuf);
    for (u32 round = 0; round < log_n; round++) {
        alpha_out[round] = bf_next_alpha(tr, point, n_point, round);
        const u32* root = words + 4 + 4 * round;
        u32 rw[4] = {root[0], root[1], root[2], root[3]};
        tr_absorb_words<4>(tr, rw);
        const u32 prev_half_mask = (1u << (log_n - round)) - 1;
        for (u32 q = 0; q < BF_QUERIES; q++) qidx_out[round * BF_QUERIES + q] = tr_squeeze(tr) & prev_half_mask;
    }
    tr_store(tr, st);
}

template <int KIND>
__device__ __forceinline__ uint4 bv_node(uint4 l, uint4 r, const u32* t0_s, const unsigned char* sb_s) {
    if (KIND == NODE_AES_MMO) return aes_node(l, r, t0_s, sb_s);
    return b3_node(l, r);
}
// verify_batch_opening (pcs.rs:345-438).  One CTA per tree; result[blockIdx.x] = 1 when the tree's openings hash up to its root.
template <int KIND>
__global__ void __launch_bounds__(128) bf_verify_batch_kernel(const u32* __restrict__ words, const BvTree* __restrict__ trees, u32* result) {
    __shared__ u32 idx_a[BV_MAX_OPENED], idx_b[BV_MAX_OPENED];
    __shared__ uint4 dig_a[BV_MAX_OPENED], dig_b[BV_MAX_OPENED];
    __shared__ int left_src[BV_MAX_OPENED], right_src[BV_MAX_OPENED];     // >= 0: entry of the current list; < 0: ~j = sibling digest j of the proof
    __shared__ u32 par_idx[BV_MAX_OPENED];
    __shared__ u32 n_cur, n_par, fail;
    __shared__ u32 t0_s[256];
    __shared__ unsigned char sb_s[256];
    const BvTree t = trees[blockIdx.x];
    if (KIND == NODE_AES_MMO) for (int i = threadIdx.x; i < 256; i += blockDim.x) { t0_s[i] = AES_T0[i]; sb_s[i] = AES_SBOX[i]; }
    if (threadIdx.x == 0) { fail = (t.n_idx != t.n_val || t.n_idx == 0 || t.n_idx > BV_MAX_OPENED) ? 1u : 0u; }
    __syncthreads();
    if (fail) { if (threadIdx.x == 0) result[blockIdx.x] = 0; return; }
    // leaves: (index, hash_leaf(value)) sorted by index, the first of equal indices kept
    const u32 n0 = t.n_idx;
    for (u32 i = threadIdx.x; i < n0; i += blockDim.x) {
        const u32 my = words[t.idx_off + i];
        u32 rank = 0;
        for (u32 j = 0; j < n0; j++) {
            const u32 o = words[t.idx_off + j];
            rank += (o < my || (o == my && j < i)) ? 1u : 0u;
        }
        idx_b[rank] = my;
        dig_b[rank] = make_uint4(words[t.val_off + i], 0u, 0u, 0u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        u32 n = 0;
        for (u32 i = 0; i < n0; i++)
            if (i == 0 || idx_b[i] != idx_b[i - 1]) { idx_a[n] = idx_b[i]; dig_a[n] = dig_b[i]; n++; }
        n_cur = n;
    }
    __syncthreads();
    u32* idx_cur = idx_a; uint4* dig_cur = dig_a;
    u32* idx_nxt = idx_b; uint4* dig_nxt = dig_b;
    u32 dig_base = t.dig_off;            // first digest word of the current level's siblings
    for (u32 k = 0; k < t.log_height; k++) {
        const u32 n_auth = k < t.n_levels ? words[t.cnt_off + k] : 0u;
        if (threadIdx.x == 0) {
            // pairs in ascending order; a sibling that is not in the list is the next unused digest of this level
            u32 used = 0, np = 0;
            const u32 n = n_cur;
            for (u32 i = 0; i < n;) {
                const u32 id = idx_cur[i];
                const bool both = (id & 1u) == 0 && i + 1 < n && idx_cur[i + 1] == (id | 1u);
                if (both) { left_src[np] = (int)i; right_src[np] = (int)(i + 1); i += 2; }
                else {
                    if (id & 1u) { left_src[np] = ~(int)used; right_src[np] = (int)i; }
                    else { left_src[np] = (int)i; right_src[np] = ~(int)used; }
                    used++;
                    i += 1;
                }
                par_idx[np] = id >> 1;
                np++;
            }
            // the proof must hold exactly the missing siblings of this level (none when the level is absent or empty)
            if (used != n_auth) fail = 1;
            n_par = np;
        }
        __syncthreads();
        if (fail) break;
        const u32 np = n_par;
        for (u32 pi = threadIdx.x; pi < np; pi += blockDim.x) {
            const int ls = left_src[pi], rs = right_src[pi];
            const uint4 l = ls >= 0 ? dig_cur[ls] : *reinterpret_cast<const uint4*>(words + dig_base + 4 * (u32)(~ls));
            const uint4 r = rs >= 0 ? dig_cur[rs] : *reinterpret_cast<const uint4*>(words + dig_base + 4 * (u32)(~rs));
            dig_nxt[pi] = bv_node<KIND>(l, r, t0_s, sb_s);
            idx_nxt[pi] = par_idx[pi];
        }
        __syncthreads();
        if (threadIdx.x == 0) n_cur = np;
        u32* ti = idx_cur; idx_cur = idx_nxt; idx_nxt = ti;
        uint4* td = dig_cur; dig_cur = dig_nxt; dig_nxt = td;
        dig_base += 4 * n_auth;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        bool ok = !fail && n_cur == 1 && idx_cur[0] == 0;
        if (ok) {
            const u32* root = words + t.root_off;
            const uint4 d = dig_cur[0];
            ok = d.x == root[0] && d.y == root[1] && d.z == root[2] && d.w == root[3];
        }
        result[blockIdx.x] = ok ? 1u : 0u;
    }
}

// Fold consistency of one query (basefold.rs:677-713): one warp per (round, query).
__global__ void bf_verify_fold_kernel(const u32* __restrict__ words, const BvTree* __restrict__ trees, u32 log_n, const u32* __restrict__ alpha,
                                      const u32* __restrict__ qidx, const u32* __restrict__ w_flat, u32* result) {
    const u32 item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= log_n * BF_QUERIES) return;
    const u32 round = item / BF_QUERIES;
    const BvTree bp = trees[2 * round], fbp = trees[2 * round + 1];
    const u32 prev_half = 1u << (log_n - round);
    const u32 idx = qidx[item] & (prev_half - 1);
    // first position of an index in a batch proof (`iter().position`), found by the warp
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
    bool ok = find(bp, idx, lv) && find(bp, idx + prev_half, rv) && find(fbp, idx, fv);
    if (ok) {
        const u32 fold_level = log_n - 1 - round;
        const u32 w = w_flat[((1u << fold_level) - 1) + (idx & ((1u << fold_level) - 1))];
        const u32 two_inv = (ZKB_P + 1) / 2;
        const u32 l = lv % ZKB_P, r = rv % ZKB_P;                         // from_canonical_u32 of an arbitrary word
        const u32 expect = add31(mul31(add31(l, r), two_inv), mul31(mul31(alpha[round], sub31(l, r)), w));
        ok = (fv % ZKB_P) == expect;
    }
    if (lane == 0) result[item] = ok ? 1u : 0u;
}

// Enqueue the whole check; returns the number of result words (all must be 1) at result_dev.
struct BvRun { u32 n_results = 0; u32* result_dev = nullptr; };
inline BvRun basefold_verify_enqueue(zkb_ctx* c, TrState* tr, const BvParsed& pr, const u32* point_dev, u32 n_point, int kind) {
    if (kind != NODE_BLAKE3 && kind != NODE_AES_MMO) throw ArgFail{ZKB_E_ARG, "unknown node hash"};
    if (kind == NODE_AES_MMO) aes_tables_upload();
    const u32 log_n = pr.log_n, n_trees = 2 * log_n;
    BfTables tb = bf_tables(c, log_n);
    u32* words = (u32*)c->scratch(pr.words.size() * 4 + 16);
    BvTree* trees = (BvTree*)c->scratch(pr.trees.size() * sizeof(BvTree) + 16);
    u32* alpha = (u32*)c->scratch((size_t)log_n * 4 + 16);
    u32* qidx = (u32*)c->scratch((size_t)log_n * BF_QUERIES * 4 + 16);
    BvRun run;
    run.n_results = n_trees + log_n * BF_QUERIES;
    run.result_dev = (u32*)c->scratch((size_t)run.n_results * 4 + 16);
    ZKB_CUDA(cudaMemcpyAsync(words, pr.words.data(), pr.words.size() * 4, cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemcpyAsync(trees, pr.trees.data(), pr.trees.size() * sizeof(BvTree), cudaMemcpyHostToDevice, c->stream));
    ZKB_CUDA(cudaMemsetAsync(run.result_dev, 0, (size_t)run.n_results * 4, c->stream));
    // the Merkle checks need only the proof: second stream, joined before the results are read
    cudaStream_t main_stream = c->stream, side = c->capturing ? main_stream : c->side_stream();
    if (side != main_stream) {
        cudaEvent_t fork = c->side_event(0);
        ZKB_CUDA(cudaEventRecord(fork, main_stream));
        ZKB_CUDA(cudaStreamWaitEvent(side, fork, 0));
    }
    if (kind == NODE_AES_MMO) bf_verify_batch_kernel<NODE_AES_MMO><<<n_trees, 128, 0, side>>>(words, trees, run.result_dev);
    else bf_verify_batch_kernel<NODE_BLAKE3><<<n_trees, 128, 0, side>>>(words, trees, run.result_dev);
    ZKB_LAUNCHED(c);
    bf_verify_chain_kernel<<<1, 32, exclusive_smem(bf_verify_chain_kernel, c), main_stream>>>(tr, words, log_n, point_dev, n_point, alpha, qidx);
    ZKB_LAUNCHED(c);
    const u32 items = log_n * BF_QUERIES;
    bf_verify_fold_kernel<<<(items + 7) / 8, 256, 0, main_stream>>>(words, trees, log_n, alpha, qidx, tb.w_flat, run.result_dev + n_trees);
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
