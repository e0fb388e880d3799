// Basefold polynomial commitment, single polynomial
// (rust/zk_ml_prover/src/proving/basefold.rs:106-585).
//
//   tables      T = 1 + (u32 LE of the blake3 XOF of a per-size seed) mod (p - 1), 2^L - 1 values,
//               level i (2^i values) at offset 2^i - 1; w = 1 / (2 T)               basefold.rs:106-157, 323-328
//   encode      cw = [c || c]; level l: chunks of 2^(l+1), L' = L + T R, R' = L - T R   basefold.rs:169-238
//   fold        cw'[j] = (l + r) / 2 + alpha (l - r) w[j mod |w|], l = cw[j], r = cw[j + half]   basefold.rs:250-316
//   opening     per round: alpha, fold coefficients and codeword, Merkle tree of the folded
//               codeword, absorb root, 24 query positions, openings in both trees    basefold.rs:483-585
//
// XOF output block b of a root node is one compression with counter b, so the tables are
// generated one 64-byte block per thread.  Encoding never mixes the two halves of [c || c]
// (chunks are at most 2^log_n long), so one half is computed and written twice.  Levels below
// 2^12 run in shared memory in one pass; higher levels go six at a time through tiles of
// 64 consecutive values x 64 strided rows.  Each fold is fused with the first ten levels of the
// Merkle tree over its output.  The whole opening runs without host round trips: challenges,
// roots, query positions and the raw authentication paths are written to the proof record.
#pragma once
#include "engine.cuh"
#include "merkle.cuh"
#include <algorithm>
#include <map>
#include <mutex>

namespace zkb {

// Full 16-word output of the blake3 compression (needed for XOF blocks).
__device__ inline void b3_compress16(const u32* cv, const u32* m, u32 counter_lo, u32 counter_hi, u32 blen, u32 flags, u32* out16) {
    u32 s0 = cv[0], s1 = cv[1], s2 = cv[2], s3 = cv[3], s4 = cv[4], s5 = cv[5], s6 = cv[6], s7 = cv[7];
    u32 s8 = 0x6a09e667u, s9 = 0xbb67ae85u, s10 = 0x3c6ef372u, s11 = 0xa54ff53au;
    u32 s12 = counter_lo, s13 = counter_hi, s14 = blen, s15 = flags;
    u32 w[16];
#pragma unroll
    for (int i = 0; i < 16; i++) w[i] = m[i];
#pragma unroll
    for (int r = 0; r < 7; r++) {
        B3_G(s0, s4, s8, s12, w[0], w[1]);   B3_G(s1, s5, s9, s13, w[2], w[3]);
        B3_G(s2, s6, s10, s14, w[4], w[5]);  B3_G(s3, s7, s11, s15, w[6], w[7]);
        B3_G(s0, s5, s10, s15, w[8], w[9]);  B3_G(s1, s6, s11, s12, w[10], w[11]);
        B3_G(s2, s7, s8, s13, w[12], w[13]); B3_G(s3, s4, s9, s14, w[14], w[15]);
        if (r < 6) {
            u32 t[16] = {w[2], w[6], w[3], w[10], w[7], w[0], w[4], w[13], w[1], w[11], w[12], w[5], w[9], w[14], w[15], w[8]};
#pragma unroll
            for (int i = 0; i < 16; i++) w[i] = t[i];
        }
    }
    out16[0] = s0 ^ s8;   out16[1] = s1 ^ s9;   out16[2] = s2 ^ s10;  out16[3] = s3 ^ s11;
    out16[4] = s4 ^ s12;  out16[5] = s5 ^ s13;  out16[6] = s6 ^ s14;  out16[7] = s7 ^ s15;
    out16[8] = s8 ^ cv[0];   out16[9] = s9 ^ cv[1];   out16[10] = s10 ^ cv[2];  out16[11] = s11 ^ cv[3];
    out16[12] = s12 ^ cv[4]; out16[13] = s13 ^ cv[5]; out16[14] = s14 ^ cv[6];  out16[15] = s15 ^ cv[7];
}

struct BfSeed { u32 w[8]; };

// One thread = one XOF block = 16 table entries and their fold weights (one inversion per thread).
__global__ void __launch_bounds__(128) bf_tables_kernel(BfSeed seed, size_t total, u32* __restrict__ t_flat, u32* __restrict__ w_flat) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b * 16 >= total) return;
    u32 cv[8], m[16], o[16];
#pragma unroll
    for (int i = 0; i < 8; i++) { cv[i] = B3_IV[i]; m[i] = seed.w[i]; m[8 + i] = 0; }
    b3_compress16(cv, m, (u32)b, (u32)(b >> 32), 32, B3_CHUNK_START | B3_CHUNK_END | B3_ROOT, o);
    u32 t[16], pre[16];
    u32 acc = 1;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        t[i] = 1 + o[i] % (ZKB_P - 1);
        pre[i] = acc;
        acc = mul31(acc, add31(t[i], t[i]));
    }
    u32 inv = inv31(acc);
#pragma unroll
    for (int i = 15; i >= 0; i--) {
        u32 wv = mul31(pre[i], inv);
        inv = mul31(inv, add31(t[i], t[i]));
        size_t g = b * 16 + i;
        if (g < total) { t_flat[g] = t[i]; w_flat[g] = wv; }
    }
}

// ---- encode -------------------------------------------------------------------------------------
struct CoefSrc { const u32* p; u32 rows, cols, log_cols_pad; };

constexpr int BF_LOW_LOG = 12;
// Levels 0..K-1 on tiles of 2^K coefficients (K <= BF_LOW_LOG), entirely in shared memory.
__global__ void __launch_bounds__(256) bf_encode_low_kernel(CoefSrc src, u32 K, const u32* __restrict__ t_flat, u32* __restrict__ cw,
                                                            size_t n_pad, int dup) {
    __shared__ u32 s[1 << BF_LOW_LOG];
    __shared__ u32 tw[1 << BF_LOW_LOG];
    const u32 T = 1u << K;
    const size_t base = (size_t)blockIdx.x << K;
    for (u32 i = threadIdx.x; i < T; i += blockDim.x) {
        s[i] = coef_at(src.p, src.rows, src.cols, src.log_cols_pad, base + i);
        if (i + 1 < T) tw[i] = t_flat[i];
    }
    __syncthreads();
    for (u32 l = 0; l < K; l++) {
        const u32 half = 1u << l;
        for (u32 b = threadIdx.x; b < T / 2; b += blockDim.x) {
            u32 j = b & (half - 1);
            u32 iL = ((b >> l) << (l + 1)) + j, iR = iL + half;
            u32 rhs = mul31(s[iR], tw[half - 1 + j]);
            u32 L = s[iL];
            s[iL] = add31(L, rhs);
            s[iR] = sub31(L, rhs);
        }
        __syncthreads();
    }
    for (u32 i = threadIdx.x; i < T; i += blockDim.x) {
        cw[base + i] = s[i];
        if (dup) cw[n_pad + base + i] = s[i];
    }
}
// Levels l0 .. l0+r-1 (r <= 6, l0 >= 6): a CTA holds 2^r rows (stride 2^l0) of 64 consecutive values.
__global__ void __launch_bounds__(256) bf_encode_high_kernel(u32* __restrict__ cw, u32 l0, u32 r, const u32* __restrict__ t_flat,
                                                             size_t n_pad, int dup) {
    __shared__ u32 s[64 * 64];
    const u32 rows = 1u << r;
    const size_t lo_chunks = (size_t(1) << l0) >> 6;
    const size_t H = blockIdx.x / lo_chunks, lc = blockIdx.x % lo_chunks;
    const size_t base = (H << (l0 + r)) + (lc << 6);
    for (u32 e = threadIdx.x; e < rows * 64; e += blockDim.x) s[e] = cw[base + ((size_t)(e >> 6) << l0) + (e & 63)];
    __syncthreads();
    for (u32 st = 0; st < r; st++) {
        const u32 l = l0 + st;
        const u32* t = t_flat + ((size_t(1) << l) - 1);
        for (u32 b = threadIdx.x; b < rows * 32; b += blockDim.x) {
            u32 x = b & 63, pm = b >> 6;
            u32 mlow = pm & ((1u << st) - 1), mhigh = pm >> st;
            u32 midL = (mhigh << (st + 1)) | mlow, midR = midL | (1u << st);
            u32 tv = t[((size_t)mlow << l0) + (lc << 6) + x];
            u32 rhs = mul31(s[midR * 64 + x], tv);
            u32 L = s[midL * 64 + x];
            s[midL * 64 + x] = add31(L, rhs);
            s[midR * 64 + x] = sub31(L, rhs);
        }
        __syncthreads();
    }
    for (u32 e = threadIdx.x; e < rows * 64; e += blockDim.x) {
        size_t g = base + ((size_t)(e >> 6) << l0) + (e & 63);
        cw[g] = s[e];
        if (dup) cw[n_pad + g] = s[e];
    }
}

// ---- per-round transcript step and openings ------------------------------------------------------
constexpr u32 BF_QUERIES = 24;       // pcs.rs:19
struct BfRound {
    TrState* tr;
    const u32* point; u32 n_point;   // device-resident evaluation point
    u32 round, log_n;
    u32* alpha_next;                 // where the next round's challenge goes (null after the last round)
    // trees: prev has height h_prev over prev_values, folded has height h_prev - 1
    const u32* prev_values; const uint4* prev_nodes;
    const u32* fold_values; const uint4* fold_nodes;
    u32 h_prev;
    u32* rec;                        // [root 4][idx 24][48 prev paths][24 folded paths]
};
__host__ __device__ __forceinline__ size_t bf_round_words(u32 h_prev) {
    size_t pw_prev = 2 + 4 * (size_t)(h_prev - 1), pw_fold = h_prev >= 2 ? 2 + 4 * (size_t)(h_prev - 2) : 2;
    return 4 + BF_QUERIES + 2 * BF_QUERIES * pw_prev + BF_QUERIES * pw_fold;
}
// The challenge of a round: the point coordinate (absorbed) while there is one, else a squeeze
// (basefold.rs:508-513).
__device__ __forceinline__ u32 bf_next_alpha(Tr& tr, const u32* point, u32 n_point, u32 round) {
    if (round < n_point) { u32 a = point[round]; tr_absorb_u32(tr, a); return a; }
    return tr_squeeze(tr);
}
__global__ void __launch_bounds__(256) bf_round_kernel(BfRound p) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    __shared__ u32 idx_s[BF_QUERIES];
    const u32 h_fold = p.h_prev - 1;
    const uint4 root = p.fold_nodes[mk_layer_offset(h_fold, h_fold)];
    if (threadIdx.x == 0) {
        Tr tr;
        tr_load(tr, p.tr, trbuf);
        u32 rw[4] = {root.x, root.y, root.z, root.w};
        tr_absorb_words<4>(tr, rw);
        p.rec[0] = root.x; p.rec[1] = root.y; p.rec[2] = root.z; p.rec[3] = root.w;
        const u32 prev_half_mask = (1u << (p.h_prev - 1)) - 1;
        for (u32 q = 0; q < BF_QUERIES; q++) {
            u32 v = tr_squeeze(tr) & prev_half_mask;     // (squeeze mod 2^h_prev) mod prev_half
            idx_s[q] = v;
            p.rec[4 + q] = v;
        }
        if (p.alpha_next) *p.alpha_next = bf_next_alpha(tr, p.point, p.n_point, p.round + 1);
        tr_store(tr, p.tr);
    }
    __syncthreads();
    const size_t prev_half = size_t(1) << (p.h_prev - 1);
    const size_t pw_prev = 2 + 4 * (size_t)(p.h_prev - 1), pw_fold = h_fold >= 1 ? 2 + 4 * (size_t)(h_fold - 1) : 2;
    u32* out_prev = p.rec + 4 + BF_QUERIES;
    u32* out_fold = out_prev + 2 * BF_QUERIES * pw_prev;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (u32 item = warp; item < 3 * BF_QUERIES; item += nwarps) {
        if (item < 2 * BF_QUERIES) {
            size_t pos = idx_s[item >> 1] + ((item & 1) ? prev_half : 0);
            mk_gather_path(p.prev_values, size_t(1) << p.h_prev, p.prev_nodes, p.h_prev, pos, out_prev + item * pw_prev, lane, 32);
        } else {
            u32 q = item - 2 * BF_QUERIES;
            mk_gather_path(p.fold_values, prev_half, p.fold_nodes, h_fold, idx_s[q], out_fold + q * pw_fold, lane, 32);
        }
    }
}
// First challenge, after the commitment root has been absorbed (basefold.rs:461 / 508-513).
__global__ void bf_begin_kernel(TrState* st, const uint4* root, const u32* point, u32 n_point, u32* alpha0, u32* rec_root) {
    __shared__ __align__(16) unsigned char trbuf[TR_SCRATCH_BYTES];
    Tr tr;
    tr_load(tr, st, trbuf);
    uint4 r = *root;
    u32 rw[4] = {r.x, r.y, r.z, r.w};
    tr_absorb_words<4>(tr, rw);
    rec_root[0] = r.x; rec_root[1] = r.y; rec_root[2] = r.z; rec_root[3] = r.w;
    *alpha0 = bf_next_alpha(tr, point, n_point, 0);
    tr_store(tr, st);
}

// ---- host side ----------------------------------------------------------------------------------
struct BfTables { u32* t_flat; u32* w_flat; };

// One table set per (device, log_n) for the life of the process, as the reference caches them
// (basefold.rs:377-393).  The seed is blake3("basefold-foldable-code" || log_n as u64 LE).
inline BfTables bf_tables(zkb_ctx* c, u32 log_n) {
    static std::mutex mu;
    static std::map<std::pair<int, u32>, BfTables> cache;
    std::lock_guard<std::mutex> g(mu);
    auto key = std::make_pair(c->device, log_n);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    const size_t total = (size_t(1) << log_n) - 1;
    BfTables tb{};
    ZKB_CUDA(cudaMalloc(&tb.t_flat, (total + 1) * 4));
    ZKB_CUDA(cudaMalloc(&tb.w_flat, (total + 1) * 4));
    // seed: a 30-byte message hashed on the device through the generic commit path
    u32* seed_dev = (u32*)c->scratch(32);
    unsigned char msg[30];
    memcpy(msg, "basefold-foldable-code", 22);
    for (int i = 0; i < 8; i++) msg[22 + i] = (unsigned char)((uint64_t)log_n >> (8 * i));
    commit_large(c, b3_prefix(msg, 30), nullptr, 0, seed_dev);
    BfSeed seed;
    ZKB_CUDA(cudaMemcpyAsync(seed.w, seed_dev, 32, cudaMemcpyDeviceToHost, c->stream));
    ZKB_CUDA(cudaStreamSynchronize(c->stream));
    const size_t blocks = (total + 15) / 16;
    bf_tables_kernel<<<(unsigned)((blocks + 127) / 128), 128, 0, c->stream>>>(seed, total, tb.t_flat, tb.w_flat);
    ZKB_LAUNCHED(c);
    ZKB_CUDA(cudaStreamSynchronize(c->stream));
    cache[key] = tb;
    return tb;
}

// cw (2 * 2^log_n words) = encode of the zero-padded coefficients.
inline void bf_encode(zkb_ctx* c, CoefSrc src, u32 log_n, const BfTables& tb, u32* cw) {
    const size_t n_pad = size_t(1) << log_n;
    const u32 K = log_n < (u32)BF_LOW_LOG ? log_n : (u32)BF_LOW_LOG;
    bf_encode_low_kernel<<<(unsigned)(n_pad >> K), 256, 0, c->stream>>>(src, K, tb.t_flat, cw, n_pad, K == log_n);
    ZKB_LAUNCHED(c);
    u32 l0 = K;
    while (l0 < log_n) {
        u32 rem = log_n - l0;
        u32 r = rem <= 6 ? rem : (rem < 12 ? (rem + 1) / 2 : 6);
        bf_encode_high_kernel<<<(unsigned)(n_pad >> (r + 6)), 256, 0, c->stream>>>(cw, l0, r, tb.t_flat, n_pad, l0 + r == log_n);
        ZKB_LAUNCHED(c);
        l0 += r;
    }
}

template <int KIND>
inline void mk_launch(zkb_ctx* c, int mode, const u32* values, size_t n_valid, size_t n_in, u32 k0, u32 h, uint4* nodes, const MkFold& f) {
    const size_t tile = n_in < (size_t)MK_TILE ? n_in : (size_t)MK_TILE;
    const unsigned grid = (unsigned)(n_in / tile);
    if (mode == MK_VALUES) mk_tile_kernel<KIND, MK_VALUES><<<grid, MK_THREADS, 0, c->stream>>>(values, n_valid, n_in, k0, h, nodes, f);
    else if (mode == MK_DIGESTS) mk_tile_kernel<KIND, MK_DIGESTS><<<grid, MK_THREADS, 0, c->stream>>>(values, n_valid, n_in, k0, h, nodes, f);
    else mk_tile_kernel<KIND, MK_FOLD><<<grid, MK_THREADS, 0, c->stream>>>(values, n_valid, n_in, k0, h, nodes, f);
    ZKB_LAUNCHED(c);
}
// Build every layer of a tree of height h; the first launch reads leaves (values, or a fold).
inline void mk_build(zkb_ctx* c, int kind, int first_mode, const u32* values, size_t n_valid, u32 h, uint4* nodes, const MkFold& f) {
    u32 k0 = 0;
    int mode = first_mode;
    while (k0 < h) {
        size_t n_in = size_t(1) << (h - k0);
        if (kind == NODE_AES_MMO) mk_launch<NODE_AES_MMO>(c, mode, values, n_valid, n_in, k0, h, nodes, f);
        else mk_launch<NODE_BLAKE3>(c, mode, values, n_valid, n_in, k0, h, nodes, f);
        k0 += (h - k0) < (u32)MK_TILE_LOG ? (h - k0) : (u32)MK_TILE_LOG;
        mode = MK_DIGESTS;
    }
}
inline void aes_tables_upload() {
    static std::mutex mu;
    static std::map<int, bool> done;
    int dev = 0;
    ZKB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> g(mu);
    if (done[dev]) return;
    AesTables t = aes_make_tables();
    ZKB_CUDA(cudaMemcpyToSymbol(AES_T0, t.t0, sizeof(t.t0)));
    ZKB_CUDA(cudaMemcpyToSymbol(AES_SBOX, t.sbox, sizeof(t.sbox)));
    done[dev] = true;
}

// Record layout of one opening, filled by basefold_enqueue and read by basefold_finish.
struct BfPending {
    u32 log_n = 0;
    size_t num_coeffs = 0;
    size_t root_off = 0, final_off = 0;
    std::vector<size_t> round_off;
};

// Enqueue commit + opening of the polynomial `src` (num_coeffs live coefficients, padded view of
// 2^log_n) at the device-resident point.  The transcript first absorbs the commitment root.
inline BfPending basefold_enqueue(zkb_ctx* c, TrState* tr, CoefSrc src, size_t num_coeffs, u32 log_n, const u32* point_dev, u32 n_point,
                                  int kind) {
    if (log_n < 1 || log_n > 28) throw ArgFail{ZKB_E_TOO_LARGE, "basefold: log_n out of range"};
    if (kind != NODE_BLAKE3 && kind != NODE_AES_MMO) throw ArgFail{ZKB_E_ARG, "unknown node hash"};
    if (kind == NODE_AES_MMO) aes_tables_upload();
    BfTables tb = bf_tables(c, log_n);
    const size_t n_pad = size_t(1) << log_n;
    BfPending pd;
    pd.log_n = log_n; pd.num_coeffs = num_coeffs;
    // Every fold challenge that is a coordinate of the point is known before the opening starts (it is
    // absorbed, not squeezed: basefold.rs:508-513), so the folds and trees of those rounds do not wait for
    // the transcript: they run ahead on a second stream, each round into buffers of its own, while the
    // context's stream runs the hash chain (root absorb, 24 query squeezes) and the path gathers behind them.
    const bool ahead = n_point >= log_n && !c->opt_bf_in_order && !c->capturing;
    u32* cwA = (u32*)c->scratch(2 * n_pad * 4);
    u32* cwB = ahead ? nullptr : (u32*)c->scratch(n_pad * 4);
    u32* eval = (u32*)c->scratch((n_pad / 2 + 4) * 4);
    uint4* treeA = (uint4*)c->scratch(mk_node_count(log_n + 1) * 16 + 16);
    uint4* treeB = ahead ? nullptr : (uint4*)c->scratch(mk_node_count(log_n) * 16 + 16);
    u32* alpha = (u32*)c->scratch((log_n + 1) * 4);
    std::vector<u32*> cws;
    std::vector<uint4*> trees;
    if (ahead) {
        for (u32 round = 0; round < log_n; round++) {
            cws.push_back((u32*)c->scratch((size_t(4) << (log_n - round)) + 16));
            trees.push_back((uint4*)c->scratch(mk_node_count(log_n - round) * 16 + 16));
        }
    }

    c->prof_mark();
    bf_encode(c, src, log_n, tb, cwA);
    c->prof_mark();
    MkFold none{};
    mk_build(c, kind, MK_VALUES, cwA, 2 * n_pad, log_n + 1, treeA, none);
    c->prof_mark();
    cudaStream_t main_stream = c->stream, side = nullptr;
    if (ahead) {
        side = c->side_stream();
        cudaEvent_t fork = c->side_event(log_n);
        ZKB_CUDA(cudaEventRecord(fork, main_stream));
        ZKB_CUDA(cudaStreamWaitEvent(side, fork, 0));
    }
    pd.root_off = c->rec_alloc(4);
    bf_begin_kernel<<<1, 1, 0, c->stream>>>(tr, treeA + mk_layer_offset(log_n + 1, log_n + 1), point_dev, n_point, alpha, c->rec_dev + pd.root_off);
    ZKB_LAUNCHED(c);

    u32* prev_cw = cwA; u32* next_cw = ahead ? cws[0] : cwB;
    uint4* prev_tree = treeA; uint4* next_tree = ahead ? trees[0] : treeB;
    for (u32 round = 0; round < log_n; round++) {
        const u32 h_prev = log_n + 1 - round;
        const size_t half = size_t(1) << (h_prev - 1);
        const u32 fold_level = log_n - 1 - round;
        MkFold f{};
        f.prev = prev_cw; f.out = next_cw;
        f.weights = tb.w_flat + ((size_t(1) << fold_level) - 1);
        f.w_len = size_t(1) << fold_level;
        f.alpha = ahead ? point_dev + round : alpha + round;
        f.eval_src = eval; f.eval_dst = eval; f.eval_half = half / 2;
        f.coef = src.p; f.coef_rows = src.rows; f.coef_cols = src.cols; f.coef_log_cols_pad = src.log_cols_pad;
        f.eval_from_coef = round == 0;
        if (ahead) {
            c->stream = side;
            try { mk_build(c, kind, MK_FOLD, nullptr, half, h_prev - 1, next_tree, f); } catch (...) { c->stream = main_stream; throw; }
            c->stream = main_stream;
            ZKB_CUDA(cudaEventRecord(c->side_event(round), side));
            ZKB_CUDA(cudaStreamWaitEvent(main_stream, c->side_event(round), 0));
        } else {
            mk_build(c, kind, MK_FOLD, nullptr, half, h_prev - 1, next_tree, f);
        }
        c->prof_mark();
        BfRound rp{};
        rp.tr = tr; rp.point = point_dev; rp.n_point = n_point; rp.round = round; rp.log_n = log_n;
        rp.alpha_next = round + 1 < log_n ? alpha + round + 1 : nullptr;
        rp.prev_values = prev_cw; rp.prev_nodes = prev_tree; rp.fold_values = next_cw; rp.fold_nodes = next_tree;
        rp.h_prev = h_prev;
        size_t off = c->rec_alloc(bf_round_words(h_prev));
        rp.rec = c->rec_dev + off;
        pd.round_off.push_back(off);
        bf_round_kernel<<<1, 256, exclusive_smem(bf_round_kernel, c), c->stream>>>(rp);
        ZKB_LAUNCHED(c);
        c->prof_mark();
        if (ahead) {
            prev_cw = next_cw; prev_tree = next_tree;
            if (round + 1 < log_n) { next_cw = cws[round + 1]; next_tree = trees[round + 1]; }
        } else {
            std::swap(prev_cw, next_cw);
            std::swap(prev_tree, next_tree);
        }
    }
    pd.final_off = c->rec_alloc(1);
    ZKB_CUDA(cudaMemcpyAsync(c->rec_dev + pd.final_off, eval, 4, cudaMemcpyDeviceToDevice, c->stream));
    return pd;
}

// ---- serialisation (host, after the record has been fetched) --------------------------------------
// BatchMerkleProof (pcs.rs:43-53) of `positions` from raw paths: indices and values in caller
// order; per level the digests of the siblings that are not themselves known, ascending
// (pcs.rs:299-330).  raw[i] points at the path record of positions[i].
template <class Ser>
inline void put_batch_proof(Ser& s, const std::vector<size_t>& positions, const std::vector<const u32*>& raw, u32 h) {
    s.u64le(positions.size());
    for (size_t p : positions) s.u32le((u32)p);
    s.u64le(positions.size());
    for (const u32* r : raw) s.u32le(r[0]);
    // (node index at the current level, a position that lies below it), ascending and unique
    std::vector<std::pair<size_t, size_t>> known, next;
    known.reserve(positions.size());
    for (size_t i = 0; i < positions.size(); i++) known.emplace_back(positions[i], i);
    std::sort(known.begin(), known.end());
    known.erase(std::unique(known.begin(), known.end(), [](auto& a, auto& b) { return a.first == b.first; }), known.end());
    s.u64le(h);
    std::vector<const u32*> lvl;
    for (u32 k = 0; k < h; k++) {
        lvl.clear();
        next.clear();
        for (size_t i = 0; i < known.size(); i++) {
            const size_t node = known[i].first;
            // the sibling, if known, is the neighbour in the sorted list
            const bool sib_known = (node & 1) ? (i > 0 && known[i - 1].first == node - 1) : (i + 1 < known.size() && known[i + 1].first == node + 1);
            if (!sib_known) lvl.push_back(k == 0 ? raw[known[i].second] + 1 : raw[known[i].second] + 2 + 4 * (size_t)(k - 1));
            if (next.empty() || next.back().first != (node >> 1)) next.emplace_back(node >> 1, known[i].second);
        }
        s.u64le(lvl.size());
        for (const u32* d : lvl) {
            if (k == 0) { s.u32le(d[0]); s.u32le(0); s.u32le(0); s.u32le(0); }     // hash_leaf of the sibling value
            else { s.u32le(d[0]); s.u32le(d[1]); s.u32le(d[2]); s.u32le(d[3]); }
        }
        known.swap(next);
    }
}
template <class Ser>
inline void put_digest(Ser& s, const u32* d) { for (int i = 0; i < 4; i++) s.u32le(d[i]); }

// bincode(BasefoldCommitment) (basefold.rs:39-47)
template <class Ser>
inline void put_basefold_commitment(Ser& s, const u32* rec_host, const BfPending& pd) {
    put_digest(s, rec_host + pd.root_off);
    s.u64le(pd.num_coeffs);
    s.u64le(pd.log_n);
}
// bincode(BasefoldOpeningProof) (basefold.rs:50-64)
template <class Ser>
inline void put_basefold_proof(Ser& s, const u32* rec_host, const BfPending& pd) {
    const u32 log_n = pd.log_n;
    s.u64le(log_n);
    for (u32 r = 0; r < log_n; r++) put_digest(s, rec_host + pd.round_off[r]);
    s.u64le(log_n);
    for (u32 r = 0; r < log_n; r++) {
        const u32 h_prev = log_n + 1 - r, h_fold = h_prev - 1;
        const u32* rec = rec_host + pd.round_off[r];
        const u32* idx = rec + 4;
        const size_t prev_half = size_t(1) << (h_prev - 1);
        const size_t pw_prev = 2 + 4 * (size_t)(h_prev - 1), pw_fold = 2 + 4 * (size_t)(h_fold - 1);
        const u32* out_prev = rec + 4 + BF_QUERIES;
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
    s.u32le(rec_host[pd.final_off]);
    s.u64le(0);                                   // final_coeffs: empty
}

}  // namespace zkb
