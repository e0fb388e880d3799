// Host-side sumcheck engine: decides which launches a sumcheck needs, keeps every value a
// proof needs in a device "record" buffer that is copied back once, and offers small launch
// helpers to the protocol layer.  Nothing here synchronises with the device.
#pragma once
#include <map>
#include <mutex>
#include "context.cuh"
#include "trscript.cuh"
#include "sumcheck_pipe.cuh"
#include "prep.cuh"
#include "logup.cuh"
#include "forward.cuh"
#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace zkb {

constexpr size_t MULTI_MIN_HALF = 4096;   // below this many pairs the single-CTA tail takes over

struct KindInfo { int nt; int in_w[3]; int w; u32 mask; u32 nstored; u32 nabs; };
inline KindInfo kind_info(int kind) {
    switch (kind) {
        case ZKB_SC_PRODUCT:              return {2, {1, 1, 0}, 1, 0b0111, 3, 3};
        case ZKB_SC_TRIPLE:               return {3, {1, 1, 1}, 1, 0b1111, 4, 4};
        case ZKB_SC_PRODUCT_ONES:         return {1, {1, 0, 0}, 1, 0b0101, 2, 3};
        case ZKB_SC_PRODUCT_EF:           return {2, {1, 1, 0}, 4, 0b0101, 2, 3};
        case ZKB_SC_PRODUCT_EF_FULL:      return {2, {4, 4, 0}, 4, 0b0111, 3, 3};
        case ZKB_SC_PRODUCT_EF_MIXED:     return {2, {4, 1, 0}, 4, 0b0111, 3, 3};
        case ZKB_SC_TRIPLE_EF_FULL:       return {3, {4, 4, 4}, 4, 0b1101, 3, 4};
        case ZKB_SC_PRODUCT_ONES_EF_FULL: return {1, {4, 0, 0}, 4, 0b0101, 2, 3};
    }
    throw ArgFail{ZKB_E_ARG, "unknown sumcheck kind"};
}

// Where one sumcheck's outputs live in the record buffer (offsets in u32 words).
struct ScRec {
    int kind = 0;
    u32 nv = 0;            // static number of rounds (upper bound when dyn_off is set)
    size_t polys = 0;      // [nv][nabs][w]
    size_t chal = 0;       // [nv][w]
    size_t fin = 0;        // [3][w]
    long dyn_off = -1;     // record offset of {n_active, num_vars, n} when the round count is device-resident
};
struct ScOpts {
    bool clobber[3] = {false, false, false};   // table may be folded in place (EF inputs only)
    u32 post_squeezes = 0;
    long post_off = -1;        // record offset for the post-squeezed challenges (-1: discard)
    const u32* dyn_nv = nullptr;
    long dyn_off = -1;
    bool check_zero_sum = false;
    const ScXch* xch = nullptr;    // device copy of the exchange descriptor: `tables_dev` are this GPU's slices
    u32 xch_world = 1;
};

inline int grid_for(zkb_ctx* c, size_t items, int per_cta = 256, int ctas_per_sm = 8) {
    size_t want = (items + per_cta - 1) / per_cta;
    size_t cap = (size_t)c->sm_count * c->wide_ctas_per_sm(ctas_per_sm, ctas_per_sm < 3 ? ctas_per_sm : 3);
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}
#define ZKB_LAUNCHED(c) (c)->launched(__FILE__, __LINE__)


// fused2: product sumcheck over base tables with EF challenges whose destination tables were sized
// for the two-challenge fold (a quarter of the input): round 1 is a message-only launch and the
// first tables written are those folded with r_0 and r_1 (sc_product_base_fold2_kernel).
template <int KIND, class SrcT, class ChalT>
void run_sumcheck(zkb_ctx* c, ScTables tb, u32 num_vars, ScIO io, bool dynamic, bool fused2 = false) {
    // split over several GPUs: the tables are this GPU's slice of 2^local_vars elements
    const u32 local_vars = io.xch ? io.xch_local_vars : num_vars;
    size_t size = size_t(1) << local_vars;
    bool pending = false, in_src = true;
    u32 round = 0;
    const int per_sm = c->wide_ctas_per_sm(8, 2);
    const int max_grid = c->sm_count * per_sm < SC_MAX_GRID ? c->sm_count * per_sm : SC_MAX_GRID;
    c->prof_used = 0;
    c->prof_mark();
    while (!dynamic && round < local_vars) {
        size_t half = pending ? size / 4 : size / 2;
        if (half < MULTI_MIN_HALF) break;
        size_t want = (half + 255) / 256;
        int grid = (int)(want < (size_t)max_grid ? want : (size_t)max_grid);
        // base-field tables of a product sumcheck: vectorised launches (4 pair indices per thread)
        constexpr bool base_product_t = KIND == SC_PRODUCT && std::is_same<SrcT, Fp>::value;
        const bool base_product = base_product_t && ((((uintptr_t)tb.src[0]) | ((uintptr_t)tb.src[1])) & 15) == 0;   // 16-byte loads
        // the folding variant of the vectorised kernel needs 98 registers: one CTA per SM when sharing
        const size_t vcap = (pending && c->polite) ? (size_t)c->sm_count : (size_t)max_grid;
        int vgrid = (int)(((half + 3) / 4 + 255) / 256 < vcap ? ((half + 3) / 4 + 255) / 256 : vcap);
        if (!pending) {
            if constexpr (base_product_t) {
                if (base_product) sc_product_base_kernel<ChalT, false><<<vgrid, 256, 0, c->stream>>>(tb, half, round, io);
                else sc_round_kernel<KIND, SrcT, ChalT, false><<<grid, 256, 0, c->stream>>>(tb, half, round, io);
            } else sc_round_kernel<KIND, SrcT, ChalT, false><<<grid, 256, 0, c->stream>>>(tb, half, round, io);
        } else if (in_src) {
            bool done = false;
            if constexpr (base_product_t && std::is_same<ChalT, Fe>::value) {
                if (base_product && fused2) {
                    // round 1: message only; round 2: both challenges folded in, tables shrink to a quarter
                    sc_product_base_kernel<Fe, true, false><<<vgrid, 256, 0, c->stream>>>(tb, half, round, io);
                    ZKB_LAUNCHED(c);
                    c->prof_mark();
                    round++;
                    const size_t E = size / 8;
                    const int vec = c->opt_fold2_vec ? c->opt_fold2_vec : 2;
                    const size_t want2 = (E / vec + 255) / 256;
                    const int g2 = (int)(want2 < (size_t)max_grid ? want2 : (size_t)max_grid);
                    if (vec == 1) sc_product_base_fold2_kernel<1><<<g2, 256, 0, c->stream>>>(tb, E, round, io);
                    else if (vec == 4) sc_product_base_fold2_kernel<4><<<g2, 256, 0, c->stream>>>(tb, E, round, io);
                    else sc_product_base_fold2_kernel<2><<<g2, 256, 0, c->stream>>>(tb, E, round, io);
                    size /= 2;                          // two folds in all: one here, one below
                    done = true;
                } else if (base_product) { sc_product_base_kernel<Fe, true><<<vgrid, 256, 0, c->stream>>>(tb, half, round, io); done = true; }
            }
            if (!done) sc_round_kernel<KIND, SrcT, ChalT, true><<<grid, 256, 0, c->stream>>>(tb, half, round, io);
            for (int t = 0; t < 3; t++) tb.src[t] = tb.dst[t];
            in_src = false;
            size /= 2;
        } else {
            sc_round_kernel<KIND, ChalT, ChalT, true><<<grid, 256, 0, c->stream>>>(tb, half, round, io);
            size /= 2;
        }
        ZKB_LAUNCHED(c);
        c->prof_mark();
        pending = true;
        round++;
    }
    // product sumchecks over EF tables: the tail that overlaps the table work with the hash chain
    constexpr bool pipe_t = KIND == SC_PRODUCT && std::is_same<ChalT, Fe>::value;
    const bool pipe = pipe_t && !c->opt_plain_tail && !io.xch && !dynamic && !io.dyn_nv && (!in_src || std::is_same<SrcT, Fe>::value);
    if (pipe) {
        if constexpr (pipe_t) sc_tail_product_pipe_kernel<<<1, c->pipe_threads(PIPE_THREADS), 0, c->stream>>>(tb, size, round, num_vars, pending ? 1 : 0, io);
    } else if (in_src)
        sc_tail_kernel<KIND, SrcT, ChalT><<<1, c->single_cta_threads(), 0, c->stream>>>(tb, size, round, num_vars, pending ? 1 : 0, io);
    else
        sc_tail_kernel<KIND, ChalT, ChalT><<<1, c->single_cta_threads(), 0, c->stream>>>(tb, size, round, num_vars, 1, io);
    ZKB_LAUNCHED(c);
    c->prof_mark();
    ZKB_CUDA(cudaGetLastError());
}

__global__ void widen_kernel(const u32* __restrict__ in, Fe* out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        st_fe(out + i, Fe{in[i], 0, 0, 0});
}

// Enqueue one sumcheck over device tables; every round message, challenge and final value goes
// to the context's record buffer.  Tables not marked clobber are left untouched.
inline ScRec sumcheck_enqueue(zkb_ctx* c, TrState* tr, int kind, const u32* const* tables_dev, u32 num_vars, const ScOpts& o = ScOpts()) {
    KindInfo ki = kind_info(kind);
    if (num_vars < 1 || num_vars > 34) throw ArgFail{ZKB_E_ARG, "num_vars out of range"};
    u32 log_world = 0;
    while ((1u << log_world) < o.xch_world) log_world++;
    if (o.xch && ((1u << log_world) != o.xch_world || num_vars < log_world + 1 || o.dyn_nv))
        throw ArgFail{ZKB_E_ARG, "split sumcheck: world must be a power of two below 2^num_vars, static round count"};
    const u32 local_vars = o.xch ? num_vars - log_world : num_vars;
    const size_t n = size_t(1) << local_vars;      // elements per table held by this GPU
    const bool ef_inputs = ki.in_w[0] == 4;
    ScTables tb{};
    // product sumcheck over 16-byte aligned base tables with EF challenges, at least 2^15 elements:
    // the two-challenge fold applies and the folded tables need a quarter of the input length
    const bool fused2 = kind == ZKB_SC_PRODUCT_EF && !o.dyn_nv && local_vars >= 15 && !c->opt_no_fused2 &&
                        ((((uintptr_t)tables_dev[0]) | ((uintptr_t)tables_dev[1])) & 15) == 0;
    const size_t dst_elems = fused2 ? n / 4 : (n / 2 > 2 ? n / 2 : 2);
    for (int t = 0; t < ki.nt; t++) {
        tb.src[t] = tables_dev[t];
        if (o.clobber[t] && ki.in_w[t] == 4) tb.dst[t] = const_cast<u32*>(tables_dev[t]);
        else tb.dst[t] = c->scratch(dst_elems * 4 * ki.w);
    }
    if (kind == ZKB_SC_PRODUCT_EF_MIXED) {      // widen g once; then it is PRODUCT_EF_FULL with the same message layout
        Fe* g = (Fe*)c->scratch(n * 16);
        widen_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(tables_dev[1], g, n);
        ZKB_LAUNCHED(c);
        tb.src[1] = g;
        tb.dst[1] = g;
    }
    (void)ef_inputs;
    ScRec r;
    r.kind = kind; r.nv = num_vars; r.dyn_off = o.dyn_off;
    r.polys = c->rec_alloc((size_t)num_vars * ki.nabs * ki.w);
    r.chal = c->rec_alloc((size_t)num_vars * ki.w);
    r.fin = c->rec_alloc(3 * (size_t)ki.w);
    ScIO io{};
    io.tr = tr; io.partials = c->partials; io.counter = c->counter;
    io.polys = c->rec_dev + r.polys; io.chal = c->rec_dev + r.chal; io.fin = c->rec_dev + r.fin;
    io.dyn_nv = o.dyn_nv; io.status = c->status;
    io.post_squeezes = o.post_squeezes;
    io.post_out = o.post_off >= 0 ? c->rec_dev + o.post_off : nullptr;
    io.check_zero_sum = o.check_zero_sum ? 1u : 0u;
    io.xch = o.xch; io.xch_local_vars = local_vars;
    const bool dyn = o.dyn_nv != nullptr;
    switch (kind) {
        case ZKB_SC_PRODUCT:              run_sumcheck<SC_PRODUCT, Fp, Fp>(c, tb, num_vars, io, dyn); break;
        case ZKB_SC_TRIPLE:               run_sumcheck<SC_TRIPLE, Fp, Fp>(c, tb, num_vars, io, dyn); break;
        case ZKB_SC_PRODUCT_ONES:         run_sumcheck<SC_ONES, Fp, Fp>(c, tb, num_vars, io, dyn); break;
        case ZKB_SC_PRODUCT_EF:           run_sumcheck<SC_PRODUCT, Fp, Fe>(c, tb, num_vars, io, dyn, fused2); break;
        case ZKB_SC_PRODUCT_EF_FULL:
        case ZKB_SC_PRODUCT_EF_MIXED:     run_sumcheck<SC_PRODUCT, Fe, Fe>(c, tb, num_vars, io, dyn); break;
        case ZKB_SC_TRIPLE_EF_FULL:       run_sumcheck<SC_TRIPLE, Fe, Fe>(c, tb, num_vars, io, dyn); break;
        case ZKB_SC_PRODUCT_ONES_EF_FULL: run_sumcheck<SC_ONES, Fe, Fe>(c, tb, num_vars, io, dyn); break;
    }
    return r;
}

// ---- small launch helpers -------------------------------------------------------------------
// Dynamic shared memory that a single-CTA kernel on the hash chain asks for although it uses none of it: no CTA of
// another context's kernel that needs shared memory of its own then shares the SM (its instruction cache, its L1) with
// the chain.  Measured with the transcript scripts alone on the 32-layer 4B-shape step: 27.45 -> 26.74 ms; a lone
// layer 17.63 -> 17.47 ms.  (The tails already fill an SM's register file.)
constexpr size_t EXCLUSIVE_SMEM = 200 * 1024;
template <class K>
inline size_t exclusive_smem(K kernel, zkb_ctx* c) {
    if (c->opt_shared_sm == 1) return 0;
    const size_t want = c->opt_shared_sm >= 16 ? (size_t)c->opt_shared_sm * 1024 : EXCLUSIVE_SMEM;
    const int device = c->device;
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, bool> done;
    std::lock_guard<std::mutex> g(mu);
    auto key = std::make_pair((const void*)kernel, device);
    if (!done[key]) {
        ZKB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        done[key] = true;
    }
    return want;
}
struct ScriptBuilder {
    TrScript s{};
    u32 inl_used = 0;
    void bytes(const void* p, size_t n) {
        if (s.nops >= TRSCRIPT_MAX_OPS || inl_used + n > TRSCRIPT_INLINE) throw ArgFail{ZKB_E_TOO_LARGE, "transcript script too long"};
        memcpy(s.inl + inl_used, p, n);
        s.ops[s.nops++] = TrOp{TROP_BYTES, (u32)n, 0, inl_used, nullptr, nullptr};
        inl_used += (u32)n;
    }
    void str(const char* z) { bytes(z, strlen(z)); }
    void word(u32 v) { bytes(&v, 4); }
    void push(TrOp op) {
        if (s.nops >= TRSCRIPT_MAX_OPS) throw ArgFail{ZKB_E_TOO_LARGE, "transcript script too long"};
        s.ops[s.nops++] = op;
    }
    void words_dev(const u32* p, u32 n, u32 pad = 0) { push(TrOp{TROP_WORDS_DEV, n, pad > n ? pad : n, 0, p, nullptr}); }
    void pairs_dev(const u32* a, const u32* b, u32 n) { push(TrOp{TROP_PAIRS_DEV, n, 0, 0, a, b}); }
    void squeeze(u32* dst, u32 n) { push(TrOp{TROP_SQUEEZE, n, 0, 0, dst, nullptr}); }
    void bytes_dev_n(const u32* p) { push(TrOp{TROP_BYTES_DEV_N, 0, 0, 0, p, nullptr}); }
    void run(zkb_ctx* c, TrState* tr) {
        if (!s.nops) return;
        tr_script_kernel<<<1, TRSCRIPT_THREADS, exclusive_smem(tr_script_kernel, c), c->stream>>>(tr, s);
        ZKB_LAUNCHED(c);
        s.nops = 0; inl_used = 0;
    }
};

inline B3Prefix b3_prefix(const void* p, size_t n) {
    B3Prefix pre{};
    if (n > 64) throw ArgFail{ZKB_E_TOO_LARGE, "blake3 prefix too long"};
    memcpy(pre.b, p, n);
    pre.len = (u32)n;
    return pre;
}
// commit_weights_fast of a device vector (at most ~2^20 words) -> 8 words at record offset;
// optionally absorbed straight into the transcript.
inline size_t commit_small(zkb_ctx* c, const u32* words, u32 n_words, const u32* n_words_dev, u32 max_words, TrState* absorb_into) {
    size_t off = c->rec_alloc(8);
    size_t max_chunks = ((size_t)max_words * 4 + 7 + 1023) / 1024 + 1;
    u32* cvs = (u32*)c->scratch(max_chunks * 32);
    b3_commit_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(b3_prefix("weights", 7), words, n_words, n_words_dev, cvs, c->rec_dev + off, absorb_into);
    ZKB_LAUNCHED(c);
    return off;
}
// blake3(prefix || words) of a large device buffer; result (8 words) written to out_dev.
inline void commit_large(zkb_ctx* c, const B3Prefix& pre, const u32* words, size_t n_words, u32* out_dev) {
    size_t total = pre.len + n_words * 4;
    size_t n_chunks = total == 0 ? 1 : (total + 1023) / 1024;
    u32* a = (u32*)c->scratch(n_chunks * 32);
    u32* b = (u32*)c->scratch(((n_chunks + 1) / 2) * 32);
    b3_chunks_kernel<<<grid_for(c, n_chunks, 128), 128, 0, c->stream>>>(pre, words, n_words, a);
    ZKB_LAUNCHED(c);
    size_t n = n_chunks;
    while (n > 1) {
        b3_merge_kernel<<<grid_for(c, (n + 1) / 2, 128), 128, 0, c->stream>>>(a, n, b);
        ZKB_LAUNCHED(c);
        u32* t = a; a = b; b = t;
        n = (n + 1) / 2;
    }
    ZKB_CUDA(cudaMemcpyAsync(out_dev, a, 32, cudaMemcpyDeviceToDevice, c->stream));
}

}  // namespace zkb
