// One Qwen3.5-style layer at seq_len = 1: resident weights, forward trace on the device, and
// the EF layer prover in the reference's transcript order.
//
//   qwen_forward_indexed               rust/zk_ml_prover/src/transformer/qwen.rs:211-325
//   prove_qwen_layer_precommitted_ef   rust/zk_ml_prover/src/transformer/qwen.rs:795-912
//   QwenLayerProofEF / strip_redundant rust/zk_ml_prover/src/transformer/qwen.rs:711-791
//   per-layer transcript seed          rust/zk_ml_prover/src/pipeline/prove.rs:166-168
#pragma once
#include "protocols2.cuh"

namespace zkb {

struct QwenDims {
    u32 d_model, d_ff, nq, nkv, d_head, v_heads, v_d_head;
    u32 v_dim() const { return (v_heads ? v_heads : nkv) * (v_d_head ? v_d_head : d_head); }
    u32 q_dim() const { return nq * d_head; }
    u32 k_dim() const { return nkv * d_head; }
    bool is_gqa() const { return nq != nkv; }
    u32 aod() const { return is_gqa() ? q_dim() : v_dim(); }
};

enum { W_NORM1 = 0, W_Q, W_K, W_V, W_O, W_GPROJ, W_NORM2, W_GATE, W_UP, W_DOWN, W_COUNT };

}  // namespace zkb

struct zkb_qwen_layer {
    zkb_ctx* ctx = nullptr;
    zkb::QwenDims dm{};
    zkb::u32* w[zkb::W_COUNT] = {};
    size_t w_len[zkb::W_COUNT] = {};
    zkb::u32* roots_dev = nullptr;        // 8 commitments x 8 words: q, k, v, o, g_proj, gate, up, down
    zkb::u32 roots_host[64] = {};
    const zkb::u32* silu = nullptr;       // table output columns (device), shared between layers
    const zkb::u32* sigmoid = nullptr;
    zkb::u32 n_table = 0;
    int bind_mode = 0, node_hash = 0;     // weight binding of the eight matmul proofs (BIND_*, NODE_*)
    // forward trace (device, each zero-padded to the next power of two)
    zkb::u32 *x = nullptr, *norm1_x = nullptr, *norm1_out = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn_out = nullptr,
             *g_raw = nullptr, *g_q = nullptr, *g_sig = nullptr, *gated_attn = nullptr, *gated_out = nullptr, *h = nullptr,
             *norm2_x = nullptr, *norm2_out = nullptr, *gate_raw = nullptr, *gate_q = nullptr, *gate_silu = nullptr, *up = nullptr,
             *swiglu = nullptr, *down = nullptr, *out = nullptr, *n1_scalars = nullptr, *n2_scalars = nullptr;
    zkb::u32* trace_block = nullptr;
    bool have_trace = false;
    cudaEvent_t fwd_done = nullptr;      // recorded after the forward kernels; the next layer's stream waits on it
    // Optional stream shared by the forward passes of a whole model (high priority, layers in order):
    // the forward chain then runs back to back, ahead of the proof kernels of earlier layers, and
    // this layer's own stream only waits for fwd_done before its proof.
    cudaStream_t fwd_stream = nullptr;
    cudaEvent_t own_idle = nullptr;      // recorded on the layer's own stream behind every enqueued proof
    bool fwd_on_shared = false;          // the last forward ran on fwd_stream: the proof has to wait for fwd_done
    // pending proof
    struct Pending;
    Pending* pending = nullptr;
    // pending verification (zkb_qwen_layer_verify_begin): the check words on the device and what the host decided while decoding
    zkb::u32* v_ok_dev = nullptr;
    zkb::u32 v_n_ok = 0;
    bool v_host_ok = false, v_active = false;
    // Transcript seed of the proof being enqueued, device-resident so that the launch sequence does
    // not depend on it: [byte count, "qwen-layer-{idx}" bytes, 32 bytes of input hash].
    zkb::u32* seed_dev = nullptr;
    zkb::u32* seed_host = nullptr;        // pinned
    // The launch sequence of a layer proof is fixed once its shapes, binding mode and arena are:
    // it is captured into a CUDA graph on the second proof and replayed afterwards.
    cudaGraphExec_t graph_exec = nullptr;
    Pending* graph_pending = nullptr;     // record offsets of the captured sequence
    size_t graph_rec_used = 0;
    uint64_t graph_launches = 0, graph_epoch = 0;
    int graph_bind = -1, graph_hash = -1;
    uint64_t proofs_enqueued = 0;
    bool use_graph = true;
    // A capture is only tried when the arena has not changed since the last proof that was enqueued launch by launch
    // (after zkb_ctx_trim, or a change of shapes, the arena first has to grow back to its final size).
    uint64_t eager_epoch = ~0ull;
    int capture_failures = 0;
};

namespace zkb {

inline size_t pad_pow2(size_t n) { return size_t(1) << log2_ceil_u(n); }

// Warps per row: enough to give every SM about 32 warps even for short matrices.
// The bulk-copy ring kernel, when asked for (ZKB_OPT_MATVEC_RING) and the shape allows it: whole rows of a multiple of 16 bytes, at most 64 KB each,
// 16-byte aligned matrices and input.  Returns false when the register-staged kernel has to run.
inline bool launch_matvec_forward_bulk(zkb_ctx* c, const MatvecBatch& mb, const u32* x, size_t n) {
    if (!c->opt_mv_ring || n % 4 || n * 4 > 65536 || n < 128 || ((uintptr_t)x & 15)) return false;
    for (u32 t = 0; t < mb.count; t++) if ((uintptr_t)mb.W[t] & 15) return false;
    MvbShape sh{};
    sh.n = (u32)n;
    sh.n_al = (u32)((n + 31) & ~size_t(31));
    sh.R = 16;
    while (sh.R > 1 && (size_t)sh.R * n * 4 > 40960) sh.R /= 2;
    const size_t stage = (size_t)sh.R * n * 4, smem_limit = 200 * 1024;
    if ((size_t)sh.n_al * 4 + 2 * stage + 1024 > smem_limit) return false;
    sh.S = (u32)((smem_limit - (size_t)sh.n_al * 4 - 1024) / stage);
    if (sh.S > 4) sh.S = 4;
    u32 n_tiles = 0;
    for (u32 t = 0; t < mb.count; t++) n_tiles += (mb.first[t + 1] - mb.first[t] + sh.R - 1) / sh.R;
    static std::mutex mu;
    static std::map<int, bool> ready;
    {
        std::lock_guard<std::mutex> g(mu);
        if (!ready[c->device]) {
            ZKB_CUDA(cudaFuncSetAttribute(matvec_forward_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            ready[c->device] = true;
        }
    }
    const u32 grid = n_tiles < (u32)c->sm_count ? n_tiles : (u32)c->sm_count;
    launch_pdl_smem(matvec_forward_bulk_kernel, dim3(grid), dim3(MVB_THREADS), mvb_smem_bytes(sh), c->stream, mb, x, sh, n_tiles, c->status);
    return true;
}
inline void launch_matvec_forward(zkb_ctx* c, const MatvecBatch& mb, const u32* x, size_t n) {
    if (launch_matvec_forward_bulk(c, mb, x, n)) return;
    const size_t m = mb.first[mb.count];
    const size_t want_warps = (size_t)c->sm_count * 32;
    int wpr = 1;
    while (wpr < 8 && m * wpr < want_warps && n / (4 * (size_t)wpr * 2) >= 128) wpr *= 2;
    const size_t rows_per_cta = 8 / wpr;
    size_t ctas = (m + rows_per_cta - 1) / rows_per_cta;
    const size_t cap = (size_t)c->sm_count * c->wide_ctas_per_sm(8, 3);
    int grid = (int)(ctas < cap ? ctas : cap);
    if (grid < 1) grid = 1;
    switch (wpr) {
        case 1: launch_pdl(matvec_forward_kernel<1>, dim3(grid), dim3(256), c->stream, mb, x, n, c->opt_mv_prefetch); break;
        case 2: launch_pdl(matvec_forward_kernel<2>, dim3(grid), dim3(256), c->stream, mb, x, n, c->opt_mv_prefetch); break;
        case 4: launch_pdl(matvec_forward_kernel<4>, dim3(grid), dim3(256), c->stream, mb, x, n, c->opt_mv_prefetch); break;
        default: launch_pdl(matvec_forward_kernel<8>, dim3(grid), dim3(256), c->stream, mb, x, n, c->opt_mv_prefetch); break;
    }
}
// y = W x for one matrix; the tail y[m..m_pad) is zeroed unless the caller keeps it zero itself.
inline void matvec_forward(zkb_ctx* c, const u32* W, const u32* x, u32 m, u32 n, u32* y, u32 m_pad, bool zero_tail = true) {
    if (zero_tail && m_pad > m) ZKB_CUDA(cudaMemsetAsync(y + m, 0, (size_t)(m_pad - m) * 4, c->stream));
    MatvecBatch mb{};
    mb.W[0] = W; mb.y[0] = y; mb.first[0] = 0; mb.first[1] = m; mb.count = 1;
    int rg = c->range_begin(ZKB_RANGE_MATVEC_FORWARD, 4.0 * m * n);
    launch_matvec_forward(c, mb, x, n);
    c->range_end(rg);
    ZKB_LAUNCHED(c);
}
// Several matrices with the same input and column count in one launch (tails must already be zero).
inline void matvec_forward_batch(zkb_ctx* c, int count, const u32* const* W, u32* const* y, const u32* m, const u32* x, u32 n) {
    MatvecBatch mb{};
    u32 rows = 0;
    for (int t = 0; t < count; t++) { mb.W[t] = W[t]; mb.y[t] = y[t]; mb.first[t] = rows; rows += m[t]; }
    mb.first[count] = rows;
    mb.count = (u32)count;
    int rg = c->range_begin(ZKB_RANGE_MATVEC_FORWARD, 4.0 * rows * n);
    launch_matvec_forward(c, mb, x, n);
    c->range_end(rg);
    ZKB_LAUNCHED(c);
}

// Forward pass; the input x (d_model words) must already be in L->x.
inline void qwen_forward(zkb_qwen_layer* L) {
    zkb_ctx* c = L->ctx;
    const QwenDims& d = L->dm;
    const u32 dm = d.d_model, dmp = (u32)pad_pow2(dm), aod = d.aod(), aodp = (u32)pad_pow2(aod), dffp = (u32)pad_pow2(d.d_ff);
    launch_pdl(rmsnorm_forward_kernel, dim3(1), dim3(c->single_cta_threads()), c->stream, (const u32*)L->x, (const u32*)L->w[W_NORM1], dm, dmp,
               L->norm1_out, L->norm1_x, L->n1_scalars, c->status, (const u32*)nullptr, (u32*)nullptr);
    ZKB_LAUNCHED(c);
    // The trace buffers were zeroed when the layer was created and nothing writes their padded
    // tails, so no launch has to clear them.  q, k, v and the gate projection share norm1_out.
    {
        const u32* Wm[4] = {L->w[W_Q], L->w[W_K], L->w[W_V], L->w[W_GPROJ]};
        u32* ym[4] = {L->q, L->k, L->v, L->g_raw};
        const u32 mm[4] = {d.q_dim(), d.k_dim(), d.v_dim(), aod};
        matvec_forward_batch(c, 4, Wm, ym, mm, L->norm1_out, dm);
    }
    if (d.is_gqa()) {
        launch_pdl(replicate_heads_kernel, dim3(grid_for(c, aodp)), dim3(256), c->stream, (const u32*)L->v, d.nq, d.nq / d.nkv, d.d_head, aodp, L->attn_out);
    } else {
        // attn_out = v (qwen.rs:272-284 with one group per head): a kernel rather than a copy, so the chain of dependent launches is not broken
        launch_pdl(replicate_heads_kernel, dim3(grid_for(c, aodp)), dim3(256), c->stream, (const u32*)L->v, aod / d.d_head, 1u, d.d_head, aodp, L->attn_out);
    }
    ZKB_LAUNCHED(c);
    unsigned long long* mx = reinterpret_cast<unsigned long long*>(L->n1_scalars + 4);   // two 8-byte slots after the scalars
    launch_pdl(requant_lookup_mul_apply_kernel, dim3(grid_for(c, aodp)), dim3(256), c->stream, (const u32*)L->g_raw, aod, aodp, mx, L->sigmoid, L->n_table,
               (const u32*)L->attn_out, L->g_q, L->g_sig, L->gated_attn, c->status);
    ZKB_LAUNCHED(c);
    matvec_forward(c, L->w[W_O], L->gated_attn, dm, aod, L->gated_out, dmp, false);
    // h = x + gated_out and the second norm in one launch
    launch_pdl(rmsnorm_forward_kernel, dim3(1), dim3(c->single_cta_threads()), c->stream, (const u32*)L->x, (const u32*)L->w[W_NORM2], dm, dmp,
               L->norm2_out, L->norm2_x, L->n2_scalars, c->status, (const u32*)L->gated_out, L->h);
    ZKB_LAUNCHED(c);
    {
        const u32* Wm[2] = {L->w[W_GATE], L->w[W_UP]};
        u32* ym[2] = {L->gate_raw, L->up};
        const u32 mm[2] = {d.d_ff, d.d_ff};
        matvec_forward_batch(c, 2, Wm, ym, mm, L->norm2_out, dm);
    }
    unsigned long long* mx2 = reinterpret_cast<unsigned long long*>(L->n2_scalars + 4);
    launch_pdl(requant_lookup_mul_apply_kernel, dim3(grid_for(c, dffp)), dim3(256), c->stream, (const u32*)L->gate_raw, d.d_ff, dffp, mx2, L->silu, L->n_table,
               (const u32*)L->up, L->gate_q, L->gate_silu, L->swiglu, c->status);
    ZKB_LAUNCHED(c);
    matvec_forward(c, L->w[W_DOWN], L->swiglu, dm, d.d_ff, L->down, dmp, false);
    launch_pdl(add_vec_kernel, dim3(grid_for(c, dmp)), dim3(256), c->stream, (const u32*)L->h, (const u32*)L->down, dm, dmp, L->out);
    ZKB_LAUNCHED(c);
    ZKB_CUDA(cudaGetLastError());
    L->have_trace = true;
}

}  // namespace zkb

struct zkb_qwen_layer::Pending {
    zkb::RmsNormRec norm1, norm2;
    zkb::MatmulRec mq, mk, mv, mo, mg, mgate, mup, mdown;
    size_t seq1 = 0;
    zkb::GateRec sig_gate, swiglu;
    zkb::AddRec res1, res2;
    size_t res1_point = 0, res2_point = 0;
};

namespace zkb {

// The launches of one layer proof; record offsets go to P.  No synchronisation, no allocation
// once the arena has its final size (so it can run under stream capture).
inline void qwen_prove_launches(zkb_qwen_layer* L, zkb_qwen_layer::Pending& P) {
    zkb_ctx* c = L->ctx;
    const QwenDims& d = L->dm;
    const u32 dm = d.d_model, aod = d.aod();
    TrState* tr = (TrState*)c->scratch(sizeof(TrState));
    tr_init_kernel<<<1, 1, 0, c->stream>>>(tr);
    ZKB_LAUNCHED(c);
    {   // Transcript::new("qwen-layer-{idx}"); absorb input hash; dims; the eight roots
        ScriptBuilder sb;
        sb.bytes_dev_n(L->seed_dev);
        sb.str("qwen-dims-v1");
        u32 dims[12] = {d.d_model, d.d_ff, d.nq, d.nkv, d.d_head, d.v_heads, d.v_d_head, d.v_dim(), d.q_dim(), d.k_dim(), aod, d.is_gqa() ? 1u : 0u};
        sb.bytes(dims, sizeof dims);
        sb.words_dev(L->roots_dev, 64);
        sb.run(c, tr);
    }
    P.norm1 = prove_rmsnorm_ef(c, tr, L->norm1_x, L->w[W_NORM1], L->norm1_out, dm, L->n1_scalars);
    P.mq = prove_matmul_succinct_ef(c, tr, L->w[W_Q], L->norm1_out, L->q, d.q_dim(), dm, L->bind_mode, L->node_hash);
    P.mk = prove_matmul_succinct_ef(c, tr, L->w[W_K], L->norm1_out, L->k, d.k_dim(), dm, L->bind_mode, L->node_hash);
    P.mv = prove_matmul_succinct_ef(c, tr, L->w[W_V], L->norm1_out, L->v, d.v_dim(), dm, L->bind_mode, L->node_hash);
    P.seq1 = c->rec_alloc(2);
    seq1_consistency_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(tr, L->attn_out, aod, log2_ceil_u(aod), L->v, d.v_dim(), log2_ceil_u(d.v_dim()),
                                                      d.is_gqa() ? 1u : 0u, log2_ceil_u(d.nkv), log2_ceil_u(d.d_head), c->rec_dev + P.seq1);
    ZKB_LAUNCHED(c);
    P.mo = prove_matmul_succinct_ef(c, tr, L->w[W_O], L->gated_attn, L->gated_out, dm, aod, L->bind_mode, L->node_hash);
    P.mg = prove_matmul_succinct_ef(c, tr, L->w[W_GPROJ], L->norm1_out, L->g_raw, aod, dm, L->bind_mode, L->node_hash);
    // prove_sigmoid_gate_ef(gate = g_q, gate_sigmoid = g_sig, input = attn_out, output = gated_attn)
    P.sig_gate = prove_gate_ef(c, tr, L->sigmoid, L->n_table, L->g_q, L->g_sig, L->attn_out, L->g_sig, L->gated_attn, aod);
    const u32 log_d = log2_ceil_u(dm);
    P.res1_point = c->rec_alloc(4 * (size_t)log_d);
    { ScriptBuilder sb; sb.squeeze(c->rec_dev + P.res1_point, 4 * log_d); sb.run(c, tr); }
    P.res1 = prove_add_ef(c, tr, L->x, L->gated_out, L->h, dm, (const Fe*)(c->rec_dev + P.res1_point), log_d);
    P.norm2 = prove_rmsnorm_ef(c, tr, L->norm2_x, L->w[W_NORM2], L->norm2_out, dm, L->n2_scalars);
    P.mgate = prove_matmul_succinct_ef(c, tr, L->w[W_GATE], L->norm2_out, L->gate_raw, d.d_ff, dm, L->bind_mode, L->node_hash);
    P.mup = prove_matmul_succinct_ef(c, tr, L->w[W_UP], L->norm2_out, L->up, d.d_ff, dm, L->bind_mode, L->node_hash);
    // prove_swiglu_ef(gate = gate_q, gate_silu, up, output = swiglu): hadamard(gate_silu, up)
    P.swiglu = prove_gate_ef(c, tr, L->silu, L->n_table, L->gate_q, L->gate_silu, L->gate_silu, L->up, L->swiglu, d.d_ff);
    P.mdown = prove_matmul_succinct_ef(c, tr, L->w[W_DOWN], L->swiglu, L->down, dm, d.d_ff, L->bind_mode, L->node_hash);
    P.res2_point = c->rec_alloc(4 * (size_t)log_d);
    { ScriptBuilder sb; sb.squeeze(c->rec_dev + P.res2_point, 4 * log_d); sb.run(c, tr); }
    P.res2 = prove_add_ef(c, tr, L->h, L->down, L->out, dm, (const Fe*)(c->rec_dev + P.res2_point), log_d);
    ZKB_CUDA(cudaGetLastError());
}

inline void qwen_graph_drop(zkb_qwen_layer* L);

// Enqueue the whole layer proof (no synchronisation): eagerly the first time (the arena grows to
// its final size), captured into a graph the second time, replayed from then on.
inline void qwen_prove_enqueue_inner(zkb_qwen_layer* L, u32 layer_idx, const uint8_t input_hash[32]) {
    zkb_ctx* c = L->ctx;
    if (!L->have_trace) throw ArgFail{ZKB_E_ARG, "zkb_qwen_layer_prove: run the forward pass first"};
    if (L->fwd_on_shared) {            // the forward ran on the shared stream: order the proof behind it
        ZKB_CUDA(cudaStreamWaitEvent(c->stream, L->fwd_done, 0));
        L->fwd_on_shared = false;
    }
    {   // seed block -> device
        char seed[48];
        int n = snprintf(seed, sizeof seed, "qwen-layer-%u", layer_idx);
        unsigned char* b = reinterpret_cast<unsigned char*>(L->seed_host + 1);
        memset(L->seed_host, 0, 128);
        memcpy(b, seed, (size_t)n);
        memcpy(b + n, input_hash, 32);
        L->seed_host[0] = (u32)n + 32;
        ZKB_CUDA(cudaMemcpyAsync(L->seed_dev, L->seed_host, 128, cudaMemcpyHostToDevice, c->stream));
    }
    c->rec_reset();
    c->scratch_reset();
    delete L->pending;
    L->pending = nullptr;
    const bool graph_ok = L->use_graph && !c->profile;
    if (graph_ok && L->graph_exec && L->graph_epoch == c->arena_epoch && L->graph_bind == L->bind_mode && L->graph_hash == L->node_hash) {
        L->pending = new zkb_qwen_layer::Pending(*L->graph_pending);
        c->rec_used = L->graph_rec_used;
        ZKB_CUDA(cudaGraphLaunch(L->graph_exec, c->stream));
        c->launches += L->graph_launches;
        L->proofs_enqueued++;
        return;
    }
    c->trace_clear();                  // a new launch sequence starts (replays above keep the captured one)
    L->pending = new zkb_qwen_layer::Pending();
    if (!graph_ok) {                   // profiling or graphs switched off: launch by launch, keep any captured graph
        qwen_prove_launches(L, *L->pending);
        L->proofs_enqueued++;
        return;
    }
    qwen_graph_drop(L);
    if (L->proofs_enqueued >= 1 && L->eager_epoch == c->arena_epoch && L->capture_failures < 3) {
        const uint64_t launches0 = c->launches;
        cudaGraph_t graph = nullptr;
        ZKB_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
        c->capturing = true;               // only once the capture is really open: a failed begin must not leave the flag set
        bool fine = true;
        std::string why;
        try {
            qwen_prove_launches(L, *L->pending);
        } catch (const CudaFail& e) { fine = false; why = e.msg; }
        catch (const ArgFail& e) { fine = false; why = e.msg; }
        cudaError_t ce = cudaStreamEndCapture(c->stream, &graph);
        c->capturing = false;
        if (fine && ce == cudaSuccess && graph) {
            cudaGraphExec_t exec = nullptr;
            ce = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (ce == cudaSuccess) {
                L->graph_exec = exec;
                L->graph_pending = new zkb_qwen_layer::Pending(*L->pending);
                L->graph_rec_used = c->rec_used;
                L->graph_launches = c->launches - launches0;
                L->graph_epoch = c->arena_epoch;
                L->graph_bind = L->bind_mode; L->graph_hash = L->node_hash;
                ZKB_CUDA(cudaGraphLaunch(exec, c->stream));
                L->proofs_enqueued++;
                return;
            }
        } else if (graph) {
            cudaGraphDestroy(graph);
        }
        // capture did not work out (e.g. the arena had to grow): clear the sticky error, go on eagerly; a later proof tries again
        cudaGetLastError();
        L->capture_failures++;
        c->launches = launches0;
        c->rec_reset();
        c->scratch_reset();
        c->trace_clear();
        delete L->pending;
        L->pending = new zkb_qwen_layer::Pending();
    }
    qwen_prove_launches(L, *L->pending);
    L->eager_epoch = c->arena_epoch;
    L->proofs_enqueued++;
}
inline void qwen_prove_enqueue(zkb_qwen_layer* L, u32 layer_idx, const uint8_t input_hash[32]) {
    qwen_prove_enqueue_inner(L, layer_idx, input_hash);
    // a later forward on a shared stream must not overwrite the trace while this proof reads it
    ZKB_CUDA(cudaEventRecord(L->own_idle, L->ctx->stream));
}
inline void qwen_graph_drop(zkb_qwen_layer* L) {
    if (L->graph_exec) { cudaGraphExecDestroy(L->graph_exec); L->graph_exec = nullptr; }
    delete L->graph_pending;
    L->graph_pending = nullptr;
}

// Wait for the enqueued proof and serialise QwenLayerProofEF (after strip_redundant) as bincode.
inline std::vector<uint8_t> qwen_prove_finish(zkb_qwen_layer* L, uint32_t* status_out) {
    zkb_ctx* c = L->ctx;
    if (!L->pending) throw ArgFail{ZKB_E_ARG, "no proof enqueued"};
    c->rec_fetch();
    *status_out = c->read_status();
    auto& P = *L->pending;
    const QwenDims& d = L->dm;
    Ser s;
    s.rec = c->rec_host;
    put_rmsnorm(s, P.norm1, true);
    put_matmul(s, P.mq, true); put_matmul(s, P.mk, true); put_matmul(s, P.mv, true);
    // RowAttentionProof {row_proofs: [], num_heads, seq_len, d_head, seq1_consistency: Some{..}}
    s.u64le(0); s.u64le(d.nq); s.u64le(1); s.u64le(d.d_head);
    s.u8(1); s.u32le(s.rec[P.seq1]); s.u32le(s.rec[P.seq1 + 1]); s.u8(d.is_gqa() ? 1 : 0);
    put_matmul(s, P.mo, true); put_matmul(s, P.mg, true);
    put_gate(s, P.sig_gate, true);
    put_add(s, P.res1, true);
    put_rmsnorm(s, P.norm2, true);
    put_matmul(s, P.mgate, true); put_matmul(s, P.mup, true);
    put_gate(s, P.swiglu, true);
    put_matmul(s, P.mdown, true);
    put_add(s, P.res2, true);
    for (int i = 0; i < 8; i++) {       // weight commitments of the unpadded matrices
        static const int widx[8] = {W_Q, W_K, W_V, W_O, W_GPROJ, W_GATE, W_UP, W_DOWN};
        for (int k = 0; k < 8; k++) s.u32le(L->roots_host[8 * i + k]);
        u64 nw = L->w_len[widx[i]];
        s.u64le(nw);
        s.u64le(nw <= 1 ? 1 : log2_ceil_u(nw));
        s.u32le(0);
    }
    delete L->pending;
    L->pending = nullptr;
    return s.b;
}

}  // namespace zkb
