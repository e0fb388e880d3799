// C ABI, part 3: resident Qwen-style layers (weights uploaded and committed once, as the
// reference's server preload does, rust/zk_ml_prover/src/server.rs:46-94), forward pass and
// layer proof.  Included by zkb200.cu.

extern "C" {

int32_t zkb_qwen_layer_create(zkb_ctx* c, const uint64_t dims[7], const uint32_t* const weights[10], const uint32_t* silu_table_dev,
                              const uint32_t* sigmoid_table_dev, uint32_t n_table, zkb_qwen_layer** out) {
    if (!c || !dims || !weights || !silu_table_dev || !sigmoid_table_dev || !out) return ZKB_E_ARG;
    *out = nullptr;
    zkb_qwen_layer* L = new (std::nothrow) zkb_qwen_layer();
    if (!L) return ZKB_E_CUDA;
    try {
        c->use();
        L->ctx = c;
        QwenDims& d = L->dm;
        d.d_model = (u32)dims[0]; d.d_ff = (u32)dims[1]; d.nq = (u32)dims[2]; d.nkv = (u32)dims[3]; d.d_head = (u32)dims[4];
        d.v_heads = (u32)dims[5]; d.v_d_head = (u32)dims[6];
        if (!d.d_model || !d.d_ff || !d.nq || !d.nkv || !d.d_head || (d.nq % d.nkv)) throw ArgFail{ZKB_E_ARG, "bad layer dimensions"};
        if (n_table != 65536 && n_table != 256) throw ArgFail{ZKB_E_ARG, "table must have 65536 or 256 entries"};
        L->silu = silu_table_dev; L->sigmoid = sigmoid_table_dev; L->n_table = n_table;
        const size_t dm = d.d_model, aod = d.aod();
        const size_t lens[W_COUNT] = {dm, (size_t)d.q_dim() * dm, (size_t)d.k_dim() * dm, (size_t)d.v_dim() * dm, dm * aod, aod * dm,
                                      dm, (size_t)d.d_ff * dm, (size_t)d.d_ff * dm, dm * d.d_ff};
        for (int i = 0; i < W_COUNT; i++) {
            if (!weights[i]) throw ArgFail{ZKB_E_ARG, "null weight tensor"};
            L->w_len[i] = lens[i];
            ZKB_CUDA(cudaMalloc(&L->w[i], (lens[i] + 4) * 4));
            ZKB_CUDA(cudaMemcpyAsync(L->w[i], weights[i], lens[i] * 4, cudaMemcpyHostToDevice, c->stream));
        }
        // commit_qwen_layer (qwen.rs:148-161): blake3 of each unpadded matrix
        ZKB_CUDA(cudaEventCreateWithFlags(&L->fwd_done, cudaEventDisableTiming));
        ZKB_CUDA(cudaEventCreateWithFlags(&L->own_idle, cudaEventDisableTiming));
        ZKB_CUDA(cudaMalloc(&L->roots_dev, 64 * 4));
        ZKB_CUDA(cudaMalloc(&L->seed_dev, 128));
        ZKB_CUDA(cudaHostAlloc(&L->seed_host, 128, cudaHostAllocDefault));
        static const int widx[8] = {W_Q, W_K, W_V, W_O, W_GPROJ, W_GATE, W_UP, W_DOWN};
        for (int i = 0; i < 8; i++) {
            commit_large(c, b3_prefix("weights", 7), L->w[widx[i]], L->w_len[widx[i]], L->roots_dev + 8 * i);
            ZKB_CUDA(cudaStreamSynchronize(c->stream));
            c->scratch_reset();
        }
        ZKB_CUDA(cudaMemcpyAsync(L->roots_host, L->roots_dev, 256, cudaMemcpyDeviceToHost, c->stream));
        // trace buffers, each padded to a power of two (zero tails)
        const size_t dmp = pad_pow2(dm), aodp = pad_pow2(aod), dffp = pad_pow2(d.d_ff);
        const size_t qp = pad_pow2(d.q_dim()), kp = pad_pow2(d.k_dim()), vp = pad_pow2(d.v_dim());
        const size_t total = 8 * dmp + 2 * dmp + qp + kp + vp + 5 * aodp + 6 * dffp + 64;
        ZKB_CUDA(cudaMalloc(&L->trace_block, total * 4));
        ZKB_CUDA(cudaMemsetAsync(L->trace_block, 0, total * 4, c->stream));
        u32* p = L->trace_block;
        auto take = [&](size_t n) { u32* r = p; p += n; return r; };
        L->x = take(dmp); L->norm1_x = take(dmp); L->norm1_out = take(dmp); L->gated_out = take(dmp); L->h = take(dmp);
        L->norm2_x = take(dmp); L->norm2_out = take(dmp); L->down = take(dmp); L->out = take(dmp); take(dmp);
        L->q = take(qp); L->k = take(kp); L->v = take(vp);
        L->attn_out = take(aodp); L->g_raw = take(aodp); L->g_q = take(aodp); L->g_sig = take(aodp); L->gated_attn = take(aodp);
        L->gate_raw = take(dffp); L->gate_q = take(dffp); L->gate_silu = take(dffp); L->up = take(dffp); L->swiglu = take(dffp); take(dffp);
        L->n1_scalars = take(8); L->n2_scalars = take(8);
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    } catch (const CudaFail& e) {
        c->err = e.msg;
        zkb_qwen_layer_destroy(L);
        return ZKB_E_CUDA;
    } catch (const ArgFail& e) {
        c->err = e.msg;
        zkb_qwen_layer_destroy(L);
        return e.code;
    }
    *out = L;
    return ZKB_OK;
}

void zkb_qwen_layer_destroy(zkb_qwen_layer* L) {
    if (!L) return;
    if (L->ctx) {
        cudaSetDevice(L->ctx->device);
        cudaStreamSynchronize(L->ctx->stream);
    }
    for (int i = 0; i < W_COUNT; i++) if (L->w[i]) cudaFree(L->w[i]);
    if (L->fwd_done) cudaEventDestroy(L->fwd_done);
    if (L->own_idle) cudaEventDestroy(L->own_idle);
    qwen_graph_drop(L);
    if (L->seed_dev) cudaFree(L->seed_dev);
    if (L->seed_host) cudaFreeHost(L->seed_host);
    if (L->roots_dev) cudaFree(L->roots_dev);
    if (L->trace_block) cudaFree(L->trace_block);
    delete L->pending;
    delete L;
}

// Replay of the captured launch sequence on (default) or off: with it off every proof is
// enqueued launch by launch.
int32_t zkb_qwen_layer_use_graph(zkb_qwen_layer* L, int32_t on) {
    if (!L) return ZKB_E_ARG;
    L->use_graph = on != 0;
    return ZKB_OK;
}
// What the next zkb_qwen_layer_prove_begin will do: 0 = enqueue launch by launch, 1 = capture the
// launch sequence into a graph (slower once; callers that drive several layers from several
// threads may prefer to let captures happen one at a time), 2 = replay the captured graph.
int32_t zkb_qwen_layer_graph_state(const zkb_qwen_layer* L) {
    if (!L || !L->use_graph || L->ctx->profile) return 0;
    if (L->graph_exec && L->graph_epoch == L->ctx->arena_epoch && L->graph_bind == L->bind_mode && L->graph_hash == L->node_hash) return 2;
    return (L->proofs_enqueued >= 1 && L->eager_epoch == L->ctx->arena_epoch && L->capture_failures < 3) ? 1 : 0;
}
// Weight binding used by the layer's eight matmul proofs from now on.
int32_t zkb_qwen_layer_set_binding(zkb_qwen_layer* L, int32_t bind_mode, int32_t node_hash) {
    if (!L || bind_mode < BIND_BLAKE3 || bind_mode > BIND_PCS_FULL || (node_hash != NODE_BLAKE3 && node_hash != NODE_AES_MMO)) return ZKB_E_ARG;
    L->bind_mode = bind_mode;
    L->node_hash = node_hash;
    return ZKB_OK;
}

int32_t zkb_qwen_layer_commitments(zkb_qwen_layer* L, uint8_t roots[256]) {
    if (!L || !roots) return ZKB_E_ARG;
    memcpy(roots, L->roots_host, 256);
    return ZKB_OK;
}

// x: d_model words (host, or device when x_on_device).  y (optional): d_model words, host or
// device like x.  Keeps the trace inside the layer for the following prove call.
int32_t zkb_qwen_layer_forward(zkb_qwen_layer* L, const uint32_t* x, int32_t x_on_device, uint32_t* y, int32_t y_on_device) {
    if (!L || !x) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        clear_status(c);
        ZKB_CUDA(cudaMemcpyAsync(L->x, x, (size_t)L->dm.d_model * 4, x_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
        qwen_forward(L);
        L->fwd_on_shared = false;
        if (y) ZKB_CUDA(cudaMemcpyAsync(y, L->out, (size_t)L->dm.d_model * 4, y_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, c->stream));
        uint32_t st = c->read_status();
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
    });
}
// Asynchronous forward for a chain of layers on different contexts: the input is the previous
// layer's device-resident output (prev != NULL; this layer's stream waits for prev's forward
// through an event, the host does not) or x (host or device, prev == NULL).  Nothing is waited
// for and no status is read; errors of the forward pass surface at zkb_qwen_layer_prove_end.
// The caller must have issued prev's forward before this call.
int32_t zkb_qwen_layer_forward_async(zkb_qwen_layer* L, zkb_qwen_layer* prev, const uint32_t* x, int32_t x_on_device) {
    if (!L || (!prev && !x)) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        const size_t bytes = (size_t)L->dm.d_model * 4;
        // with a shared forward stream the kernels below go there; the context's own stream is put
        // back before returning (a context is driven by one host thread at a time)
        cudaStream_t own = c->stream;
        cudaStream_t S = L->fwd_stream ? L->fwd_stream : own;
        if (L->fwd_stream) ZKB_CUDA(cudaStreamWaitEvent(S, L->own_idle, 0));      // not before the layer's previous proof has finished with the trace
        struct Restore { zkb_ctx* c; cudaStream_t s; ~Restore() { c->stream = s; } } restore{c, own};
        c->stream = S;
        clear_status(c);               // on the stream the forward kernels run on, so that the clear cannot overtake or erase their status writes
        if (prev) {
            if (prev->dm.d_model != L->dm.d_model) throw ArgFail{ZKB_E_ARG, "layer widths differ"};
            if (!(L->fwd_stream && prev->fwd_stream == L->fwd_stream)) ZKB_CUDA(cudaStreamWaitEvent(S, prev->fwd_done, 0));
            ZKB_CUDA(cudaMemcpyAsync(L->x, prev->out, bytes, cudaMemcpyDeviceToDevice, S));
        } else {
            ZKB_CUDA(cudaMemcpyAsync(L->x, x, bytes, x_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, S));
        }
        qwen_forward(L);
        ZKB_CUDA(cudaEventRecord(L->fwd_done, S));
        L->fwd_on_shared = L->fwd_stream != nullptr;
    });
}
// Shared forward stream (see zkb_stream_create): pass NULL to go back to the layer's own stream.
int32_t zkb_qwen_layer_set_forward_stream(zkb_qwen_layer* L, void* stream) {
    if (!L) return ZKB_E_ARG;
    L->fwd_stream = (cudaStream_t)stream;
    return ZKB_OK;
}
// A stream of the highest (high_priority != 0) or default priority on the context's device.
int32_t zkb_stream_create(zkb_ctx* c, int32_t high_priority, void** out) {
    if (!c || !out) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        int lo = 0, hi = 0;
        ZKB_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        cudaStream_t s = nullptr;
        ZKB_CUDA(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, high_priority ? hi : lo));
        *out = (void*)s;
    });
}
void zkb_stream_destroy(void* stream) {
    if (stream) cudaStreamDestroy((cudaStream_t)stream);
}
// Wait for this layer's forward pass only (not for a proof queued behind it on the same
// stream) and copy its output (d_model words) to host memory.
int32_t zkb_qwen_layer_read_output(zkb_qwen_layer* L, uint32_t* y_host) {
    if (!L || !y_host) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaEventSynchronize(L->fwd_done));
        ZKB_CUDA(cudaMemcpy(y_host, L->out, (size_t)L->dm.d_model * 4, cudaMemcpyDeviceToHost));
    });
}
// Wait (on the host) until this layer's forward pass has finished on the GPU - not for a proof
// queued behind it.  Afterwards the output at zkb_qwen_layer_output_dev may be read by work on
// any stream or handed to another GPU.
int32_t zkb_qwen_layer_wait_forward(zkb_qwen_layer* L) {
    if (!L) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaEventSynchronize(L->fwd_done));
    });
}
// Device address of the layer output (d_model words), so the next layer can read it in place.
const uint32_t* zkb_qwen_layer_output_dev(const zkb_qwen_layer* L) { return L ? L->out : nullptr; }

// Enqueue the whole layer proof on the layer's context without waiting for it.
int32_t zkb_qwen_layer_prove_begin(zkb_qwen_layer* L, uint32_t layer_idx, const uint8_t input_hash[32]) {
    if (!L || !input_hash) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        qwen_prove_enqueue(L, layer_idx, input_hash);
    });
}
// Wait for the proof started by prove_begin and write QwenLayerProofEF (bincode, after
// strip_redundant) to out.
int32_t zkb_qwen_layer_prove_end(zkb_qwen_layer* L, uint8_t* out, size_t cap, size_t* len) {
    if (!L) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        uint32_t st = 0;
        std::vector<uint8_t> b = qwen_prove_finish(L, &st);
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
        rc = emit(c, b, out, cap, len);
        if (rc) return rc;
    });
}
int32_t zkb_qwen_layer_prove(zkb_qwen_layer* L, uint32_t layer_idx, const uint8_t input_hash[32], uint8_t* out, size_t cap, size_t* len) {
    int32_t rc = zkb_qwen_layer_prove_begin(L, layer_idx, input_hash);
    if (rc) return rc;
    return zkb_qwen_layer_prove_end(L, out, cap, len);
}

// verify_qwen_layer_ef_indexed (qwen.rs:932-1097): the layer object must hold the forward trace of the input
// the proof is about (zkb_qwen_layer_forward).  y_expected (d_model words, host; may be null) is compared with the
// layer's output as the reference compares its recomputed output with the claimed one.
int32_t zkb_qwen_layer_verify_begin(zkb_qwen_layer* L, uint32_t layer_idx, const uint8_t input_hash[32], const uint8_t* proof, size_t len,
                                    const uint32_t* y_expected) {
    if (!L || !input_hash || !proof) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    L->v_active = false;
    ZKB_TRY(c, {
        c->use();
        clear_status(c);
        LvResult r = qwen_verify_enqueue(L, layer_idx, input_hash, proof, len, y_expected);
        L->v_ok_dev = r.ok_dev; L->v_n_ok = r.n_ok; L->v_host_ok = r.host_ok; L->v_active = true;
    });
}
int32_t zkb_qwen_layer_verify_end(zkb_qwen_layer* L, int32_t* accepted) {
    if (!L || !accepted) return ZKB_E_ARG;
    *accepted = 0;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        if (!L->v_active) throw ArgFail{ZKB_E_ARG, "zkb_qwen_layer_verify_end: no verification was begun"};
        L->v_active = false;
        std::vector<u32> flags(L->v_n_ok);
        ZKB_CUDA(cudaMemcpyAsync(flags.data(), L->v_ok_dev, (size_t)L->v_n_ok * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
        bool ok = L->v_host_ok;
        for (u32 v : flags) ok = ok && v == 1;
        *accepted = ok ? 1 : 0;
    });
}
int32_t zkb_qwen_layer_verify(zkb_qwen_layer* L, uint32_t layer_idx, const uint8_t input_hash[32], const uint8_t* proof, size_t len,
                              const uint32_t* y_expected, int32_t* accepted) {
    if (!accepted) return ZKB_E_ARG;
    *accepted = 0;
    int32_t rc = zkb_qwen_layer_verify_begin(L, layer_idx, input_hash, proof, len, y_expected);
    if (rc) return rc;
    return zkb_qwen_layer_verify_end(L, accepted);
}

}  // extern "C"
