// C ABI, part 2: field helpers, commitments, the matrix kernels and the sub-protocol provers.
// Host-pointer entry points: inputs are copied to the device inside the call, the proof comes
// back as the reference's bincode bytes.  Included by zkb200.cu inside extern "C".

namespace {

// Upload `n` words and zero-pad to `n_pad` in scratch memory.
u32* up_pad(zkb_ctx* c, const uint32_t* host, size_t n, size_t n_pad) {
    if (n_pad < n) n_pad = n;
    u32* d = (u32*)c->scratch((n_pad ? n_pad : 1) * 4);
    if (n) ZKB_CUDA(cudaMemcpyAsync(d, host, n * 4, cudaMemcpyHostToDevice, c->stream));
    if (n_pad > n) ZKB_CUDA(cudaMemsetAsync(d + n, 0, (n_pad - n) * 4, c->stream));
    return d;
}
int32_t emit(zkb_ctx* c, const std::vector<uint8_t>& b, uint8_t* out, size_t cap, size_t* len) {
    if (len) *len = b.size();
    if (b.size() > cap || !out) { c->err = "output buffer too small"; return ZKB_E_TOO_LARGE; }
    memcpy(out, b.data(), b.size());
    return ZKB_OK;
}
int32_t status_to_code(zkb_ctx* c, uint32_t st) {
    if (st == 0) return ZKB_OK;
    switch (st) {
        case ST_LOGUP_IDENTITY: c->err = "LogUp identity failed — invalid lookups"; return ZKB_E_LOGUP_IDENTITY;
        case ST_ALPHA_COLLISION: c->err = "alpha collision with lookup encoding"; return ZKB_E_ALPHA_COLLISION;
        case ST_NOT_QR: c->err = "rmsnorm_forward: could not find QR perturbation in 200 attempts"; return ZKB_E_NOT_QR;
        case ST_LOOKUP_KEY: c->err = "lookup_fast: key not found"; return ZKB_E_ARG;
        case ST_ATT_ZERO_SUM: c->err = "attention: the softmax denominator is zero"; return ZKB_E_ARG;
        case ST_COPY_TIMEOUT: c->err = "forward matvec: a bulk copy into shared memory did not complete within its wait limit"; return ZKB_E_CUDA;
    }
    c->err = "device status " + std::to_string(st);
    return ZKB_E_CUDA;
}
void clear_status(zkb_ctx* c) { ZKB_CUDA(cudaMemsetAsync(c->status, 0, 4, c->stream)); }

}  // namespace

extern "C" {

int32_t zkb_commit_weights_fast(zkb_ctx* c, const uint32_t* w, size_t n, int32_t on_device, uint8_t root[32]) {
    if (!c || (!w && n) || !root) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const u32* d = on_device ? w : up_pad(c, w, n, n);
        u32* out = (u32*)c->scratch(32);
        commit_large(c, b3_prefix("weights", 7), d, n, out);
        ZKB_CUDA(cudaMemcpyAsync(root, out, 32, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_eq_evals(zkb_ctx* c, const uint32_t* r, uint32_t k, int32_t ef, uint32_t* out) {
    if (!c || (!r && k) || !out || k > 28) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const int w = ef ? 4 : 1;
        size_t n = size_t(1) << k;
        u32* dr = up_pad(c, r, (size_t)k * w, (size_t)k * w + 4);
        u32* de = (u32*)c->scratch(n * 4 * w);
        if (ef) eq_evals_kernel<Fe><<<grid_for(c, n), 256, 0, c->stream>>>((const Fe*)dr, k, (Fe*)de);
        else eq_evals_kernel<Fp><<<grid_for(c, n), 256, 0, c->stream>>>((const Fp*)dr, k, (Fp*)de);
        ZKB_LAUNCHED(c);
        ZKB_CUDA(cudaMemcpyAsync(out, de, n * 4 * w, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_fold_eq_matvec(zkb_ctx* c, const uint32_t* W, size_t m, size_t n, const uint32_t* r, uint32_t log_m, int32_t ef,
                           int32_t w_on_device, uint32_t* out) {
    if (!c || !W || !r || !out || m == 0 || n == 0 || (size_t(1) << log_m) < m) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const int w = ef ? 4 : 1;
        const size_t m_pad = size_t(1) << log_m, n_pad = size_t(1) << log2_ceil_u(n);
        if (w_on_device && n % 4 == 0) need_align16(W, "W");
        const u32* dW = w_on_device ? W : up_pad(c, W, m * n, m * n);
        u32* dr = up_pad(c, r, (size_t)log_m * w, (size_t)log_m * w + 4);
        u32* eq = (u32*)c->scratch(m_pad * 4 * w);
        if (ef) eq_evals_kernel<Fe><<<grid_for(c, m_pad), 256, 0, c->stream>>>((const Fe*)dr, log_m, (Fe*)eq);
        else eq_evals_kernel<Fp><<<grid_for(c, m_pad), 256, 0, c->stream>>>((const Fp*)dr, log_m, (Fp*)eq);
        ZKB_LAUNCHED(c);
        u32* res = (u32*)c->scratch(n_pad * w * 4);
        size_t rows_per = 0;
        dim3 grid = fold_launch_dims(c->sm_count, m, n, &rows_per);
        u32* slabs = (u32*)c->scratch((size_t)grid.y * n * w * 4 + 16);
        if (ef) {
            fold_eq_matvec_kernel<4, false><<<fold_grid(grid, c->sm_count, c->polite), FOLD_THREADS, 0, c->stream>>>(dW, m, n, eq, rows_per, nullptr, slabs);
            fold_finalize_partials_kernel<4><<<grid_for(c, n_pad * 4), 256, 0, c->stream>>>(slabs, grid.y, n, n_pad, res);
        } else {
            fold_eq_matvec_kernel<1, false><<<fold_grid(grid, c->sm_count, c->polite), FOLD_THREADS, 0, c->stream>>>(dW, m, n, eq, rows_per, nullptr, slabs);
            fold_finalize_partials_kernel<1><<<grid_for(c, n_pad), 256, 0, c->stream>>>(slabs, grid.y, n, n_pad, res);
        }
        c->launches += 2;
        ZKB_CUDA(cudaGetLastError());
        ZKB_CUDA(cudaMemcpyAsync(out, res, n_pad * w * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_matvec_forward(zkb_ctx* c, const uint32_t* W, const uint32_t* x, size_t m, size_t n, int32_t w_on_device, uint32_t* y) {
    if (!c || !W || !x || !y || m == 0 || n == 0) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        if (w_on_device && n % 4 == 0) need_align16(W, "W");
        clear_status(c);
        const u32* dW = w_on_device ? W : up_pad(c, W, m * n, m * n);
        u32* dx = up_pad(c, x, n, n + 4);
        u32* dy = (u32*)c->scratch(m * 4);
        matvec_forward(c, dW, dx, (u32)m, (u32)n, dy, (u32)m);
        ZKB_CUDA(cudaGetLastError());
        ZKB_CUDA(cudaMemcpyAsync(y, dy, m * 4, cudaMemcpyDeviceToHost, c->stream));
        uint32_t st = c->read_status();
        c->scratch_reset();
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
    });
}

int32_t zkb_prove_matmul_succinct_ef_bind(zkb_ctx* c, zkb_transcript* t, const uint32_t* W, const uint32_t* x, const uint32_t* y, size_t m,
                                          size_t n, int32_t w_on_device, int32_t bind_mode, int32_t node_hash, uint8_t* out, size_t cap,
                                          size_t* len) {
    if (!c || !t || !W || !x || !y || m == 0 || n == 0) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        const size_t n_pad = size_t(1) << log2_ceil_u(n);
        if (w_on_device && n % 4 == 0) need_align16(W, "W");
        const u32* dW = w_on_device ? W : up_pad(c, W, m * n, m * n);
        u32* dx = up_pad(c, x, n, n_pad);
        u32* dy = up_pad(c, y, m, m);
        MatmulRec R = prove_matmul_succinct_ef(c, t->dev, dW, dx, dy, (u32)m, (u32)n, bind_mode, node_hash);
        c->rec_fetch();
        Ser s; s.rec = c->rec_host;
        put_matmul(s, R, false);
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}
int32_t zkb_prove_matmul_succinct_ef(zkb_ctx* c, zkb_transcript* t, const uint32_t* W, const uint32_t* x, const uint32_t* y, size_t m,
                                     size_t n, int32_t w_on_device, uint8_t* out, size_t cap, size_t* len) {
    return zkb_prove_matmul_succinct_ef_bind(c, t, W, x, y, m, n, w_on_device, BIND_BLAKE3, NODE_BLAKE3, out, cap, len);
}

int32_t zkb_prove_matmul_succinct(zkb_ctx* c, zkb_transcript* t, const uint32_t* W, const uint32_t* x, const uint32_t* y, size_t m, size_t n,
                                  int32_t w_on_device, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || !W || !x || !y || m == 0 || n == 0) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        const size_t n_pad = size_t(1) << log2_ceil_u(n);
        if (w_on_device && n % 4 == 0) need_align16(W, "W");
        const u32* dW = w_on_device ? W : up_pad(c, W, m * n, m * n);
        u32* dx = up_pad(c, x, n, n_pad);
        u32* dy = up_pad(c, y, m, m);
        MatmulRec R = prove_matmul_succinct_base(c, t->dev, dW, dx, dy, (u32)m, (u32)n);
        c->rec_fetch();
        Ser s; s.rec = c->rec_host;
        put_matmul_base(s, R);
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}
// prove_mle_eval_bound / prove_mle_eval_no_merkle with base-field challenges.
int32_t zkb_prove_mle_eval(zkb_ctx* c, zkb_transcript* t, const uint32_t* w, size_t n, const uint32_t* point, uint32_t k,
                           const uint8_t* label, size_t label_len, const uint8_t root[32], uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || (!w && n) || !point || k < 1 || k > 30 || n > (size_t(1) << k) || (label_len && (!label || !root)) || label_len > 63) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        u32* dw = up_pad(c, w, n, size_t(1) << k);
        u32* dp = up_pad(c, point, k, (size_t)k + 4);
        u32* droot = nullptr;
        std::string lab;
        if (label_len) {
            lab.assign((const char*)label, label_len);
            droot = up_pad(c, (const uint32_t*)root, 8, 8);
        }
        EvalRec R = prove_mle_eval_base(c, t->dev, dw, dp, k, label_len ? lab.c_str() : nullptr, droot);
        c->rec_fetch();
        Ser s; s.rec = c->rec_host;
        put_eval_base(s, R);
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

// prove_hadamard (is_add = 0) / prove_add (is_add = 1) with base-field challenges.
int32_t zkb_prove_elementwise(zkb_ctx* c, zkb_transcript* t, int32_t is_add, const uint32_t* a, const uint32_t* b, const uint32_t* cv, size_t n,
                              const uint32_t* point, uint32_t k, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || !a || !b || !cv || !point || k < 1 || k > 28 || n > (size_t(1) << k)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        const size_t np = size_t(1) << k;
        u32* da = up_pad(c, a, n, np);
        u32* db = up_pad(c, b, n, np);
        u32* dc = up_pad(c, cv, n, np);
        u32* dp = up_pad(c, point, k, (size_t)k + 4);
        Ser s;
        if (is_add) {
            AddRec R = prove_add_base(c, t->dev, da, db, dc, dp, k);
            c->rec_fetch(); s.rec = c->rec_host; put_add_base(s, R);
        } else {
            HadamardRec R = prove_hadamard_base(c, t->dev, da, db, dc, dp, k);
            c->rec_fetch(); s.rec = c->rec_host; put_hadamard_base(s, R);
        }
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

int32_t zkb_prove_elementwise_ef(zkb_ctx* c, zkb_transcript* t, int32_t is_add, const uint32_t* a, const uint32_t* b, const uint32_t* cv,
                                 size_t n, const uint32_t* point, uint32_t k, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || !a || !b || !cv || !point || n == 0 || (size_t(1) << k) < n) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        const size_t n_pad = size_t(1) << k;
        u32* da = up_pad(c, a, n, n_pad); u32* db = up_pad(c, b, n, n_pad); u32* dc = up_pad(c, cv, n, n_pad);
        u32* dp = up_pad(c, point, 4 * (size_t)k, 4 * (size_t)k);
        Ser s;
        if (is_add) {
            AddRec R = prove_add_ef(c, t->dev, da, db, dc, (u32)n, (const Fe*)dp, k);
            c->rec_fetch(); s.rec = c->rec_host; put_add(s, R, false);
        } else {
            HadamardRec R = prove_hadamard_ef(c, t->dev, da, db, dc, (u32)n, (const Fe*)dp, k);
            c->rec_fetch(); s.rec = c->rec_host; put_hadamard(s, R, false);
        }
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

int32_t zkb_rmsnorm_forward(zkb_ctx* c, const uint32_t* x, const uint32_t* gamma, size_t d, uint32_t* out, uint32_t* x_used, int32_t* delta) {
    if (!c || !x || !gamma || !out || !x_used || !delta || d == 0) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        clear_status(c);
        u32* dx = up_pad(c, x, d, d); u32* dg = up_pad(c, gamma, d, d);
        u32* dout = (u32*)c->scratch(d * 4); u32* dxu = (u32*)c->scratch(d * 4); u32* sc = (u32*)c->scratch(16);
        rmsnorm_forward_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(dx, dg, (u32)d, (u32)d, dout, dxu, sc, c->status);
        ZKB_LAUNCHED(c);
        u32 h[2];
        ZKB_CUDA(cudaMemcpyAsync(out, dout, d * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaMemcpyAsync(x_used, dxu, d * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaMemcpyAsync(h, sc, 8, cudaMemcpyDeviceToHost, c->stream));
        uint32_t st = c->read_status();
        *delta = (int32_t)h[0];
        c->scratch_reset();
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
    });
}

int32_t zkb_prove_rmsnorm_ef(zkb_ctx* c, zkb_transcript* t, const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d,
                             int32_t delta, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || !x || !gamma || !y || d == 0) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        const size_t n_pad = size_t(1) << log2_ceil_u(d);
        u32* dx = up_pad(c, x, d, n_pad); u32* dg = up_pad(c, gamma, d, n_pad); u32* dy = up_pad(c, y, d, n_pad);
        uint32_t sc_h[2] = {(uint32_t)delta, 0};
        u32* sc = up_pad(c, sc_h, 2, 4);
        RmsNormRec R = prove_rmsnorm_ef(c, t->dev, dx, dg, dy, (u32)d, sc);
        c->rec_fetch();
        Ser s; s.rec = c->rec_host;
        put_rmsnorm(s, R, false);
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

int32_t zkb_prove_rmsnorm(zkb_ctx* c, zkb_transcript* t, const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d, int32_t delta,
                          uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || !x || !gamma || !y || d == 0) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        const size_t n_pad = size_t(1) << log2_ceil_u(d);
        u32* dx = up_pad(c, x, d, n_pad); u32* dg = up_pad(c, gamma, d, n_pad); u32* dy = up_pad(c, y, d, n_pad);
        uint32_t sc_h[2] = {(uint32_t)delta, 0};
        u32* sc = up_pad(c, sc_h, 2, 4);
        RmsNormRec R = prove_rmsnorm_base(c, t->dev, dx, dg, dy, (u32)d, sc);
        c->rec_fetch();
        Ser s; s.rec = c->rec_host;
        put_rmsnorm_base(s, R);
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

int32_t zkb_prove_lookup_ef(zkb_ctx* c, zkb_transcript* t, const uint32_t* table_out, size_t n_table, const uint32_t* inputs,
                            const uint32_t* outputs, size_t n, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || !table_out || !inputs || !outputs || n == 0 || (n_table != 256 && n_table != 65536)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        clear_status(c);
        u32* dt = up_pad(c, table_out, n_table, n_table);
        u32* di = up_pad(c, inputs, n, n); u32* dout = up_pad(c, outputs, n, n);
        LookupRec R = prove_lookup_ef(c, t->dev, dt, (u32)n_table, di, dout, (u32)n);
        c->rec_fetch();
        uint32_t st = c->read_status();
        c->scratch_reset();
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
        Ser s; s.rec = c->rec_host;
        put_lookup(s, R, false, inputs, outputs);
        rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

int32_t zkb_prove_lookup(zkb_ctx* c, zkb_transcript* t, const uint32_t* table_out, size_t n_table, const uint32_t* inputs,
                         const uint32_t* outputs, size_t n, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !t || !table_out || !inputs || !outputs || n == 0 || (n_table != 256 && n_table != 65536)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        c->rec_reset();
        clear_status(c);
        u32* dt = up_pad(c, table_out, n_table, n_table);
        u32* di = up_pad(c, inputs, n, n); u32* dout = up_pad(c, outputs, n, n);
        LookupRec R = prove_lookup_base(c, t->dev, dt, (u32)n_table, di, dout, (u32)n);
        c->rec_fetch();
        uint32_t st = c->read_status();
        c->scratch_reset();
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
        Ser s; s.rec = c->rec_host;
        put_lookup_base(s, R, inputs, outputs);
        rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

}  // extern "C"
