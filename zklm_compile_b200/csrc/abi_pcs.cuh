// C ABI, part 4: Merkle trees and the Basefold commitment.  Included by zkb200.cu.

namespace {

inline u32 tree_height(size_t n) { return n <= 1 ? 1 : log2_ceil_u(n); }   // pcs.rs:143-146

// Build the tree over `n` values (device pointer d); returns the node array.
uint4* build_tree(zkb_ctx* c, const u32* d, size_t n, int kind, u32* h_out) {
    if (kind != NODE_BLAKE3 && kind != NODE_AES_MMO) throw ArgFail{ZKB_E_ARG, "unknown node hash"};
    if (kind == NODE_AES_MMO) aes_tables_upload();
    const u32 h = tree_height(n);
    if (h > 30) throw ArgFail{ZKB_E_TOO_LARGE, "tree too large"};
    uint4* nodes = (uint4*)c->scratch(mk_node_count(h) * 16 + 16);
    MkFold none{};
    mk_build(c, kind, MK_VALUES, d, n, h, nodes, none);
    *h_out = h;
    return nodes;
}

}  // namespace

extern "C" {

int32_t zkb_merkle_root(zkb_ctx* c, const uint32_t* values, size_t n, int32_t on_device, int32_t node_hash, uint8_t root[16]) {
    if (!c || (!values && n) || !root) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const u32* d = on_device ? values : up_pad(c, values, n, n);
        u32 h = 0;
        uint4* nodes = build_tree(c, d, n, node_hash, &h);
        ZKB_CUDA(cudaMemcpyAsync(root, nodes + mk_layer_offset(h, h), 16, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_merkle_layers(zkb_ctx* c, const uint32_t* values, size_t n, int32_t on_device, int32_t node_hash, uint8_t* out, size_t cap,
                          size_t* len) {
    if (!c || (!values && n) || !len) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const u32 h0 = tree_height(n);
        *len = mk_node_count(h0) * 16;
        if (!out || cap < *len) throw ArgFail{ZKB_E_TOO_LARGE, "output buffer too small"};
        const u32* d = on_device ? values : up_pad(c, values, n, n);
        u32 h = 0;
        uint4* nodes = build_tree(c, d, n, node_hash, &h);
        ZKB_CUDA(cudaMemcpyAsync(out, nodes, *len, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_merkle_batch_open(zkb_ctx* c, const uint32_t* values, size_t n, int32_t on_device, int32_t node_hash, const uint64_t* indices,
                              size_t n_idx, uint8_t* out, size_t cap, size_t* len) {
    if (!c || (!values && n) || (!indices && n_idx) || !len) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const u32* d = on_device ? values : up_pad(c, values, n, n);
        u32 h = 0;
        uint4* nodes = build_tree(c, d, n, node_hash, &h);
        for (size_t i = 0; i < n_idx; i++)
            if (indices[i] >> h) throw ArgFail{ZKB_E_ARG, "opened position outside the tree"};
        const size_t pw = 2 + 4 * (size_t)(h - 1);
        c->rec_reset();
        size_t off = c->rec_alloc(n_idx * pw + 4);
        unsigned long long* pos = (unsigned long long*)c->scratch((n_idx + 1) * 8);
        if (n_idx) {
            ZKB_CUDA(cudaMemcpyAsync(pos, indices, n_idx * 8, cudaMemcpyHostToDevice, c->stream));
            mk_open_kernel<<<(unsigned)(n_idx < 256 ? n_idx : 256), 32, 0, c->stream>>>(d, n, nodes, h, pos, (u32)n_idx, c->rec_dev + off);
            ZKB_LAUNCHED(c);
        }
        c->rec_fetch();
        Ser s;
        std::vector<size_t> p(indices, indices + n_idx);
        std::vector<const u32*> raw;
        for (size_t i = 0; i < n_idx; i++) raw.push_back(c->rec_host + off + i * pw);
        put_batch_proof(s, p, raw, h);
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

int32_t zkb_basefold_tables(zkb_ctx* c, uint32_t log_n, uint32_t* t_flat, uint32_t* w_flat) {
    if (!c || !t_flat || !w_flat || log_n < 1 || log_n > 28) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        BfTables tb = bf_tables(c, log_n);
        const size_t total = (size_t(1) << log_n) - 1;
        ZKB_CUDA(cudaMemcpyAsync(t_flat, tb.t_flat, total * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaMemcpyAsync(w_flat, tb.w_flat, total * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_basefold_encode(zkb_ctx* c, const uint32_t* coeffs, size_t n, int32_t on_device, uint32_t* codeword, int32_t out_on_device) {
    if (!c || (!coeffs && n) || !codeword) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const u32 log_n = tree_height(n);
        if (log_n > 28) throw ArgFail{ZKB_E_TOO_LARGE, "basefold: log_n out of range"};
        const size_t n_pad = size_t(1) << log_n;
        const u32* d = on_device ? coeffs : up_pad(c, coeffs, n, n);
        BfTables tb = bf_tables(c, log_n);
        u32* cw = out_on_device ? codeword : (u32*)c->scratch(2 * n_pad * 4);
        bf_encode(c, CoefSrc{d, 1, (u32)n, log_n}, log_n, tb, cw);
        if (!out_on_device) ZKB_CUDA(cudaMemcpyAsync(codeword, cw, 2 * n_pad * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_basefold_commit_and_prove(zkb_ctx* c, zkb_transcript* tr, const uint32_t* coeffs, size_t n, const uint32_t* point,
                                      uint32_t n_point, int32_t on_device, int32_t node_hash, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !tr || (!coeffs && n) || (!point && n_point) || !len) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const u32 log_n = tree_height(n);
        const u32* d = on_device ? coeffs : up_pad(c, coeffs, n, n);
        const u32* pt = on_device ? point : up_pad(c, point, n_point, (size_t)n_point + 1);
        c->rec_reset();
        BfPending pd = basefold_enqueue(c, tr->dev, CoefSrc{d, 1, (u32)n, log_n}, n, log_n, pt, n_point, node_hash);
        c->rec_fetch();
        Ser s;
        put_basefold_commitment(s, c->rec_host, pd);
        put_basefold_proof(s, c->rec_host, pd);
        c->scratch_reset();
        int32_t rc = emit(c, s.b, out, cap, len);
        if (rc) return rc;
    });
}

// verify_opening (basefold.rs:611-748).  The caller has absorbed the commitment root, as the reference's callers do.
int32_t zkb_basefold_verify_opening(zkb_ctx* c, zkb_transcript* tr, const uint8_t* bytes, size_t len, const uint32_t* point, uint32_t n_point,
                                    uint32_t claimed, int32_t node_hash, int32_t* accepted) {
    if (!c || !tr || !bytes || (!point && n_point) || !accepted) return ZKB_E_ARG;
    *accepted = 0;
    ZKB_TRY(c, {
        c->use();
        BvParsed pr;
        if (!bv_parse(bytes, len, pr)) throw ArgFail{ZKB_E_ARG, "basefold: the bytes do not decode as a commitment followed by an opening proof"};
        if (pr.too_large) throw ArgFail{ZKB_E_TOO_LARGE, "basefold: more than 256 opened positions in one batch proof"};
        if (pr.trees.empty()) return ZKB_OK;                      // wrong number of fold rounds: rejected before the transcript is touched
        const u32* pt = up_pad(c, point, n_point, (size_t)n_point + 1);
        BvRun run = basefold_verify_enqueue(c, tr->dev, pr, pt, n_point, node_hash);
        std::vector<u32> res(run.n_results);
        ZKB_CUDA(cudaMemcpyAsync(res.data(), run.result_dev, (size_t)run.n_results * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
        bool ok = pr.final_value % ZKB_P == claimed % ZKB_P;
        for (u32 v : res) ok = ok && v == 1;
        *accepted = ok ? 1 : 0;
    });
}

}  // extern "C"
