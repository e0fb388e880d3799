// C ABI, part 8: row-decomposed attention at seq_len >= 2.  Included by zkb200.cu.

namespace {

struct AttDev { const u32 *q, *k, *v, *table; };
AttDev att_inputs(zkb_ctx* c, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t n, size_t n_kv, const uint32_t* table_out,
                  size_t n_table, int32_t on_device) {
    if (on_device) return AttDev{q, k, v, table_out};
    return AttDev{up_pad(c, q, n, n), up_pad(c, k, n_kv, n_kv), up_pad(c, v, n_kv, n_kv), up_pad(c, table_out, n_table, n_table)};
}
int32_t att_status(zkb_ctx* c, uint32_t st) {
    if (st == ST_LOOKUP_KEY) { c->err = "attention: a score is not an input of the exp table"; return ZKB_E_ARG; }
    return status_to_code(c, st);
}

}  // namespace

extern "C" {

int32_t zkb_row_attention_gqa_forward(zkb_ctx* c, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t num_kv_heads,
                                      size_t seq_len, size_t d_head, const uint32_t* table_out, size_t n_table, int32_t on_device, uint32_t* out) {
    if (!c || !q || !k || !v || !table_out || !out) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        att_check_dims(num_heads, seq_len, d_head, n_table);
        clear_status(c);
        att_heads_per_group(num_heads, num_kv_heads);
        const size_t n = num_heads * seq_len * d_head, n_kv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
        AttDev d = att_inputs(c, q, k, v, n, n_kv, table_out, n_table, on_device);
        u32* dout = on_device ? out : (u32*)c->scratch(n * 4);
        attention_forward_enqueue(c, d.q, d.k, d.v, (u32)num_heads, (u32)num_kv_heads, (u32)seq_len, (u32)d_head, d.table, (u32)n_table, dout);
        ZKB_CUDA(cudaGetLastError());
        if (!on_device) ZKB_CUDA(cudaMemcpyAsync(out, dout, n * 4, cudaMemcpyDeviceToHost, c->stream));
        uint32_t st = c->read_status();
        c->scratch_reset();
        int32_t rc = att_status(c, st);
        if (rc) return rc;
    });
}

int32_t zkb_row_attention_forward(zkb_ctx* c, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t seq_len,
                                  size_t d_head, const uint32_t* table_out, size_t n_table, int32_t on_device, uint32_t* out) {
    return zkb_row_attention_gqa_forward(c, q, k, v, num_heads, 0, seq_len, d_head, table_out, n_table, on_device, out);
}

int32_t zkb_prove_row_attention_gqa(zkb_ctx* c, zkb_transcript* t, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads,
                                    size_t num_kv_heads, size_t seq_len, size_t d_head, const uint32_t* table_out, size_t n_table,
                                    int32_t on_device, uint32_t* attn_out, uint8_t* out, size_t cap, size_t* len) {
    if (!c || !q || !k || !v || !table_out) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        att_check_dims(num_heads, seq_len, d_head, n_table);
        if (seq_len < 2) throw ArgFail{ZKB_E_ARG, "attention: seq_len = 1 has no row proofs (the output is V)"};
        att_heads_per_group(num_heads, num_kv_heads);
        clear_status(c);
        const size_t n = num_heads * seq_len * d_head, n_kv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
        AttDev d = att_inputs(c, q, k, v, n, n_kv, table_out, n_table, on_device);
        u32* dout = (on_device && attn_out) ? attn_out : (u32*)c->scratch(n * 4);
        const size_t rec_words = num_heads * seq_len * (size_t)att_layout((u32)seq_len, (u32)d_head).words, bind_words = num_heads * seq_len * (seq_len + d_head);
        u32* host = (u32*)c->stage_host((rec_words + bind_words) * 4);
        AttRun R = attention_prove_enqueue(c, t ? t->dev : nullptr, d.q, d.k, d.v, (u32)num_heads, (u32)num_kv_heads, (u32)seq_len, (u32)d_head, d.table, (u32)n_table, dout,
                                           host, host + rec_words);
        ZKB_CUDA(cudaGetLastError());
        if (attn_out && !on_device) ZKB_CUDA(cudaMemcpyAsync(attn_out, dout, n * 4, cudaMemcpyDeviceToHost, c->stream));
        uint32_t st = c->read_status();
        c->scratch_reset();
        int32_t rc = att_status(c, st);
        if (rc) return rc;
        AttSer count{nullptr};
        count.proof(R.L, num_heads, host, host + rec_words);
        if (len) *len = count.n;
        if (count.n > cap || !out) { c->err = "output buffer too small"; return ZKB_E_TOO_LARGE; }
        AttSer w{out};
        w.proof(R.L, num_heads, host, host + rec_words);
    });
}

int32_t zkb_prove_row_attention(zkb_ctx* c, zkb_transcript* t, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads,
                                size_t seq_len, size_t d_head, const uint32_t* table_out, size_t n_table, int32_t on_device,
                                uint32_t* attn_out, uint8_t* out, size_t cap, size_t* len) {
    return zkb_prove_row_attention_gqa(c, t, q, k, v, num_heads, 0, seq_len, d_head, table_out, n_table, on_device, attn_out, out, cap, len);
}

// verify_row_attention / verify_row_attention_gqa (attention.rs:279-385, 503-590) on bincode(RowAttentionProof).  As in the reference, q
// and the exp table are not needed: the verifier recomputes K(r, s) and V^T(r, s) from k and v and replays each row's transcript.
int32_t zkb_verify_row_attention(zkb_ctx* c, zkb_transcript* t, const uint8_t* proof, size_t len, const uint32_t* k, const uint32_t* v,
                                 size_t num_heads, size_t num_kv_heads, size_t seq_len, size_t d_head, int32_t on_device, int32_t* accepted) {
    if (!c || !proof || !k || !v || !accepted) return ZKB_E_ARG;
    *accepted = 0;
    ZKB_TRY(c, {
        c->use();
        att_check_dims(num_heads, seq_len, d_head, 65536);
        if (seq_len < 2) throw ArgFail{ZKB_E_ARG, "attention: seq_len = 1 has no row proofs"};
        att_heads_per_group(num_heads, num_kv_heads);
        AvParsed pr;
        if (!av_parse(proof, len, (u32)num_heads, (u32)seq_len, (u32)d_head, pr))
            throw ArgFail{ZKB_E_ARG, "attention: the bytes do not decode as a RowAttentionProof"};
        if (pr.reject) return ZKB_OK;                             // dimensions or vector lengths the prover does not produce
        const size_t n_kv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
        const u32* dk = on_device ? k : up_pad(c, k, n_kv, n_kv);
        const u32* dv = on_device ? v : up_pad(c, v, n_kv, n_kv);
        AvRun run = attention_verify_enqueue(c, t ? t->dev : nullptr, pr, dk, dv, (u32)num_kv_heads);
        std::vector<u32> res(run.rows);
        ZKB_CUDA(cudaMemcpyAsync(res.data(), run.result_dev, (size_t)run.rows * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
        bool ok = true;
        for (u32 r : res) ok = ok && r == 1;
        *accepted = ok ? 1 : 0;
    });
}

}  // extern "C"
