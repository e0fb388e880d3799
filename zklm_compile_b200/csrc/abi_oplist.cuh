// C ABI, part 7: the op-list mode (see oplist.cuh).  Included by zkb200.cu.

namespace {

using OL = zkb_oplist;

zkb::u32* ol_alloc(OL* L, size_t words) {
    zkb::u32* p = nullptr;
    ZKB_CUDA(cudaMalloc(&p, (words + 8) * 4));
    ZKB_CUDA(cudaMemsetAsync(p, 0, (words + 8) * 4, L->ctx->stream));
    L->owned.push_back(p);
    return p;
}
zkb::u32* ol_upload(OL* L, const uint32_t* host, size_t n, size_t n_pad) {
    zkb::u32* p = ol_alloc(L, n_pad > n ? n_pad : n);
    if (n) ZKB_CUDA(cudaMemcpyAsync(p, host, n * 4, cudaMemcpyHostToDevice, L->ctx->stream));
    return p;
}
OL::Op& ol_push(OL* L, OL::Kind kind, const char* name, zkb::u32 out_len, bool own_out) {
    OL::Op op;
    op.kind = kind;
    op.name = name ? name : "";
    op.in_len = L->cur_len;
    op.out_len = out_len;
    if (own_out) op.out = ol_alloc(L, pad_pow2(out_len));
    L->ops.push_back(op);
    L->cur_len = out_len;
    return L->ops.back();
}
// An add_* call that fails half way (an allocation, a length check) leaves the list as it was.
struct OlTxn {
    OL* L; size_t n_ops; zkb::u32 len; bool done = false;
    explicit OlTxn(OL* l) : L(l), n_ops(l->ops.size()), len(l->cur_len) {}
    ~OlTxn() { if (!done) { L->ops.erase(L->ops.begin() + (std::ptrdiff_t)n_ops, L->ops.end()); L->cur_len = len; } }
};
const zkb::u32* ol_input_of(const OL* L, size_t idx) { return idx == 0 ? L->x : L->ops[idx - 1].out; }

// The forward pass (pipeline/forward.rs:24-520) over the resident ops; the input is already in L->x.
void ol_forward(OL* L) {
    zkb_ctx* c = L->ctx;
    for (size_t i = 0; i < L->ops.size(); i++) {
        OL::Op& op = L->ops[i];
        const zkb::u32* in = ol_input_of(L, i);
        const zkb::u32 n_pad = (zkb::u32)pad_pow2(op.out_len);
        switch (op.kind) {
            case OL::LINEAR:
                matvec_forward(c, op.w, in, op.m, op.n, op.out, n_pad, false);
                if (op.b) { bias_add_kernel<<<grid_for(c, op.m), 256, 0, c->stream>>>(op.out, op.b, op.m); ZKB_LAUNCHED(c); }
                break;
            case OL::RELU:
                relu_forward_kernel<<<grid_for(c, n_pad), 256, 0, c->stream>>>(in, op.out_len, n_pad, op.out);
                ZKB_LAUNCHED(c);
                break;
            case OL::LAYERNORM:
                layernorm_forward_kernel<<<1, c->single_cta_threads(), 0, c->stream>>>(in, op.gamma, op.beta, op.out_len, n_pad, op.aux1, op.aux0, op.out,
                                                                                      op.scalars, c->status);
                ZKB_LAUNCHED(c);
                break;
            case OL::GELU:
                requant_lookup_kernel<<<grid_for(c, n_pad), 256, 0, c->stream>>>(in, op.out_len, n_pad, op.table, op.n_table, op.aux0, op.out, c->status);
                ZKB_LAUNCHED(c);
                break;
            case OL::ATTENTION:
                pad_copy_kernel<<<grid_for(c, n_pad), 256, 0, c->stream>>>(in + 2 * (size_t)op.out_len, op.out_len, n_pad, op.out);
                ZKB_LAUNCHED(c);
                break;
            case OL::ATTENTION_ROWS: {
                const size_t total = (size_t)op.heads * op.seq * op.d_head, total_kv = (size_t)(op.kv_heads ? op.kv_heads : op.heads) * op.seq * op.d_head;
                attention_forward_enqueue(c, in, op.aux0 ? op.aux0 : in + total, op.aux1 ? op.aux1 : in + total + total_kv, op.heads, op.kv_heads, op.seq,
                                          op.d_head, op.table, op.n_table, op.out);
                break;
            }
            case OL::ADD_SAVED:
                add_vec_kernel<<<grid_for(c, n_pad), 256, 0, c->stream>>>(in, L->ops[op.save_of].out, op.out_len, n_pad, op.out);
                ZKB_LAUNCHED(c);
                break;
            case OL::SET_INPUT_REQUANT:
                requant_lookup_kernel<<<grid_for(c, n_pad), 256, 0, c->stream>>>(in, op.out_len, n_pad, nullptr, 0, op.out, nullptr, c->status);
                ZKB_LAUNCHED(c);
                break;
            case OL::SAVE: case OL::PASSTHROUGH:
                op.out = const_cast<zkb::u32*>(in);        // same activation, no copy
                break;
            case OL::SET_INPUT:
                break;                                     // op.out holds the caller's values
        }
    }
    ZKB_CUDA(cudaGetLastError());
}

struct OlProofRec {
    int tag = 0;
    MatmulRec mm; ReluRec relu; LayerNormRec ln; LookupRec lk;
    size_t lk_io = 0;         // record offset of the lookup's inputs and outputs (2 n words)
    size_t h0 = 0, h1 = 0;    // record offsets of digests (8 words each)
    AttRun att; zkb::u32 att_heads = 0; size_t att_host = 0;   // attention at seq_len >= 2: word offset of its records in the staging buffer
    bool h0_zero = false;
    std::string text;
};

// Record offset of the content digest of (v, n); the digests of one proof are computed up front by ol_hash_all.
size_t ol_hash(OL* L, const zkb::u32* v, zkb::u32 n) {
    for (size_t j = 0; j < L->hash_jobs.size(); j++)
        if (L->hash_jobs[j].v == v && L->hash_jobs[j].n == n) return L->hash_base + 8 * j;
    throw ArgFail{ZKB_E_ARG, "op list: content digest not scheduled"};
}
void ol_hash_all(OL* L) {
    zkb_ctx* c = L->ctx;
    if (L->hash_jobs_nops != L->ops.size()) {            // first proof, or ops were added since the last one
        L->hash_jobs.clear();
        auto want = [&](const zkb::u32* v, zkb::u32 n) {
            for (const HashJob& j : L->hash_jobs) if (j.v == v && j.n == n) return;
            L->hash_jobs.push_back(HashJob{v, n, 0});
        };
        for (size_t idx = 0; idx < L->ops.size(); idx++) {
            const OL::Op& op = L->ops[idx];
            switch (op.kind) {
                case OL::ATTENTION: case OL::PASSTHROUGH: case OL::SAVE: want(op.out, op.out_len); break;
                case OL::SET_INPUT: case OL::SET_INPUT_REQUANT:
                    want(op.out, op.out_len);
                    if (idx > 0) want(L->ops[idx - 1].out, L->ops[idx - 1].out_len);
                    break;
                default: break;
            }
        }
        if (!L->hash_jobs.empty()) {
            void* d = nullptr;
            ZKB_CUDA(cudaMalloc(&d, L->hash_jobs.size() * sizeof(HashJob)));
            L->owned.push_back(d);
            L->hash_jobs_dev = (HashJob*)d;
            ZKB_CUDA(cudaMemcpyAsync(d, L->hash_jobs.data(), L->hash_jobs.size() * sizeof(HashJob), cudaMemcpyHostToDevice, c->stream));
        }
        L->hash_jobs_nops = L->ops.size();
    }
    if (L->hash_jobs.empty()) return;
    L->hash_base = c->rec_alloc(8 * L->hash_jobs.size());
    hash_values_multi_kernel<<<(unsigned)L->hash_jobs.size(), TRSCRIPT_THREADS, 0, c->stream>>>(L->hash_jobs_dev, c->rec_dev + L->hash_base);
    ZKB_LAUNCHED(c);
}

// prove_all_ops, sequential branch (pipeline/prove.rs:191-648): enqueue everything, fetch the record once, serialise.
std::vector<uint8_t> ol_prove(OL* L, uint32_t* status_out) {
    zkb_ctx* c = L->ctx;
    c->rec_reset();
    TrState* tr = (TrState*)c->scratch(sizeof(TrState));
    tr_init_kernel<<<1, 1, 0, c->stream>>>(tr);
    ZKB_LAUNCHED(c);
    { ScriptBuilder sb; sb.str("structured-ml-proof"); sb.run(c, tr); }
    ol_hash_all(L);
    // the attention ops' row records come back through one page-locked buffer, sized before anything is enqueued
    size_t att_words = 0;
    for (const OL::Op& op : L->ops)
        if (op.kind == OL::ATTENTION_ROWS) att_words += (size_t)op.heads * op.seq * (att_layout(op.seq, op.d_head).words + op.seq + op.d_head);
    zkb::u32* att_stage = att_words ? (zkb::u32*)c->stage_host(att_words * 4) : nullptr;
    size_t att_used = 0;
    std::vector<OlProofRec> recs;
    const zkb::u32* chain_point = nullptr;        // s_point of the last pushed proof when that proof is a matmul
    for (size_t idx = L->ops.size(); idx-- > 0;) {
        OL::Op& op = L->ops[idx];
        const zkb::u32* in = ol_input_of(L, idx);
        OlProofRec R;
        switch (op.kind) {
            case OL::LINEAR: {
                ScriptBuilder sb;
                sb.bytes(op.root, 32);
                sb.run(c, tr);
                R.tag = 0;
                R.mm = prove_matmul_succinct_base(c, tr, op.w, in, op.out, op.m, op.n);
                chain_point = c->rec_dev + R.mm.sc.chal;
                recs.push_back(R);
                continue;
            }
            case OL::RELU:
                R.tag = 1;
                R.relu = prove_relu(c, tr, in, op.in_len, chain_point);
                break;
            case OL::LAYERNORM:
                R.tag = 3;
                R.ln = prove_layernorm_sqr(c, tr, op.aux0, op.gamma, op.beta, op.out, op.out_len, op.scalars);
                break;
            case OL::GELU: {
                R.tag = 4;
                R.lk = prove_lookup_base(c, tr, op.table, op.n_table, op.aux0, op.out, op.out_len);
                R.lk_io = c->rec_alloc(2 * (size_t)op.out_len);
                ZKB_CUDA(cudaMemcpyAsync(c->rec_dev + R.lk_io, op.aux0, (size_t)op.out_len * 4, cudaMemcpyDeviceToDevice, c->stream));
                ZKB_CUDA(cudaMemcpyAsync(c->rec_dev + R.lk_io + op.out_len, op.out, (size_t)op.out_len * 4, cudaMemcpyDeviceToDevice, c->stream));
                break;
            }
            case OL::ATTENTION: case OL::PASSTHROUGH: {
                R.tag = 16;
                R.h0 = ol_hash(L, op.out, op.out_len);
                ScriptBuilder sb;
                sb.words_dev(c->rec_dev + R.h0, 8);
                sb.run(c, tr);
                break;
            }
            case OL::ATTENTION_ROWS: {
                R.tag = op.kv_heads ? 12 : 5;                          // Attention / GqaAttention (prove.rs:419-432, 572-584)
                const size_t total = (size_t)op.heads * op.seq * op.d_head, total_kv = (size_t)(op.kv_heads ? op.kv_heads : op.heads) * op.seq * op.d_head;
                const size_t rec_words = (size_t)op.heads * op.seq * att_layout(op.seq, op.d_head).words;
                R.att_host = att_used; R.att_heads = op.heads;
                R.att = attention_prove_enqueue(c, tr, in, op.aux0 ? op.aux0 : in + total, op.aux1 ? op.aux1 : in + total + total_kv, op.heads, op.kv_heads,
                                                op.seq, op.d_head, op.table, op.n_table, nullptr, att_stage + att_used, att_stage + att_used + rec_words);
                att_used += rec_words + (size_t)op.heads * op.seq * (op.seq + op.d_head);
                break;
            }
            case OL::ADD_SAVED: {
                R.tag = 6;
                std::string s = op.name;                    // layer.name.replacen("add_", "save_", 1)
                size_t at = s.find("add_");
                if (at != std::string::npos) s.replace(at, 4, "save_");
                R.text = s;
                break;
            }
            case OL::SAVE: {
                R.tag = 8;
                R.text = op.name;
                R.h0 = ol_hash(L, op.out, op.out_len);
                ScriptBuilder sb;
                sb.words_dev(c->rec_dev + R.h0, 8);
                sb.run(c, tr);
                break;
            }
            case OL::SET_INPUT: case OL::SET_INPUT_REQUANT: {
                R.tag = 7;
                R.h1 = ol_hash(L, op.out, op.out_len);
                ScriptBuilder sb;
                if (idx > 0) {
                    R.h0 = ol_hash(L, L->ops[idx - 1].out, L->ops[idx - 1].out_len);
                    sb.words_dev(c->rec_dev + R.h0, 8);
                } else {
                    R.h0_zero = true;
                    unsigned char z[32] = {0};
                    sb.bytes(z, 32);
                }
                sb.words_dev(c->rec_dev + R.h1, 8);
                sb.run(c, tr);
                break;
            }
        }
        chain_point = nullptr;
        recs.push_back(R);
    }
    ZKB_CUDA(cudaGetLastError());
    c->rec_fetch();
    *status_out = c->read_status();
    Ser s;
    s.rec = c->rec_host;
    s.u64le(recs.size());
    for (const OlProofRec& R : recs) {
        s.u32le((u32)R.tag);
        switch (R.tag) {
            case 0: put_matmul_base(s, R.mm); break;
            case 1: put_relu(s, R.relu); break;
            case 3: put_layernorm_sqr(s, R.ln); break;
            case 4: put_lookup_base(s, R.lk, s.rec + R.lk_io, s.rec + R.lk_io + R.lk.n); break;
            case 5: case 12: {
                const zkb::u32* hrec = att_stage + R.att_host;
                const zkb::u32* hbind = hrec + (size_t)R.att.rows * R.att.L.words;
                AttSer count{nullptr};
                count.proof(R.att.L, R.att_heads, hrec, hbind);
                const size_t at = s.b.size();
                s.b.resize(at + count.n);
                AttSer w{s.b.data() + at};
                w.proof(R.att.L, R.att_heads, hrec, hbind);
                break;
            }
            case 6: s.u64le(R.text.size()); for (char ch : R.text) s.u8((uint8_t)ch); break;
            case 7:
                if (R.h0_zero) for (int i = 0; i < 8; i++) s.u32le(0); else s.words(R.h0, 8);
                s.words(R.h1, 8);
                break;
            case 8: s.u64le(R.text.size()); for (char ch : R.text) s.u8((uint8_t)ch); s.words(R.h0, 8); break;
            case 16: break;
        }
    }
    c->scratch_reset();
    return s.b;
}

}  // namespace

extern "C" {

// requantize_to_i16_field (transformer/mod.rs:293-324) and, with a table, the activation lookup
// (qwen.rs:286-316: table[requantised value]) of a vector, on the device.
int32_t zkb_requantize_lookup(zkb_ctx* c, const uint32_t* raw, size_t n, int32_t on_device, const uint32_t* table_out_dev, uint32_t n_table,
                              uint32_t* q_out, uint32_t* t_out) {
    if (!c || !raw || !q_out || n == 0 || n > (size_t(1) << 28) || (table_out_dev && n_table != 256 && n_table != 65536) ||
        (table_out_dev && !t_out)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        clear_status(c);
        const u32* d = on_device ? raw : up_pad(c, raw, n, n);
        u32* q = (u32*)c->scratch(n * 4);
        u32* t = table_out_dev ? (u32*)c->scratch(n * 4) : nullptr;
        requant_lookup_kernel<<<grid_for(c, n), 256, 0, c->stream>>>(d, (u32)n, (u32)n, table_out_dev, n_table, q, t, c->status);
        ZKB_LAUNCHED(c);
        ZKB_CUDA(cudaGetLastError());
        ZKB_CUDA(cudaMemcpyAsync(q_out, q, n * 4, cudaMemcpyDeviceToHost, c->stream));
        if (t) ZKB_CUDA(cudaMemcpyAsync(t_out, t, n * 4, cudaMemcpyDeviceToHost, c->stream));
        uint32_t st = c->read_status();
        c->scratch_reset();
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
    });
}

int32_t zkb_oplist_create(zkb_ctx* c, uint32_t input_len, zkb_oplist** out) {
    if (!c || !out || input_len == 0) return ZKB_E_ARG;
    *out = nullptr;
    zkb_oplist* L = new (std::nothrow) zkb_oplist();
    if (!L) return ZKB_E_CUDA;
    L->ctx = c;
    try {
        c->use();
        L->in_len = L->cur_len = input_len;
        L->x = ol_alloc(L, pad_pow2(input_len));
    } catch (const CudaFail& e) { c->err = e.msg; delete L; return ZKB_E_CUDA; }
    *out = L;
    return ZKB_OK;
}
void zkb_oplist_destroy(zkb_oplist* L) {
    if (!L) return;
    if (L->ctx) { cudaSetDevice(L->ctx->device); cudaStreamSynchronize(L->ctx->stream); }
    for (void* p : L->owned) cudaFree(p);
    delete L;
}
int32_t zkb_oplist_add_linear(zkb_oplist* L, const char* name, const uint32_t* W, const uint32_t* bias, size_t m, size_t n) {
    if (!L || !W || m == 0 || n == 0) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        if (n != L->cur_len) throw ArgFail{ZKB_E_LENGTH, "linear: column count differs from the activation length"};
        OlTxn txn(L);
        OL::Op& op = ol_push(L, OL::LINEAR, name, (u32)m, true);
        op.m = (u32)m; op.n = (u32)n;
        op.w = ol_upload(L, W, m * n, m * n);
        if (bias) op.b = ol_upload(L, bias, m, m);
        // commit_weights_fast(W), absorbed in front of the matmul proof (prove.rs:210-211): once, at load time
        u32* root = (u32*)c->scratch(32);
        commit_large(c, b3_prefix("weights", 7), op.w, m * n, root);
        ZKB_CUDA(cudaMemcpyAsync(op.root, root, 32, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
        txn.done = true;
    });
}
int32_t zkb_oplist_add_simple(zkb_oplist* L, int32_t kind, const char* name, const char* aux) {
    if (!L) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        const u32 n = L->cur_len;
        OlTxn txn(L);
        switch (kind) {
            case ZKB_OP_RELU: ol_push(L, OL::RELU, name, n, true); break;
            case ZKB_OP_ATTENTION_SEQ1:
                if (n % 3) throw ArgFail{ZKB_E_LENGTH, "attention: the activation is not a Q | K | V concatenation"};
                ol_push(L, OL::ATTENTION, name, n / 3, true);
                break;
            case ZKB_OP_PASSTHROUGH: ol_push(L, OL::PASSTHROUGH, name, n, false); break;
            case ZKB_OP_SAVE: { OL::Op& op = ol_push(L, OL::SAVE, name, n, false); op.aux = aux ? aux : ""; break; }
            case ZKB_OP_ADD_SAVED: {
                int found = -1;
                for (size_t i = 0; i < L->ops.size(); i++)
                    if (L->ops[i].kind == OL::SAVE && L->ops[i].aux == (aux ? aux : "")) found = (int)i;
                if (found < 0) throw ArgFail{ZKB_E_ARG, "add_saved: no saved buffer of that name"};
                if (L->ops[found].out_len != n) throw ArgFail{ZKB_E_LENGTH, "add_saved: dimension mismatch"};
                OL::Op& op = ol_push(L, OL::ADD_SAVED, name, n, true);
                op.save_of = found;
                break;
            }
            case ZKB_OP_SET_INPUT_REQUANT: ol_push(L, OL::SET_INPUT_REQUANT, name, n, true); break;
            default: throw ArgFail{ZKB_E_ARG, "unknown op kind"};
        }
        txn.done = true;
    });
}
int32_t zkb_oplist_add_layernorm(zkb_oplist* L, const char* name, const uint32_t* gamma, const uint32_t* beta, size_t d) {
    if (!L || !gamma || !beta || d == 0) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        if (d != L->cur_len) throw ArgFail{ZKB_E_LENGTH, "layernorm: width differs from the activation length"};
        OlTxn txn(L);
        OL::Op& op = ol_push(L, OL::LAYERNORM, name, (u32)d, true);
        op.gamma = ol_upload(L, gamma, d, d);
        op.beta = ol_upload(L, beta, d, d);
        op.aux0 = ol_alloc(L, pad_pow2(d));
        op.aux1 = ol_alloc(L, pad_pow2(d));
        op.scalars = ol_alloc(L, 8);
        txn.done = true;
    });
}
int32_t zkb_oplist_add_gelu(zkb_oplist* L, const char* name, const uint32_t* table_out_dev, uint32_t n_table) {
    if (!L || !table_out_dev || (n_table != 256 && n_table != 65536)) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        OlTxn txn(L);
        OL::Op& op = ol_push(L, OL::GELU, name, L->cur_len, true);
        op.table = table_out_dev; op.n_table = n_table;
        op.aux0 = ol_alloc(L, pad_pow2(op.out_len));
        txn.done = true;
    });
}
int32_t zkb_oplist_add_attention(zkb_oplist* L, const char* name, size_t num_heads, size_t num_kv_heads, size_t seq_len, size_t d_head,
                                 const uint32_t* table_out_dev, uint32_t n_table, const uint32_t* k_values, const uint32_t* v_values) {
    if (!L || !table_out_dev || (k_values == nullptr) != (v_values == nullptr)) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        att_check_dims(num_heads, seq_len, d_head, n_table);
        if (seq_len < 2) throw ArgFail{ZKB_E_ARG, "attention: seq_len = 1 is ZKB_OP_ATTENTION_SEQ1"};
        att_heads_per_group(num_heads, num_kv_heads);
        const size_t total = num_heads * seq_len * d_head, total_kv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
        // "attention" asserts Q | K | V exactly (forward.rs:219-221); "gqa_attention" slices what it needs (forward.rs:564-574)
        if (k_values ? L->cur_len < total : (num_kv_heads ? L->cur_len < total + 2 * total_kv : L->cur_len != 3 * total))
            throw ArgFail{ZKB_E_LENGTH, "attention: the activation is not Q | K | V of (heads, seq_len, d_head) (or Q alone when K and V are given)"};
        OlTxn txn(L);
        OL::Op& op = ol_push(L, OL::ATTENTION_ROWS, name, (u32)total, true);
        op.heads = (u32)num_heads; op.kv_heads = (u32)num_kv_heads; op.seq = (u32)seq_len; op.d_head = (u32)d_head;
        op.table = table_out_dev; op.n_table = n_table;
        if (k_values) { op.aux0 = ol_upload(L, k_values, total_kv, total_kv); op.aux1 = ol_upload(L, v_values, total_kv, total_kv); }
        txn.done = true;
    });
}
// New K and V for an attention op that was added with its own (the reference's request carries them with every op, protocol.rs:714-722).
int32_t zkb_oplist_set_attention_kv(zkb_oplist* L, uint32_t op_index, const uint32_t* k_values, const uint32_t* v_values) {
    if (!L || !k_values || !v_values || op_index >= L->ops.size()) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        OL::Op& op = L->ops[op_index];
        if (op.kind != OL::ATTENTION_ROWS || !op.aux0 || !op.aux1) throw ArgFail{ZKB_E_ARG, "not an attention op that holds its own K and V"};
        const size_t total_kv = (size_t)(op.kv_heads ? op.kv_heads : op.heads) * op.seq * op.d_head;
        ZKB_CUDA(cudaMemcpyAsync(op.aux0, k_values, total_kv * 4, cudaMemcpyHostToDevice, c->stream));
        ZKB_CUDA(cudaMemcpyAsync(op.aux1, v_values, total_kv * 4, cudaMemcpyHostToDevice, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    });
}
int32_t zkb_oplist_add_set_input(zkb_oplist* L, const char* name, const uint32_t* values, size_t n) {
    if (!L || !values || n == 0) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        OlTxn txn(L);
        OL::Op& op = ol_push(L, OL::SET_INPUT, name, (u32)n, false);
        op.out = ol_upload(L, values, n, pad_pow2(n));
        txn.done = true;
    });
}
uint32_t zkb_oplist_output_len(const zkb_oplist* L) { return L ? L->cur_len : 0; }
int32_t zkb_oplist_forward(zkb_oplist* L, const uint32_t* x) {
    if (!L || !x) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        clear_status(c);
        ZKB_CUDA(cudaMemcpyAsync(L->x, x, (size_t)L->in_len * 4, cudaMemcpyHostToDevice, c->stream));
        ol_forward(L);
        uint32_t st = c->read_status();
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
    });
}
int32_t zkb_oplist_activation(zkb_oplist* L, uint32_t op_index, uint32_t* out, size_t cap, size_t* len) {
    if (!L || !len || op_index >= L->ops.size()) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        const OL::Op& op = L->ops[op_index];
        *len = op.out_len;
        if (!out || cap < op.out_len) throw ArgFail{ZKB_E_TOO_LARGE, "output buffer too small"};
        if (!op.out) throw ArgFail{ZKB_E_ARG, "run the forward pass first"};
        ZKB_CUDA(cudaMemcpyAsync(out, op.out, (size_t)op.out_len * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    });
}
int32_t zkb_oplist_prove(zkb_oplist* L, const uint32_t* x, uint8_t* out, size_t cap, size_t* len) {
    if (!L || !x) return ZKB_E_ARG;
    zkb_ctx* c = L->ctx;
    ZKB_TRY(c, {
        c->use();
        clear_status(c);
        ZKB_CUDA(cudaMemcpyAsync(L->x, x, (size_t)L->in_len * 4, cudaMemcpyHostToDevice, c->stream));
        ol_forward(L);
        uint32_t st = 0;
        std::vector<uint8_t> b = ol_prove(L, &st);
        int32_t rc = status_to_code(c, st);
        if (rc) return rc;
        rc = emit(c, b, out, cap, len);
        if (rc) return rc;
    });
}

}  // extern "C"
