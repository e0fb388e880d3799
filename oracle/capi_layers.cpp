// CPU ORACLE — TEST INFRASTRUCTURE ONLY.
//
// C entry points for the matmul / MLE-eval / element-wise / RMSNorm / LogUp / Qwen-layer
// restatements.  Proofs come back as bincode bytes (oracle/bincode.hpp).
#include "attention.hpp"
#include "oplist.hpp"
#include "unbincode.hpp"
#include <cstring>

using namespace zko;

static VF vf(const uint32_t* p, size_t n) { VF v(n); for (size_t i = 0; i < n; i++) v[i] = F(p[i]); return v; }
static VEF vef(const uint32_t* p, size_t n) { VEF v(n); for (size_t i = 0; i < n; i++) v[i] = EF::from_u32x4(p + 4 * i); return v; }
static Transcript& T(void* t) { return *static_cast<Transcript*>(t); }
static size_t emit(const std::vector<uint8_t>& b, uint8_t* out, size_t cap) {
    if (out && b.size() <= cap) memcpy(out, b.data(), b.size());
    return b.size();
}
static void out_f(const VF& v, uint32_t* o) { for (size_t i = 0; i < v.size(); i++) o[i] = v[i].v; }

extern "C" {

void zko_commit_weights_fast(const uint32_t* w, size_t n, uint8_t* root) {
    auto c = commit_weights_fast(vf(w, n));
    memcpy(root, c.root.data(), 32);
}
void zko_matmul_forward(const uint32_t* w, const uint32_t* x, size_t m, size_t n, uint32_t* y) {
    out_f(matmul_forward(vf(w, m * n), vf(x, n), m, n), y);
}
void zko_fold_eq_matvec(const uint32_t* w, size_t m, size_t n, const uint32_t* r, size_t log_m, uint32_t* out) {
    out_f(fold_eq_matvec(vf(w, m * n), m, n, size_t(1) << log2_ceil(n), vf(r, log_m)), out);
}
void zko_fold_eq_matvec_ef(const uint32_t* w, size_t m, size_t n, const uint32_t* r, size_t log_m, uint32_t* out) {
    VEF o = fold_eq_matvec_ef(vf(w, m * n), m, n, size_t(1) << log2_ceil(n), vef(r, log_m));
    for (size_t i = 0; i < o.size(); i++) o[i].to_u32x4(out + 4 * i);
}
size_t zko_prove_matmul_succinct(void* t, const uint32_t* w, const uint32_t* x, const uint32_t* y, size_t m, size_t n,
                                 uint8_t* out, size_t cap) {
    Bin b; b.put(prove_matmul_succinct(vf(w, m * n), vf(x, n), vf(y, m), m, n, T(t)));
    return emit(b.b, out, cap);
}
size_t zko_prove_matmul_succinct_ef(void* t, const uint32_t* w, const uint32_t* x, const uint32_t* y, size_t m, size_t n,
                                    uint8_t* out, size_t cap) {
    Bin b; b.put(prove_matmul_succinct_ef(vf(w, m * n), vf(x, n), vf(y, m), m, n, T(t)));
    return emit(b.b, out, cap);
}
// prove + verify round trip of the restated verifier (1 = accepted)
int zko_matmul_succinct_roundtrip(const uint32_t* w, const uint32_t* x, const uint32_t* y, size_t m, size_t n, int ef, int tamper) {
    Transcript pt("rt"), vt("rt");
    VF W = vf(w, m * n), X = vf(x, n), Y = vf(y, m);
    if (ef) {
        auto p = prove_matmul_succinct_ef(W, X, Y, m, n, pt);
        if (tamper) p.matmul_proof.x_at_s[0] ^= 1;
        return verify_matmul_succinct_ef(p, Y, m, n, vt).valid;
    }
    auto p = prove_matmul_succinct(W, X, Y, m, n, pt);
    if (tamper) p.matmul_proof.x_at_s ^= 1;
    return verify_matmul_succinct(p, Y, m, n, vt).valid;
}
size_t zko_prove_mle_eval_ef_base_bound(void* t, const uint32_t* w, size_t n, const uint32_t* point, size_t k,
                                        const uint8_t* label, size_t label_len, uint8_t* out, size_t cap, uint32_t* claimed) {
    VF W = vf(w, n);
    WeightCommitment c = commit_weights_fast(padded(W, size_t(1) << k));
    EF cl;
    Bin b; b.put(prove_mle_eval_ef_base_bound(W, vef(point, k), std::string((const char*)label, label_len), c, T(t), &cl));
    cl.to_u32x4(claimed);
    return emit(b.b, out, cap);
}
size_t zko_prove_mle_eval_bound(void* t, const uint32_t* w, size_t n, const uint32_t* point, size_t k,
                                const uint8_t* label, size_t label_len, uint8_t* out, size_t cap, uint32_t* claimed) {
    VF W = vf(w, n);
    WeightCommitment c = commit_weights_fast(padded(W, size_t(1) << k));
    F cl;
    Bin b; b.put(prove_mle_eval_bound(W, vf(point, k), std::string((const char*)label, label_len), c, T(t), &cl));
    *claimed = cl.v;
    return emit(b.b, out, cap);
}
// base-field hadamard (is_add = 0) / add (is_add = 1)
size_t zko_prove_elementwise(void* t, int is_add, const uint32_t* a, const uint32_t* b_, const uint32_t* c, size_t n, const uint32_t* point,
                             size_t k, uint8_t* out, size_t cap) {
    Bin b;
    if (is_add) b.put(prove_add(vf(a, n), vf(b_, n), vf(c, n), vf(point, k), T(t)));
    else b.put(prove_hadamard(vf(a, n), vf(b_, n), vf(c, n), vf(point, k), T(t)));
    return emit(b.b, out, cap);
}
int zko_elementwise_base_roundtrip(int is_add, const uint32_t* a, const uint32_t* b_, const uint32_t* c, size_t n, const uint32_t* point, size_t k,
                              int tamper) {
    Transcript pt("ew"), vt("ew");
    VF pnt = vf(point, k);
    if (is_add) {
        auto p = prove_add(vf(a, n), vf(b_, n), vf(c, n), pnt, pt);
        if (tamper) p.b_fin ^= 1;
        return verify_add(p, pnt, vt);
    }
    auto p = prove_hadamard(vf(a, n), vf(b_, n), vf(c, n), pnt, pt);
    if (tamper) p.fin_a ^= 1;
    return verify_hadamard(p, pnt, vt);
}
size_t zko_prove_hadamard_ef(void* t, const uint32_t* a, const uint32_t* b_, const uint32_t* c, size_t n, const uint32_t* point,
                             size_t k, uint8_t* out, size_t cap) {
    Bin b; b.put(prove_hadamard_ef(vf(a, n), vf(b_, n), vf(c, n), vef(point, k), T(t)));
    return emit(b.b, out, cap);
}
size_t zko_prove_add_ef(void* t, const uint32_t* a, const uint32_t* b_, const uint32_t* c, size_t n, const uint32_t* point,
                        size_t k, uint8_t* out, size_t cap) {
    Bin b; b.put(prove_add_ef(vf(a, n), vf(b_, n), vf(c, n), vef(point, k), T(t)));
    return emit(b.b, out, cap);
}
int zko_elementwise_roundtrip(const uint32_t* a, const uint32_t* b_, const uint32_t* c, size_t n, int is_add, int tamper) {
    Transcript pt("rt"), vt("rt");
    size_t k = log2_ceil(n);
    VEF point = pt.squeeze_ef_many(k);
    vt.squeeze_ef_many(k);
    if (is_add) {
        auto p = prove_add_ef(vf(a, n), vf(b_, n), vf(c, n), point, pt);
        if (tamper) p.c_eval[1] ^= 1;
        return verify_add_ef(p, point, vt);
    }
    auto p = prove_hadamard_ef(vf(a, n), vf(b_, n), vf(c, n), point, pt);
    if (tamper) p.c_eval[1] ^= 1;
    return verify_hadamard_ef(p, point, vt);
}
// out/x_used: d u32 each; returns delta; -1000 on failure
int32_t zko_rmsnorm_forward(const uint32_t* x, const uint32_t* gamma, size_t d, uint32_t* out, uint32_t* x_used) {
    VF o, xu; int32_t delta = 0;
    try { rmsnorm_forward(vf(x, d), vf(gamma, d), o, xu, delta); } catch (const ForwardFailure&) { return -1000; }
    out_f(o, out); out_f(xu, x_used);
    return delta;
}
void zko_requantize(const uint32_t* v, size_t n, uint32_t* out) { out_f(requantize_to_i16_field(vf(v, n)), out); }
size_t zko_prove_rmsnorm_ef(void* t, const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d, int32_t delta,
                            uint8_t* out, size_t cap) {
    Bin b; b.put(prove_rmsnorm_ef(vf(x, d), vf(gamma, d), vf(y, d), delta, T(t)));
    return emit(b.b, out, cap);
}
int zko_rmsnorm_roundtrip(const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d, int32_t delta, int tamper) {
    Transcript pt("rt"), vt("rt");
    auto p = prove_rmsnorm_ef(vf(x, d), vf(gamma, d), vf(y, d), delta, pt);
    if (tamper) p.s_g[0] ^= 1;
    return verify_rmsnorm_ef(p, vf(y, d), d, vt);
}
// returns proof length; 0 with *status = 3 (LogUp identity) or 4 (alpha collision) on the reference's panics
size_t zko_prove_lookup_ef(void* t, const uint32_t* table_out, size_t n_table, const uint32_t* in, const uint32_t* outv, size_t n,
                           uint8_t* out, size_t cap, int* status) {
    *status = 0;
    try {
        Bin b; b.put(prove_lookup_ef(table_from_outputs(std::vector<uint32_t>(table_out, table_out + n_table)), vf(in, n), vf(outv, n), T(t)));
        return emit(b.b, out, cap);
    } catch (const LookupFailure& e) {
        *status = std::string(e.what()).find("alpha") == 0 ? 4 : 3;
        return 0;
    }
}
size_t zko_prove_rmsnorm(void* t, const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d, int32_t delta, uint8_t* out, size_t cap) {
    Bin b; b.put(prove_rmsnorm(vf(x, d), vf(gamma, d), vf(y, d), delta, T(t)));
    return emit(b.b, out, cap);
}
int zko_rmsnorm_base_roundtrip(const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d, int32_t delta, int tamper) {
    Transcript pt("rn"), vt("rn");
    auto p = prove_rmsnorm(vf(x, d), vf(gamma, d), vf(y, d), delta, pt);
    if (tamper == 1) p.s_g ^= 1;
    if (tamper == 2) p.perturbation_delta += 1;
    return verify_rmsnorm(p, vf(y, d), d, vt);
}
size_t zko_prove_lookup(void* t, const uint32_t* table_out, size_t n_table, const uint32_t* in, const uint32_t* outv, size_t n,
                        uint8_t* out, size_t cap, int* status) {
    *status = 0;
    try {
        Bin b; b.put(prove_lookup(table_from_outputs(std::vector<uint32_t>(table_out, table_out + n_table)), vf(in, n), vf(outv, n), T(t)));
        return emit(b.b, out, cap);
    } catch (const LookupFailure& e) {
        *status = std::string(e.what()).find("alpha") == 0 ? 4 : 3;
        return 0;
    }
}
int zko_lookup_base_roundtrip(const uint32_t* table_out, size_t n_table, const uint32_t* in, const uint32_t* outv, size_t n, int tamper) {
    Transcript pt("rt"), vt("rt");
    LookupTable tb = table_from_outputs(std::vector<uint32_t>(table_out, table_out + n_table));
    auto p = prove_lookup(tb, vf(in, n), vf(outv, n), pt);
    if (tamper == 1) p.fin_h ^= 1;
    if (tamper == 2) p.outputs[0] ^= 1;
    return verify_lookup(p, n, vt);
}
int zko_lookup_roundtrip(const uint32_t* table_out, size_t n_table, const uint32_t* in, const uint32_t* outv, size_t n, int tamper) {
    Transcript pt("rt"), vt("rt");
    LookupTable tb = table_from_outputs(std::vector<uint32_t>(table_out, table_out + n_table));
    auto p = prove_lookup_ef(tb, vf(in, n), vf(outv, n), pt);
    if (tamper) p.h_at_s[2] ^= 1;
    return verify_lookup_ef_with_data(p, n, vf(in, n), vf(outv, n), vt);
}

// ---- Qwen layer.  dims = {d_model, d_ff, num_q_heads, num_kv_heads, d_head, v_num_heads, v_d_head};
// weights = {norm1_gamma, w_q, w_k, w_v, w_o, w_g_proj, norm2_gamma, w_gate, w_up, w_down}.
static ModelConfig cfg_of(const uint64_t* d) {
    ModelConfig c;
    c.d_model = d[0]; c.d_ff = d[1]; c.num_q_heads = d[2]; c.num_kv_heads = d[3]; c.d_head = d[4]; c.v_num_heads = d[5]; c.v_d_head = d[6];
    return c;
}
static QwenLayerWeights weights_of(const ModelConfig& c, const uint32_t* const* w) {
    QwenLayerWeights W;
    size_t dm = c.d_model, aod = c.attn_out_dim();
    W.norm1_gamma = vf(w[0], dm); W.w_q = vf(w[1], c.q_dim() * dm); W.w_k = vf(w[2], c.k_dim() * dm);
    W.w_v = vf(w[3], c.v_dim() * dm); W.w_o = vf(w[4], dm * aod); W.w_g_proj = vf(w[5], aod * dm);
    W.norm2_gamma = vf(w[6], dm); W.w_gate = vf(w[7], c.d_ff * dm); W.w_up = vf(w[8], c.d_ff * dm); W.w_down = vf(w[9], dm * c.d_ff);
    return W;
}
// Forward + prove one layer on a fresh transcript seeded as the reference's layer fan-out does
// (label "qwen-layer-{idx}", then the 32-byte hash of the model input).  Writes the layer output
// to y (d_model u32) and the bincode proof to out; returns its length.  verify != 0 also runs
// the restated verifier and stores its verdict in *accepted.
size_t zko_qwen_layer_prove(const uint64_t* dims, const uint32_t* const* weights, const uint32_t* x, const uint32_t* silu_out,
                            const uint32_t* sigmoid_out, size_t n_table, uint32_t layer_idx, const uint8_t* input_hash,
                            uint32_t* y, uint8_t* out, size_t cap, int verify, int* accepted) {
    ModelConfig c = cfg_of(dims);
    QwenLayerWeights W = weights_of(c, weights);
    LookupTable silu = table_from_outputs(std::vector<uint32_t>(silu_out, silu_out + n_table));
    LookupTable sigm = table_from_outputs(std::vector<uint32_t>(sigmoid_out, sigmoid_out + n_table));
    VF X = vf(x, c.d_model);
    QwenForwardTrace t = qwen_forward(X, W, c, silu, sigm);
    out_f(t.output, y);
    std::string seed = "qwen-layer-" + std::to_string(layer_idx);
    Transcript tr(seed);
    tr.absorb_bytes(input_hash, 32);
    QwenLayerProofEF p = prove_qwen_layer_precommitted_ef(t, W, c, commit_qwen_layer(W), silu, sigm, tr);
    if (verify) {
        Transcript vt(seed);
        vt.absorb_bytes(input_hash, 32);
        *accepted = verify_qwen_layer_ef(p, X, t.output, W, c, silu, sigm, vt) ? 1 : 0;
    }
    return emit(serialize(p), out, cap);
}


// A layer kept between calls: weights converted once and committed once, as the reference's
// server does at load time (server.rs:46-94); the reference's prove_time excludes the
// commitments (pipeline/mod.rs:224-229), so whoever times forward + prove uses this handle.
struct OracleLayer {
    ModelConfig c;
    QwenLayerWeights W;
    QwenLayerCommitments com;
    LookupTable silu, sigm;
    QwenForwardTrace trace;      // of the most recent zko_qwen_layer_forward_h
    bool have_trace = false;
};
void* zko_qwen_layer_new(const uint64_t* dims, const uint32_t* const* weights, const uint32_t* silu_out, const uint32_t* sigmoid_out,
                         size_t n_table) {
    OracleLayer* L = new OracleLayer();
    L->c = cfg_of(dims);
    L->W = weights_of(L->c, weights);
    L->silu = table_from_outputs(std::vector<uint32_t>(silu_out, silu_out + n_table));
    L->sigm = table_from_outputs(std::vector<uint32_t>(sigmoid_out, sigmoid_out + n_table));
    L->com = commit_qwen_layer(L->W);
    return L;
}
void zko_qwen_layer_free(void* h) { delete static_cast<OracleLayer*>(h); }
size_t zko_qwen_layer_prove_h(void* h, const uint32_t* x, uint32_t layer_idx, const uint8_t* input_hash, uint32_t* y, uint8_t* out,
                              size_t cap, int verify, int* accepted) {
    OracleLayer& L = *static_cast<OracleLayer*>(h);
    VF X = vf(x, L.c.d_model);
    QwenForwardTrace t = qwen_forward(X, L.W, L.c, L.silu, L.sigm);
    out_f(t.output, y);
    std::string seed = "qwen-layer-" + std::to_string(layer_idx);
    Transcript tr(seed);
    tr.absorb_bytes(input_hash, 32);
    QwenLayerProofEF p = prove_qwen_layer_precommitted_ef(t, L.W, L.c, L.com, L.silu, L.sigm, tr);
    if (verify) {
        Transcript vt(seed);
        vt.absorb_bytes(input_hash, 32);
        *accepted = verify_qwen_layer_ef(p, X, t.output, L.W, L.c, L.silu, L.sigm, vt) ? 1 : 0;
    }
    return emit(serialize(p), out, cap);
}
// The two halves of the call above, as the reference runs them: the forward pass of every layer
// first (pipeline/forward.rs:24), then the layer proofs (pipeline/prove.rs:158-180).
void zko_qwen_layer_forward_h(void* h, const uint32_t* x, uint32_t* y) {
    OracleLayer& L = *static_cast<OracleLayer*>(h);
    L.trace = qwen_forward(vf(x, L.c.d_model), L.W, L.c, L.silu, L.sigm);
    L.have_trace = true;
    out_f(L.trace.output, y);
}
size_t zko_qwen_layer_prove_trace_h(void* h, uint32_t layer_idx, const uint8_t* input_hash, uint8_t* out, size_t cap) {
    OracleLayer& L = *static_cast<OracleLayer*>(h);
    if (!L.have_trace) return 0;
    Transcript tr("qwen-layer-" + std::to_string(layer_idx));
    tr.absorb_bytes(input_hash, 32);
    return emit(serialize(prove_qwen_layer_precommitted_ef(L.trace, L.W, L.c, L.com, L.silu, L.sigm, tr)), out, cap);
}
// Decode a layer proof and run the restated verifier on it (the layer's own forward pass of x supplies the
// trace).  1 accept, 0 reject, -1 the bytes do not decode.
int zko_qwen_layer_verify_bytes_h(void* h, const uint32_t* x, uint32_t layer_idx, const uint8_t* input_hash, const uint32_t* y_expected,
                                  const uint8_t* bytes, size_t len) {
    OracleLayer& L = *static_cast<OracleLayer*>(h);
    QwenLayerProofEF p;
    Rd rd{bytes, len};
    if (!rd.get(p)) return -1;
    Transcript vt("qwen-layer-" + std::to_string(layer_idx));
    vt.absorb_bytes(input_hash, 32);
    VF X = vf(x, L.c.d_model), Y = vf(y_expected, L.c.d_model);
    return verify_qwen_layer_ef(p, X, Y, L.W, L.c, L.silu, L.sigm, vt) ? 1 : 0;
}
// ---- op lists (oplist.hpp): built call by call, then forward + prove in one go -------------------
struct OracleOpList { std::vector<Op> ops; };
void* zko_oplist_new() { return new OracleOpList(); }
void zko_oplist_free(void* h) { delete static_cast<OracleOpList*>(h); }
static Op& new_op(void* h, const char* type, const char* name) {
    auto& L = *static_cast<OracleOpList*>(h);
    L.ops.emplace_back();
    L.ops.back().type = type; L.ops.back().name = name;
    return L.ops.back();
}
void zko_oplist_linear(void* h, const char* name, const uint32_t* w, const uint32_t* b, size_t m, size_t n) {
    Op& o = new_op(h, "linear", name);
    o.m = m; o.n = n; o.w = vf(w, m * n); o.b = b ? vf(b, m) : VF();
}
void zko_oplist_simple(void* h, const char* type, const char* name, const char* aux) {   // relu, attention, passthrough, save (aux = save_name), add_saved (aux = add_name)
    Op& o = new_op(h, type, name);
    if (o.type == "save") o.save_name = aux;
    if (o.type == "add_saved") o.add_name = aux;
}
void zko_oplist_layernorm(void* h, const char* name, const uint32_t* gamma, const uint32_t* beta, size_t d) {
    Op& o = new_op(h, "layernorm", name);
    o.gamma = vf(gamma, d); o.beta = vf(beta, d);
}
void zko_oplist_gelu(void* h, const char* name, const uint32_t* in, const uint32_t* out, size_t n, const uint32_t* table_out, size_t n_table) {
    Op& o = new_op(h, "gelu", name);
    o.gelu_in = vf(in, n); o.gelu_out = vf(out, n);
    o.table_out.assign(table_out, table_out + n_table);
}
void zko_oplist_attention(void* h, const char* name, size_t heads, size_t kv_heads, size_t seq, size_t d_head, const uint32_t* table_out,
                          size_t n_table, const uint32_t* k, const uint32_t* v) {
    Op& o = new_op(h, "attention_rows", name);
    o.heads = heads; o.kv_heads = kv_heads; o.seq = seq; o.d_head = d_head;
    o.table_out.assign(table_out, table_out + n_table);
    const size_t nkv = (kv_heads ? kv_heads : heads) * seq * d_head;
    if (k) { o.att_k = vf(k, nkv); o.att_v = vf(v, nkv); }
}
void zko_oplist_set_input(void* h, const char* name, const uint32_t* v, size_t n) {
    Op& o = new_op(h, "set_input", name);
    o.new_input = vf(v, n);
}
// Forward pass only: the activation after op `upto` (0-based) into out (returns its length).
size_t zko_oplist_forward(void* h, const uint32_t* x, size_t n, size_t upto, uint32_t* out, size_t cap) {
    auto& L = *static_cast<OracleOpList*>(h);
    std::vector<Op> head(L.ops.begin(), L.ops.begin() + (upto + 1 < L.ops.size() ? upto + 1 : L.ops.size()));
    auto layers = oplist_forward(head, vf(x, n));
    const VF& y = layers.back().output;
    if (y.size() <= cap) out_f(y, out);
    return y.size();
}
// Forward + prove: bincode(Vec<SerializedLayerProof>) in the reference's push order.
size_t zko_oplist_prove(void* h, const uint32_t* x, size_t n, uint8_t* out, size_t cap) {
    auto& L = *static_cast<OracleOpList*>(h);
    auto layers = oplist_forward(L.ops, vf(x, n));
    return emit(oplist_prove(layers), out, cap);
}
// prove + verify round trip of the squared LayerNorm (1 = accepted); tamper flips one proof field.
int zko_layernorm_sqr_roundtrip(const uint32_t* x, const uint32_t* gamma, const uint32_t* beta, size_t d, int tamper) {
    VF X = vf(x, d), G = vf(gamma, d), B = vf(beta, d);
    LnForward f = layernorm_forward_simple(X, G, B);
    VF xu = X;
    if (f.perturbation != 0) xu[0] = xu[0] + (f.perturbation > 0 ? F(uint32_t(f.perturbation)) : F::zero() - F(uint32_t(-f.perturbation)));
    Transcript pt("ln"), vt("ln");
    LayerNormSqrProof p = prove_layernorm_sqr(xu, G, B, f.y, f.mu, pt);
    if (tamper == 1) p.s_h ^= 1;
    if (tamper == 2) p.mu ^= 1;
    if (tamper == 3) p.g_sq_fin[1] ^= 1;
    VF y = f.y;
    if (tamper == 4) y[0] = y[0] + F::one();
    return verify_layernorm_sqr(p, y, B, d, vt) ? 1 : 0;
}

// Worker threads of the row-parallel matrix loops (matmul.hpp); 1 = serial.
void zko_set_threads(int n) { matrix_threads() = n < 1 ? 1 : n; }

// ---- row attention, seq_len >= 2 (attention.rs:116-385; with num_kv_heads != 0 the GQA form, :386-590).
// q: (num_heads, seq_len, d_head); k, v: (num_kv_heads or num_heads, seq_len, d_head).
// status: 0 ok, 8 a score outside the exp table's domain or a zero softmax denominator (the reference panics on either).
size_t zko_prove_row_attention(void* t, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t num_kv_heads, size_t seq_len,
                               size_t d_head, const uint32_t* table_out, size_t n_table, uint8_t* out, size_t cap, int* status) {
    size_t n = num_heads * seq_len * d_head, nkv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
    bool ok = true;
    *status = 0;
    LookupTable tb = table_from_outputs(std::vector<uint32_t>(table_out, table_out + n_table));
    try {
        SeqAttentionProof P = prove_row_attention(vf(q, n), vf(k, nkv), vf(v, nkv), num_heads, seq_len, d_head, tb, T(t), &ok, num_kv_heads);
        if (!ok) { *status = 8; return 0; }
        Bin b; put(b, P);
        return emit(b.b, out, cap);
    } catch (const LookupFailure& e) {
        *status = std::string(e.what()).find("alpha") == 0 ? 4 : 3;
        return 0;
    }
}
int zko_row_attention_forward(const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t num_kv_heads, size_t seq_len,
                              size_t d_head, const uint32_t* table_out, size_t n_table, uint32_t* out) {
    size_t n = num_heads * seq_len * d_head, nkv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
    bool ok = true;
    LookupTable tb = table_from_outputs(std::vector<uint32_t>(table_out, table_out + n_table));
    out_f(row_attention_forward(vf(q, n), vf(k, nkv), vf(v, nkv), num_heads, seq_len, d_head, tb, &ok, num_kv_heads), out);
    return ok ? 0 : 8;
}
// prove -> verify on fresh transcripts; tamper: 1 a score, 2 an output word, 3 the softmax sum, 4 a y value's matmul final
int zko_row_attention_roundtrip(const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t num_kv_heads, size_t seq_len,
                                size_t d_head, const uint32_t* table_out, size_t n_table, int tamper) {
    size_t n = num_heads * seq_len * d_head, nkv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
    bool ok = true;
    LookupTable tb = table_from_outputs(std::vector<uint32_t>(table_out, table_out + n_table));
    Transcript pt("attn"), vt("attn");
    SeqAttentionProof P = prove_row_attention(vf(q, n), vf(k, nkv), vf(v, nkv), num_heads, seq_len, d_head, tb, pt, &ok, num_kv_heads);
    if (!ok) return -1;
    RowProof& rp = P.row_proofs[num_heads - 1][seq_len - 1];
    if (tamper == 1) rp.scores[0] ^= 1;
    if (tamper == 2) rp.output[0] ^= 1;
    if (tamper == 3) rp.softmax_proof.sum_value ^= 1;
    if (tamper == 4) rp.output_proof.x_at_s ^= 1;
    bool good = verify_row_attention(P, vf(k, nkv), vf(v, nkv), vt, num_kv_heads);
    return good && pt.squeeze().v == vt.squeeze().v;
}

// Decode bincode(RowAttentionProof) and run verify_row_attention (attention.rs:279-385; GQA :503-590) on it with the caller's dimensions.
// 1 accept, 0 reject, -1 the bytes do not decode.
static void rd_sumcheck(Rd& r, SumcheckProof& p) {
    size_t k = r.len(8);
    p.round_polys.clear();
    for (size_t i = 0; i < k && r.ok; i++) { p.round_polys.emplace_back(); r.vec_u32(p.round_polys.back()); }
    r.vec_u32(p.challenges);
}
static void rd_matmul(Rd& r, MatmulProof& p) { rd_sumcheck(r, p.sumcheck_proof); p.w_at_rs = r.u32(); p.x_at_s = r.u32(); r.vec_u32(p.r_point); r.vec_u32(p.s_point); }
int zko_row_attention_verify_bytes(void* t, const uint8_t* b, size_t n, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t num_kv_heads,
                                   size_t seq_len, size_t d_head) {
    Rd r{b, n};
    SeqAttentionProof P;
    size_t nh = r.len(8);
    for (size_t h = 0; h < nh && r.ok; h++) {
        size_t ns = r.len(8);
        P.row_proofs.emplace_back();
        for (size_t i = 0; i < ns && r.ok; i++) {
            RowProof rp;
            rd_matmul(r, rp.score_proof);
            LookupProof& lk = rp.softmax_proof.exp_lookup_proof;
            r.get(lk.table_commitment); r.get(lk.multiplicity_commitment);
            rd_sumcheck(r, lk.sumcheck_proof);
            lk.fin_ones = r.u32(); lk.fin_h = r.u32(); lk.alpha = r.u32(); lk.beta = r.u32();
            r.vec_u32(lk.inputs); r.vec_u32(lk.outputs); r.vec_u32(lk.multiplicities);
            r.bytes(lk.external_data_digest);
            SoftmaxProof& sp = rp.softmax_proof;
            sp.sum_value = r.u32();
            rd_sumcheck(r, sp.sum_proof); sp.sum_finals[0] = r.u32(); sp.sum_finals[1] = r.u32();
            rd_sumcheck(r, sp.output_proof); for (int j = 0; j < 3; j++) sp.output_finals[j] = r.u32();
            sp.inv_s = r.u32();
            r.vec_u32(sp.e_values); r.vec_u32(sp.y_values);
            rd_matmul(r, rp.output_proof);
            r.vec_u32(rp.scores); r.vec_u32(rp.attn_weights); r.vec_u32(rp.output);
            P.row_proofs.back().push_back(std::move(rp));
        }
    }
    P.num_heads = r.u64(); P.seq_len = r.u64(); P.d_head = r.u64();
    uint8_t opt = r.u8();
    if (opt == 1) { r.u32(); r.u32(); r.u8(); } else if (opt != 0) return -1;
    if (!r.ok || r.at != n) return -1;
    // the caller's dimensions are those of k and v; a proof that declares others, or holds a different number of rows, makes the reference index out of range
    if (P.num_heads != num_heads || P.seq_len != seq_len || P.d_head != d_head || P.row_proofs.size() != num_heads) return 0;
    for (auto& hp : P.row_proofs) if (hp.size() != seq_len) return 0;
    size_t nkv = (num_kv_heads ? num_kv_heads : num_heads) * seq_len * d_head;
    return verify_row_attention(P, vf(k, nkv), vf(v, nkv), T(t), num_kv_heads) ? 1 : 0;
}

}  // extern "C"
