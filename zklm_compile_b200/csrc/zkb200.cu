// C ABI of the backend (see include/zkb200.h) and the host-side launch logic.
#include "qwen.cuh"
#include "oplist.cuh"
#include "basefold.cuh"
#include "verify.cuh"
#include "verify_batch.cuh"
#include "attention.cuh"
#include "verify_attention.cuh"
#include "verify_layer.cuh"
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

using namespace zkb;

// =============================================================================================
// C ABI
// =============================================================================================
#define ZKB_TRY(ctxptr, ...)                                                         \
    try { __VA_ARGS__; return ZKB_OK; }                                                     \
    catch (const CudaFail& e) { if (ctxptr) (ctxptr)->err = e.msg; return ZKB_E_CUDA; } \
    catch (const ArgFail& e) { if (ctxptr) (ctxptr)->err = e.msg; return e.code; }   \
    catch (const std::bad_alloc&) { if (ctxptr) (ctxptr)->err = "host allocation failed"; return ZKB_E_CUDA; }

// Pointers that kernels read with 16-byte loads: checked on the host, before anything is
// launched, because a misaligned address on the device is a sticky context error, not a status.
static inline void need_align16(const void* p, const char* what) {
    if ((uintptr_t)p & 15) throw ArgFail{ZKB_E_ARG, std::string(what) + " must be 16-byte aligned (it is read with 16-byte loads)"};
}

extern "C" {

int32_t zkb_ctx_create(int32_t device, zkb_ctx** out) {
    if (!out) return ZKB_E_ARG;
    *out = nullptr;
    zkb_ctx* c = new (std::nothrow) zkb_ctx();
    if (!c) return ZKB_E_CUDA;
    c->device = device;
    // one hardware work queue per stream (up to 32), so per-layer streams do not share a queue
    setenv("CUDA_DEVICE_MAX_CONNECTIONS", "32", 0);
    try {
        int count = 0;
        ZKB_CUDA(cudaGetDeviceCount(&count));
        if (device < 0 || device >= count) throw ArgFail{ZKB_E_ARG, "no such CUDA device"};
        c->use();
        cudaDeviceProp prop;
        ZKB_CUDA(cudaGetDeviceProperties(&prop, device));
        c->sm_count = prop.multiProcessorCount;
        ZKB_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        ZKB_CUDA(cudaMalloc(&c->partials, SC_MAX_GRID * 16 * sizeof(u32)));
        ZKB_CUDA(cudaMalloc(&c->counter, 64));
        ZKB_CUDA(cudaMemsetAsync(c->counter, 0, 64, c->stream));
        ZKB_CUDA(cudaMalloc(&c->status, 64));
        ZKB_CUDA(cudaMemsetAsync(c->status, 0, 64, c->stream));
        c->rec_cap = size_t(1) << 21;                       // 8 MiB of proof record (a layer with eight Basefold openings needs ~4)
        ZKB_CUDA(cudaMalloc(&c->rec_dev, c->rec_cap * 4));
        ZKB_CUDA(cudaHostAlloc(&c->rec_host, c->rec_cap * 4, cudaHostAllocDefault));
        ZKB_CUDA(cudaEventCreate(&c->t0));
        ZKB_CUDA(cudaEventCreate(&c->t1));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    } catch (const CudaFail& e) {
        fprintf(stderr, "zkb_ctx_create: %s\n", e.msg.c_str());
        delete c;
        return ZKB_E_CUDA;
    } catch (const ArgFail& e) {
        delete c;
        return e.code;
    }
    *out = c;
    return ZKB_OK;
}

void zkb_ctx_destroy(zkb_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (auto& ch : c->chunks) cudaFree(ch.base);
    for (auto e : c->prof_events) cudaEventDestroy(e);
    for (auto& r : c->ranges) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    for (auto e : c->ev_pool) cudaEventDestroy(e);
    if (c->partials) cudaFree(c->partials);
    if (c->counter) cudaFree(c->counter);
    if (c->status) cudaFree(c->status);
    if (c->rec_dev) cudaFree(c->rec_dev);
    if (c->rec_host) cudaFreeHost(c->rec_host);
    if (c->t0) cudaEventDestroy(c->t0);
    if (c->t1) cudaEventDestroy(c->t1);
    for (cudaEvent_t e : c->side_ev) cudaEventDestroy(e);
    if (c->side) cudaStreamDestroy(c->side);
    if (c->stage) cudaFreeHost(c->stage);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

const char* zkb_last_error(const zkb_ctx* c) { return c ? c->err.c_str() : "null context"; }
uint64_t zkb_launch_count(const zkb_ctx* c) { return c ? c->launches : 0; }

void* zkb_ctx_stream(zkb_ctx* c) { return c ? (void*)c->stream : nullptr; }

int32_t zkb_ctx_sync(zkb_ctx* c) {
    if (!c) return ZKB_E_ARG;
    ZKB_TRY(c, { c->use(); ZKB_CUDA(cudaStreamSynchronize(c->stream)); });
}
int32_t zkb_timer_start(zkb_ctx* c) {
    if (!c) return ZKB_E_ARG;
    ZKB_TRY(c, { c->use(); ZKB_CUDA(cudaEventRecord(c->t0, c->stream)); });
}
int32_t zkb_timer_stop_ms(zkb_ctx* c, float* ms) {
    if (!c || !ms) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaEventRecord(c->t1, c->stream));
        ZKB_CUDA(cudaEventSynchronize(c->t1));
        ZKB_CUDA(cudaEventElapsedTime(ms, c->t0, c->t1));
    });
}
int32_t zkb_profile_enable(zkb_ctx* c, int32_t on) {
    if (!c) return ZKB_E_ARG;
    c->profile = on != 0;
    c->prof_used = 0;
    return ZKB_OK;
}
int32_t zkb_profile_read(zkb_ctx* c, float* ms, size_t cap, size_t* n) {
    if (!c || !n) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        size_t cnt = c->prof_used > 0 ? c->prof_used - 1 : 0;
        *n = cnt;
        for (size_t i = 0; i < cnt && i < cap; i++)
            ZKB_CUDA(cudaEventElapsedTime(ms + i, c->prof_events[i], c->prof_events[i + 1]));
    });
}

#ifdef ZKB_STAMP
// Experiment build only: copies the stamp records out (5 x u64 each: key, t0, t1, kind, smid) and resets the ring.
extern "C" int32_t zkb_dbg_stamps(uint64_t* out, size_t cap, size_t* n) {
    unsigned cnt = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&cnt, zkb::g_stamp_n, 4);
    if (cnt > zkb::STAMP_CAP) cnt = zkb::STAMP_CAP;
    std::vector<zkb::StampRec> h(cnt);
    if (cnt) cudaMemcpyFromSymbol(h.data(), zkb::g_stamps, sizeof(zkb::StampRec) * cnt);
    size_t k = 0;
    for (; k < cnt && k < cap; k++) {
        out[5 * k] = (uint64_t)h[k].key; out[5 * k + 1] = h[k].t0; out[5 * k + 2] = h[k].t1; out[5 * k + 3] = h[k].kind; out[5 * k + 4] = h[k].smid;
    }
    *n = k;
    unsigned zero = 0;
    cudaMemcpyToSymbol(zkb::g_stamp_n, &zero, 4);
    return 0;
}
#endif
int32_t zkb_trace_enable(zkb_ctx* c, int32_t on) {
    if (!c) return ZKB_E_ARG;
    c->trace = on != 0;
    c->trace_clear();
    return ZKB_OK;
}
int32_t zkb_trace_dump(zkb_ctx* c, zkb_ctx* base, const char* path) {
    if (!c || !path) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        FILE* f = fopen(path, "w");
        if (!f) throw zkb::ArgFail{ZKB_E_ARG, "cannot open the trace file"};
        const zkb_ctx* b = (base && !base->trace_log.empty()) ? base : c;
        fprintf(f, "index,site,ms\n");
        for (size_t i = 0; i < c->trace_log.size(); i++) {
            float t = 0;
            cudaError_t e = cudaEventElapsedTime(&t, b->trace_log[0].ev, c->trace_log[i].ev);
            if (e != cudaSuccess) { cudaGetLastError(); t = -1.f; }
            const char* file = c->trace_log[i].file;
            const char* slash = strrchr(file, '/');
            fprintf(f, "%zu,%s:%d,%.4f\n", i, slash ? slash + 1 : file, c->trace_log[i].line, t);
        }
        fclose(f);
    });
}

int32_t zkb_profile_ranges(zkb_ctx* c, double* ms, double* bytes, uint64_t* count) {
    if (!c || !ms || !bytes || !count) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        for (int i = 0; i < ZKB_RANGE_COUNT; i++) { ms[i] = 0; bytes[i] = 0; count[i] = 0; }
        for (auto& r : c->ranges) {
            float t = 0;
            ZKB_CUDA(cudaEventElapsedTime(&t, r.a, r.b));
            if (r.tag >= 0 && r.tag < ZKB_RANGE_COUNT) { ms[r.tag] += t; bytes[r.tag] += r.bytes; count[r.tag]++; }
            c->ev_pool.push_back(r.a);
            c->ev_pool.push_back(r.b);
        }
        c->ranges.clear();
    });
}

// ---- buffers
int32_t zkb_buf_alloc(zkb_ctx* c, size_t n, uint32_t** out) {
    if (!c || !out) return ZKB_E_ARG;
    ZKB_TRY(c, { c->use(); ZKB_CUDA(cudaMalloc(out, (n ? n : 1) * sizeof(u32))); });
}
int32_t zkb_buf_upload_u32(zkb_ctx* c, const uint32_t* host, size_t n, uint32_t* dst) {
    if (!c || (!host && n) || (!dst && n)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaMemcpyAsync(dst, host, n * sizeof(u32), cudaMemcpyHostToDevice, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    });
}
int32_t zkb_buf_download_u32(zkb_ctx* c, const uint32_t* src, size_t n, uint32_t* host) {
    if (!c || (!host && n) || (!src && n)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaMemcpyAsync(host, src, n * sizeof(u32), cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    });
}
int32_t zkb_buf_free(zkb_ctx* c, uint32_t* dev) {
    if (!c) return ZKB_E_ARG;
    ZKB_TRY(c, { c->use(); ZKB_CUDA(cudaStreamSynchronize(c->stream)); ZKB_CUDA(cudaFree(dev)); });
}

int32_t zkb_host_alloc(zkb_ctx* c, size_t bytes, void** out) {
    if (!c || !out) return ZKB_E_ARG;
    ZKB_TRY(c, { c->use(); ZKB_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault)); });
}
int32_t zkb_host_free(zkb_ctx* c, void* host) {
    if (!c) return ZKB_E_ARG;
    ZKB_TRY(c, { c->use(); ZKB_CUDA(cudaFreeHost(host)); });
}

// ---- transcript
int32_t zkb_tr_new(zkb_ctx* c, const uint8_t* label, size_t len, zkb_transcript** out) {
    if (!c || !out || (!label && len)) return ZKB_E_ARG;
    *out = nullptr;
    zkb_transcript* t = new (std::nothrow) zkb_transcript{c, nullptr};
    if (!t) return ZKB_E_CUDA;
    try {
        c->use();
        ZKB_CUDA(cudaMalloc(&t->dev, sizeof(TrState)));
        tr_init_kernel<<<1, 1, 0, c->stream>>>(t->dev);
        c->launches++;
        ZKB_CUDA(cudaGetLastError());
    } catch (const CudaFail& e) {
        c->err = e.msg;
        delete t;
        return ZKB_E_CUDA;
    }
    *out = t;
    return zkb_tr_absorb_bytes(t, label, len);
}
void zkb_tr_free(zkb_transcript* t) {
    if (!t) return;
    cudaSetDevice(t->ctx->device);
    cudaStreamSynchronize(t->ctx->stream);
    cudaFree(t->dev);
    delete t;
}
int32_t zkb_tr_absorb_bytes(zkb_transcript* t, const uint8_t* bytes, size_t n) {
    if (!t || (!bytes && n)) return ZKB_E_ARG;
    zkb_ctx* c = t->ctx;
    ZKB_TRY(c, {
        c->use();
        for (size_t off = 0; off < n; off += 256) {
            ByteChunk ch;
            size_t m = n - off < 256 ? n - off : 256;
            memcpy(ch.b, bytes + off, m);
            tr_absorb_bytes_kernel<<<1, 1, 0, c->stream>>>(t->dev, ch, (u32)m);
            c->launches++;
        }
        ZKB_CUDA(cudaGetLastError());
    });
}
int32_t zkb_tr_absorb_u32(zkb_transcript* t, uint32_t v) {
    uint8_t b[4] = {(uint8_t)v, (uint8_t)(v >> 8), (uint8_t)(v >> 16), (uint8_t)(v >> 24)};
    return zkb_tr_absorb_bytes(t, b, 4);
}
int32_t zkb_tr_absorb_many_dev(zkb_transcript* t, const uint32_t* dev, size_t n) {
    if (!t || (!dev && n)) return ZKB_E_ARG;
    zkb_ctx* c = t->ctx;
    ZKB_TRY(c, {
        c->use();
        if (n) {
            tr_absorb_words_kernel<<<1, 32, 0, c->stream>>>(t->dev, dev, n);
            c->launches++;
            ZKB_CUDA(cudaGetLastError());
        }
    });
}
int32_t zkb_tr_absorb_many(zkb_transcript* t, const uint32_t* host, size_t n) {
    if (!t || (!host && n)) return ZKB_E_ARG;
    zkb_ctx* c = t->ctx;
    ZKB_TRY(c, {
        c->use();
        if (n) {
            u32* d = (u32*)c->scratch(n * 4);
            ZKB_CUDA(cudaMemcpyAsync(d, host, n * 4, cudaMemcpyHostToDevice, c->stream));
            tr_absorb_words_kernel<<<1, 32, 0, c->stream>>>(t->dev, d, n);
            c->launches++;
            ZKB_CUDA(cudaGetLastError());
            ZKB_CUDA(cudaStreamSynchronize(c->stream));
            c->scratch_reset();
        }
    });
}
static int32_t squeeze_n(zkb_transcript* t, uint32_t* out, u32 count) {
    if (!t || !out) return ZKB_E_ARG;
    zkb_ctx* c = t->ctx;
    ZKB_TRY(c, {
        c->use();
        u32* d = c->status + 8;   // 8 spare words after the status word
        tr_squeeze_kernel<<<1, 1, 0, c->stream>>>(t->dev, d, count);
        c->launches++;
        ZKB_CUDA(cudaGetLastError());
        ZKB_CUDA(cudaMemcpyAsync(out, d, count * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    });
}
int32_t zkb_tr_squeeze(zkb_transcript* t, uint32_t* out) { return squeeze_n(t, out, 1); }
int32_t zkb_tr_squeeze_ef(zkb_transcript* t, uint32_t out[4]) { return squeeze_n(t, out, 4); }
int32_t zkb_tr_export(zkb_transcript* t, uint8_t state[ZKB_TR_STATE_BYTES]) {
    if (!t || !state) return ZKB_E_ARG;
    static_assert(sizeof(TrState) == ZKB_TR_STATE_BYTES, "transcript state layout");
    zkb_ctx* c = t->ctx;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaMemcpyAsync(state, t->dev, sizeof(TrState), cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    });
}
int32_t zkb_tr_import(zkb_transcript* t, const uint8_t state[ZKB_TR_STATE_BYTES]) {
    if (!t || !state) return ZKB_E_ARG;
    zkb_ctx* c = t->ctx;
    ZKB_TRY(c, {
        c->use();
        ZKB_CUDA(cudaMemcpyAsync(t->dev, state, sizeof(TrState), cudaMemcpyHostToDevice, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
    });
}

// ---- sumcheck
// Launch shapes for a context that shares the GPU with many others (see zkb_ctx::polite).
int32_t zkb_ctx_set_shared(zkb_ctx* c, int32_t on) {
    if (!c) return ZKB_E_ARG;
    c->polite = on != 0;
    c->arena_epoch++;                  // captured graphs hold the old launch shapes
    return ZKB_OK;
}

int32_t zkb_ctx_trim(zkb_ctx* c) {
    if (!c) return ZKB_E_ARG;
    ZKB_TRY(c, { c->use(); c->scratch_trim(); });
}
uint64_t zkb_ctx_scratch_bytes(const zkb_ctx* c) { return c ? (uint64_t)c->scratch_capacity() : 0; }

int32_t zkb_ctx_set_option(zkb_ctx* c, int32_t option, int32_t value) {
    if (!c) return ZKB_E_ARG;
    switch (option) {
        case ZKB_OPT_PLAIN_TAIL: c->opt_plain_tail = value != 0; break;
        case ZKB_OPT_SINGLE_CTA_THREADS:
            if (value != 0 && (value < 64 || value > 1024 || value % 32)) { c->err = "single-CTA thread count must be 0 or a multiple of 32 in [64, 1024]"; return ZKB_E_ARG; }
            c->opt_single_threads = value; break;
        case ZKB_OPT_PIPE_THREADS:
            if (value != 0 && (value < 96 || value > PIPE_THREADS || value % 32)) { c->err = "pipelined-tail thread count must be 0 or a multiple of 32 in [96, 512]"; return ZKB_E_ARG; }
            c->opt_pipe_threads = value; break;
        case ZKB_OPT_NO_FUSED_FOLD: c->opt_no_fused2 = value != 0; break;
        case ZKB_OPT_BASEFOLD_IN_ORDER: c->opt_bf_in_order = value != 0; break;
        case ZKB_OPT_MATVEC_RING: c->opt_mv_ring = value != 0; break;
        case ZKB_OPT_SHARED_SM_HASH:
            if (value != 0 && value != 1 && (value < 16 || value > 200)) return ZKB_E_ARG;
            c->opt_shared_sm = (int)value;
            break;
        case ZKB_OPT_ATTENTION_THREADS:
            if (value != 0 && value != 64 && value != 128 && value != 256) return ZKB_E_ARG;
            c->opt_att_threads = (int)value;
            break;
        case ZKB_OPT_MATVEC_PREFETCH_ROWS:
            if (value < 0 || value > 8) return ZKB_E_ARG;
            c->opt_mv_prefetch = (int)value;
            break;
        case ZKB_OPT_FOLD2_VEC:
            if (value != 0 && value != 1 && value != 2 && value != 4) { c->err = "fold2 vector width must be 0, 1, 2 or 4"; return ZKB_E_ARG; }
            c->opt_fold2_vec = value; break;
        default: c->err = "unknown option"; return ZKB_E_ARG;
    }
    c->arena_epoch++;                  // captured graphs hold the old launch shapes
    return ZKB_OK;
}

int32_t zkb_sumcheck_prove(zkb_ctx* c, zkb_transcript* t, int32_t kind, const uint32_t* const* tables,
                           uint32_t num_vars, int32_t on_device, uint32_t* round_polys, uint32_t* challenges,
                           uint32_t* finals) {
    if (!c || !t || !tables || !round_polys || !challenges || !finals) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        KindInfo ki = kind_info(kind);
        if (num_vars < 1 || num_vars > 34) throw ArgFail{ZKB_E_ARG, "num_vars out of range"};
        const size_t n = size_t(1) << num_vars;
        const u32* dev_tabs[3] = {nullptr, nullptr, nullptr};
        for (int i = 0; i < ki.nt; i++) {
            if (!tables[i]) throw ArgFail{ZKB_E_ARG, "null table"};
            if (on_device) {
                if (ki.in_w[i] == 4) need_align16(tables[i], "an extension-field table");
                dev_tabs[i] = tables[i];
            } else {
                u32* d = (u32*)c->scratch(n * 4 * ki.in_w[i]);
                ZKB_CUDA(cudaMemcpyAsync(d, tables[i], n * 4 * ki.in_w[i], cudaMemcpyHostToDevice, c->stream));
                dev_tabs[i] = d;
            }
        }
        c->rec_reset();
        ScRec r = sumcheck_enqueue(c, t->dev, kind, dev_tabs, num_vars);
        c->rec_fetch();
        const u32* rec = c->rec_host;
        size_t k = 0;
        for (u32 round = 0; round < num_vars; round++)
            for (u32 e = 0; e < ki.nabs; e++)
                if (ki.mask & (1u << e))
                    for (int wd = 0; wd < ki.w; wd++) round_polys[k++] = rec[r.polys + ((size_t)round * ki.nabs + e) * ki.w + wd];
        memcpy(challenges, rec + r.chal, (size_t)num_vars * ki.w * 4);
        if (ki.nt == 1) {   // f == 1: first final is the constant one (sumcheck.rs:901, 1434); the kernel writes g(s) to slot 0
            memset(finals, 0, ki.w * 4);
            finals[0] = 1;
            memcpy(finals + ki.w, rec + r.fin, ki.w * 4);
        } else {
            memcpy(finals, rec + r.fin, (size_t)ki.nt * ki.w * 4);
        }
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

}  // extern "C"

#include "abi_protocols.cuh"
#include "abi_field.cuh"
#include "abi_layer.cuh"
#include "abi_pcs.cuh"
#include "abi_split.cuh"
#include "abi_oplist.cuh"
#include "abi_weights.cuh"
#include "abi_attention.cuh"
#include "abi_pcs_batch.cuh"

// =============================================================================================
// Allocation-free weight fold
// =============================================================================================
// Some callers may not allocate device memory at all: code running inside a CUDA-graph capture
// or a real-time inference loop whose memory plan was fixed at start-up, and hosts that hand
// this library a pre-carved arena and forbid cudaMalloc afterwards (an allocation can
// synchronise the device and fragment their pool).  For them this one entry point does the
// weight fold  out[j] = sum_i eq[i] * W[i][j]  (EF weights eq, base-field matrix W) without
// allocating: the 64-bit column accumulators that the regular path takes from the context's
// arena live in the fixed array below, which every GPU that loads the library holds until exit.
constexpr size_t ZKB_NOALLOC_MAX_COLS = 16384;                                  // padded column count
static __device__ __align__(256) unsigned long long g_noalloc_fold_acc[ZKB_NOALLOC_MAX_COLS * 4];   // 512 KiB

namespace {
struct NoallocDev { unsigned long long* acc = nullptr; int sm_count = 0; bool ready = false; };
NoallocDev g_noalloc_dev[64];
std::mutex g_noalloc_mu;

void set_err(char* err, size_t cap, const std::string& msg) {
    if (err && cap) { size_t n = msg.size() < cap - 1 ? msg.size() : cap - 1; memcpy(err, msg.data(), n); err[n] = 0; }
}
}  // namespace

extern "C" int32_t zkb_fold_eq_matvec_ef_noalloc(const uint32_t* W_dev, size_t m, size_t n, const uint32_t* eq_dev, uint32_t* out_dev,
                                                 void* stream, char* err, size_t err_cap) {
    if (!W_dev || !eq_dev || !out_dev || m == 0 || n == 0) { set_err(err, err_cap, "null pointer or empty matrix"); return ZKB_E_ARG; }
    if (n % 4 == 0 && ((uintptr_t)W_dev & 15)) {
        set_err(err, err_cap, "zkb_fold_eq_matvec_ef_noalloc: W_dev must be 16-byte aligned when n is a multiple of 4 (rows are read with 16-byte loads)");
        return ZKB_E_ARG;
    }
    const size_t n_pad = size_t(1) << log2_ceil_u(n);
    if (n_pad > ZKB_NOALLOC_MAX_COLS) {
        set_err(err, err_cap, "zkb_fold_eq_matvec_ef_noalloc: " + std::to_string(n) + " columns pad to " + std::to_string(n_pad) +
                                  ", above the fixed scratch capacity of " + std::to_string(ZKB_NOALLOC_MAX_COLS) + " columns");
        return ZKB_E_TOO_LARGE;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) { set_err(err, err_cap, std::string("cudaGetDevice: ") + cudaGetErrorString(e)); return ZKB_E_CUDA; }
    NoallocDev& D = g_noalloc_dev[dev];
    {   // first call on this device: resolve the device address of the scratch array (the name
        // itself is only a host-side handle) with this device current
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (!D.ready) {
            unsigned long long* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_noalloc_fold_acc);
            if (e != cudaSuccess || !p) { set_err(err, err_cap, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e)); return ZKB_E_CUDA; }
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess || sms <= 0) { set_err(err, err_cap, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e)); return ZKB_E_CUDA; }
            D.acc = p; D.sm_count = sms; D.ready = true;
        }
    }
    cudaStream_t s = (cudaStream_t)stream;
    // the array keeps whatever the previous call left: the accumulators must start at zero
    e = cudaMemsetAsync(D.acc, 0, n_pad * 4 * sizeof(unsigned long long), s);
    if (e != cudaSuccess) { set_err(err, err_cap, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e)); return ZKB_E_CUDA; }
    size_t rows_per = 0;
    dim3 grid = fold_launch_dims(D.sm_count, m, n, &rows_per);
    fold_eq_matvec_kernel<4, true><<<fold_grid(grid, D.sm_count, false), FOLD_THREADS, 0, s>>>(W_dev, m, n, eq_dev, rows_per, D.acc, nullptr);
    size_t fin_items = n_pad * 4;
    int fin_grid = (int)((fin_items + 255) / 256);
    if (fin_grid > D.sm_count * 8) fin_grid = D.sm_count * 8;
    fold_finalize_kernel<4><<<fin_grid, 256, 0, s>>>(D.acc, n, n_pad, out_dev);
    e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, err_cap, std::string("kernel launch: ") + cudaGetErrorString(e)); return ZKB_E_CUDA; }
    return ZKB_OK;
}
