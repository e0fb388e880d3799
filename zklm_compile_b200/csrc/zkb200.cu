// C ABI of the backend (see include/zkb200.h) and the host-side launch logic.
#include "context.cuh"
#include <cstring>
#include <new>

using namespace zkb;

// =============================================================================================
// transcript kernels
// =============================================================================================
struct ByteChunk { unsigned char b[256]; };

__global__ void tr_init_kernel(TrState* st) {
    u32 h[8];
    tr_iv(h);
    for (int i = 0; i < 8; i++) st->h[i] = h[i];
    st->buflen = 0; st->_pad = 0; st->total = 0;
    for (int i = 0; i < 64; i++) st->buf[i] = 0;
}
__global__ void tr_absorb_bytes_kernel(TrState* st, ByteChunk c, u32 n) {
    __shared__ __align__(16) unsigned char trbuf[64];
    Tr tr;
    tr_load(tr, st, trbuf);
    tr_absorb_bytes(tr, c.b, n);
    tr_store(tr, st);
}
// One warp: lanes stage 512-word tiles into shared memory, lane 0 runs the hash chain.
__global__ void tr_absorb_words_kernel(TrState* st, const u32* __restrict__ v, size_t n) {
    __shared__ __align__(16) unsigned char trbuf[64];
    __shared__ u32 tile[512];
    Tr tr;
    if (threadIdx.x == 0) tr_load(tr, st, trbuf);
    for (size_t base = 0; base < n; base += 512) {
        size_t m = n - base < 512 ? n - base : 512;
        for (size_t i = threadIdx.x; i < m; i += blockDim.x) tile[i] = v[base + i];
        __syncwarp();
        if (threadIdx.x == 0)
            for (size_t i = 0; i < m; i++) tr_absorb_u32(tr, tile[i]);
        __syncwarp();
    }
    if (threadIdx.x == 0) tr_store(tr, st);
}
__global__ void tr_squeeze_kernel(TrState* st, u32* out, u32 count) {
    __shared__ __align__(16) unsigned char trbuf[64];
    Tr tr;
    tr_load(tr, st, trbuf);
    for (u32 i = 0; i < count; i++) out[i] = tr_squeeze(tr);
    tr_store(tr, st);
}

// =============================================================================================
// sumcheck launch logic
// =============================================================================================
namespace {

constexpr size_t MULTI_MIN_HALF = 2048;   // below this many pairs the single-CTA tail takes over

template <int KIND, class SrcT, class ChalT>
void run_sumcheck(zkb_ctx* c, ScTables tb, u32 num_vars, ScIO io) {
    size_t size = size_t(1) << num_vars;
    bool pending = false, in_src = true;
    u32 round = 0;
    const int max_grid = c->sm_count * 8 < SC_MAX_GRID ? c->sm_count * 8 : SC_MAX_GRID;
    c->prof_used = 0;
    c->prof_mark();
    while (round < num_vars) {
        size_t half = pending ? size / 4 : size / 2;
        if (half < MULTI_MIN_HALF) break;
        size_t want = (half + 255) / 256;
        int grid = (int)(want < (size_t)max_grid ? want : (size_t)max_grid);
        if (!pending) {
            sc_round_kernel<KIND, SrcT, ChalT, false><<<grid, 256, 0, c->stream>>>(tb, half, round, io);
        } else if (in_src) {
            sc_round_kernel<KIND, SrcT, ChalT, true><<<grid, 256, 0, c->stream>>>(tb, half, round, io);
            for (int t = 0; t < 3; t++) tb.src[t] = tb.dst[t];
            in_src = false;
            size /= 2;
        } else {
            sc_round_kernel<KIND, ChalT, ChalT, true><<<grid, 256, 0, c->stream>>>(tb, half, round, io);
            size /= 2;
        }
        c->launches++;
        c->prof_mark();
        pending = true;
        round++;
    }
    if (in_src)
        sc_tail_kernel<KIND, SrcT, ChalT><<<1, SC_TAIL_THREADS, 0, c->stream>>>(tb, size, round, num_vars, pending ? 1 : 0, io);
    else
        sc_tail_kernel<KIND, ChalT, ChalT><<<1, SC_TAIL_THREADS, 0, c->stream>>>(tb, size, round, num_vars, 1, io);
    c->launches++;
    c->prof_mark();
    ZKB_CUDA(cudaGetLastError());
}

__global__ void widen_kernel(const u32* __restrict__ in, Fe* out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        st_fe(out + i, Fe{in[i], 0, 0, 0});
}

struct KindInfo { int nt; int in_w[3]; int w; u32 mask; u32 nstored; };
KindInfo kind_info(int kind) {
    switch (kind) {
        case ZKB_SC_PRODUCT:              return {2, {1, 1, 0}, 1, 0b0111, 3};
        case ZKB_SC_TRIPLE:               return {3, {1, 1, 1}, 1, 0b1111, 4};
        case ZKB_SC_PRODUCT_ONES:         return {1, {1, 0, 0}, 1, 0b0101, 2};
        case ZKB_SC_PRODUCT_EF:           return {2, {1, 1, 0}, 4, 0b0101, 2};
        case ZKB_SC_PRODUCT_EF_FULL:      return {2, {4, 4, 0}, 4, 0b0111, 3};
        case ZKB_SC_PRODUCT_EF_MIXED:     return {2, {4, 1, 0}, 4, 0b0111, 3};
        case ZKB_SC_TRIPLE_EF_FULL:       return {3, {4, 4, 4}, 4, 0b1101, 3};
        case ZKB_SC_PRODUCT_ONES_EF_FULL: return {1, {4, 0, 0}, 4, 0b0101, 2};
    }
    throw ArgFail{ZKB_E_ARG, "unknown sumcheck kind"};
}

}  // namespace

namespace zkb {

// Enqueue one sumcheck on device tables; outputs go to device memory at out_polys / out_chal /
// out_fin.  No synchronisation.  `tables_dev` are left untouched; working copies come from the
// context's scratch arena (the caller rewinds it).
void sumcheck_enqueue(zkb_ctx* c, TrState* tr, int kind, const u32* const* tables_dev, u32 num_vars,
                      u32* out_polys, u32* out_chal, u32* out_fin) {
    KindInfo ki = kind_info(kind);
    if (num_vars < 1 || num_vars > 40) throw ArgFail{ZKB_E_ARG, "num_vars out of range"};
    const size_t n = size_t(1) << num_vars;
    ScTables tb{};
    const size_t dst_elems = n / 2 > 2 ? n / 2 : 2;
    for (int t = 0; t < ki.nt; t++) {
        tb.src[t] = tables_dev[t];
        tb.dst[t] = c->scratch(dst_elems * 4 * ki.w);
    }
    if (kind == ZKB_SC_PRODUCT_EF_MIXED) {      // widen g once; then it is PRODUCT_EF_FULL with the same message layout
        Fe* g = (Fe*)c->scratch(n * 16);
        int grid = (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
        widen_kernel<<<grid, 256, 0, c->stream>>>(tables_dev[1], g, n);
        c->launches++;
        tb.src[1] = g;
    }
    ScIO io{};
    io.tr = tr; io.partials = c->partials; io.counter = c->counter;
    io.polys = out_polys; io.chal = out_chal; io.fin = out_fin;
    io.store_mask = ki.mask; io.nstored = ki.nstored;
    switch (kind) {
        case ZKB_SC_PRODUCT:              run_sumcheck<SC_PRODUCT, Fp, Fp>(c, tb, num_vars, io); break;
        case ZKB_SC_TRIPLE:               run_sumcheck<SC_TRIPLE, Fp, Fp>(c, tb, num_vars, io); break;
        case ZKB_SC_PRODUCT_ONES:         run_sumcheck<SC_ONES, Fp, Fp>(c, tb, num_vars, io); break;
        case ZKB_SC_PRODUCT_EF:           run_sumcheck<SC_PRODUCT, Fp, Fe>(c, tb, num_vars, io); break;
        case ZKB_SC_PRODUCT_EF_FULL:
        case ZKB_SC_PRODUCT_EF_MIXED:     run_sumcheck<SC_PRODUCT, Fe, Fe>(c, tb, num_vars, io); break;
        case ZKB_SC_TRIPLE_EF_FULL:       run_sumcheck<SC_TRIPLE, Fe, Fe>(c, tb, num_vars, io); break;
        case ZKB_SC_PRODUCT_ONES_EF_FULL: run_sumcheck<SC_ONES, Fe, Fe>(c, tb, num_vars, io); break;
    }
}

}  // namespace zkb

// =============================================================================================
// C ABI
// =============================================================================================
#define ZKB_TRY(ctxptr, ...)                                                         \
    try { __VA_ARGS__; return ZKB_OK; }                                                     \
    catch (const CudaFail& e) { if (ctxptr) (ctxptr)->err = e.msg; return ZKB_E_CUDA; } \
    catch (const ArgFail& e) { if (ctxptr) (ctxptr)->err = e.msg; return e.code; }   \
    catch (const std::bad_alloc&) { if (ctxptr) (ctxptr)->err = "host allocation failed"; return ZKB_E_CUDA; }

extern "C" {

int32_t zkb_ctx_create(int32_t device, zkb_ctx** out) {
    if (!out) return ZKB_E_ARG;
    *out = nullptr;
    zkb_ctx* c = new (std::nothrow) zkb_ctx();
    if (!c) return ZKB_E_CUDA;
    c->device = device;
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
    if (c->partials) cudaFree(c->partials);
    if (c->counter) cudaFree(c->counter);
    if (c->status) cudaFree(c->status);
    if (c->t0) cudaEventDestroy(c->t0);
    if (c->t1) cudaEventDestroy(c->t1);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

const char* zkb_last_error(const zkb_ctx* c) { return c ? c->err.c_str() : "null context"; }
uint64_t zkb_launch_count(const zkb_ctx* c) { return c ? c->launches : 0; }

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
            if (on_device) dev_tabs[i] = tables[i];
            else {
                u32* d = (u32*)c->scratch(n * 4 * ki.in_w[i]);
                ZKB_CUDA(cudaMemcpyAsync(d, tables[i], n * 4 * ki.in_w[i], cudaMemcpyHostToDevice, c->stream));
                dev_tabs[i] = d;
            }
        }
        const size_t npoly = (size_t)num_vars * ki.nstored * ki.w, nchal = (size_t)num_vars * ki.w;
        const int nfin = ki.nt < 2 ? 2 : ki.nt;
        u32* out = (u32*)c->scratch((npoly + nchal + 3 * 4) * 4);
        u32* d_fin = out + npoly + nchal;
        // For ONES the first final is the constant 1 (sumcheck.rs:901, 1434); the kernel writes g(s) to slot 0.
        sumcheck_enqueue(c, t->dev, kind, dev_tabs, num_vars, out, out + npoly, d_fin);
        ZKB_CUDA(cudaMemcpyAsync(round_polys, out, npoly * 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaMemcpyAsync(challenges, out + npoly, nchal * 4, cudaMemcpyDeviceToHost, c->stream));
        if (ki.nt == 1) {
            memset(finals, 0, ki.w * 4);
            finals[0] = 1;
            ZKB_CUDA(cudaMemcpyAsync(finals + ki.w, d_fin, ki.w * 4, cudaMemcpyDeviceToHost, c->stream));
        } else {
            ZKB_CUDA(cudaMemcpyAsync(finals, d_fin, (size_t)nfin * ki.w * 4, cudaMemcpyDeviceToHost, c->stream));
        }
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

}  // extern "C"
