// Host-side context: one CUDA stream, a growable scratch arena, the per-stream reduction
// scratch of the sumcheck kernels, and error bookkeeping for the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>
#include "../../include/zkb200.h"
#include "sumcheck.cuh"

namespace zkb {

struct CudaFail { std::string msg; };

#define ZKB_CUDA(expr)                                                                          \
    do {                                                                                        \
        cudaError_t _e = (expr);                                                                \
        if (_e != cudaSuccess)                                                                  \
            throw ::zkb::CudaFail{std::string(#expr) + ": " + cudaGetErrorString(_e)};          \
    } while (0)

struct ArgFail { int32_t code; std::string msg; };

// Launch with programmatic stream serialisation: the kernel may begin before the previous kernel of
// the stream has finished (see pdl_wait in m31.cuh).
template <class... KArgs, class... Args>
inline void launch_pdl_smem(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    ZKB_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}
template <class... KArgs, class... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    ZKB_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}

}  // namespace zkb

struct zkb_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    zkb::u32* partials = nullptr;
    unsigned int* counter = nullptr;
    zkb::u32* status = nullptr;          // device status word(s) written by kernels
    std::string err;
    uint64_t launches = 0;

    // scratch arena: bump allocation, rewound by the caller that opened the frame
    struct Chunk { char* base; size_t cap; size_t used; };
    std::vector<Chunk> chunks;

    // record buffer: every value a proof needs, written by kernels, fetched in one copy
    zkb::u32* rec_dev = nullptr;
    zkb::u32* rec_host = nullptr;        // pinned mirror
    size_t rec_cap = 0, rec_used = 0;
    // Slots are 16-byte aligned: challenge slots are read back by kernels as EF elements (uint4 loads).
    size_t rec_alloc(size_t nwords) {
        nwords = (nwords + 3) & ~size_t(3);
        if (rec_used + nwords > rec_cap) throw zkb::ArgFail{ZKB_E_TOO_LARGE, "proof record buffer exhausted"};
        size_t off = rec_used;
        rec_used += nwords;
        return off;
    }
    void rec_reset() { rec_used = 0; }
    // Copy the used part of the record to the host and wait for it (the one sync of a proof).
    void rec_fetch() {
        if (rec_used) ZKB_CUDA(cudaMemcpyAsync(rec_host, rec_dev, rec_used * 4, cudaMemcpyDeviceToHost, stream));
        ZKB_CUDA(cudaStreamSynchronize(stream));
    }
    // Status word written by kernels (0 = ok); reading it synchronises.
    uint32_t read_status() {
        uint32_t v = 0;
        ZKB_CUDA(cudaMemcpyAsync(&v, status, 4, cudaMemcpyDeviceToHost, stream));
        ZKB_CUDA(cudaStreamSynchronize(stream));
        return v;
    }

    // stopwatch + per-launch profile
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    bool profile = false;
    std::vector<cudaEvent_t> prof_events;
    size_t prof_used = 0;

    // Launch trace: when on, every launch site records an event behind its kernel (as an event-record
    // node when the stream is being captured, so replays of the graph refresh the time stamps).
    struct TraceEntry { const char* file; int line; cudaEvent_t ev; };
    bool trace = false;
    std::vector<TraceEntry> trace_log;
    void launched(const char* file, int line) {
        launches++;
        if (!trace) return;
        cudaEvent_t e = ev_get();
        ZKB_CUDA(cudaEventRecordWithFlags(e, stream, capturing ? cudaEventRecordExternal : cudaEventRecordDefault));
        trace_log.push_back(TraceEntry{file, line, e});
    }
    void trace_clear() {
        for (auto& t : trace_log) ev_pool.push_back(t.ev);
        trace_log.clear();
    }

    // tagged event pairs around the bandwidth-bound kernels (only when profiling is on)
    struct Range { int tag; double bytes; cudaEvent_t a, b; };
    std::vector<Range> ranges;
    std::vector<cudaEvent_t> ev_pool;
    cudaEvent_t ev_get() {
        if (!ev_pool.empty()) { cudaEvent_t e = ev_pool.back(); ev_pool.pop_back(); return e; }
        cudaEvent_t e;
        ZKB_CUDA(cudaEventCreate(&e));
        return e;
    }
    int range_begin(int tag, double bytes) {
        if (!profile) return -1;
        Range r{tag, bytes, ev_get(), ev_get()};
        ZKB_CUDA(cudaEventRecord(r.a, stream));
        ranges.push_back(r);
        return (int)ranges.size() - 1;
    }
    void range_end(int id) {
        if (id >= 0) ZKB_CUDA(cudaEventRecord(ranges[id].b, stream));
    }

    void use() { ZKB_CUDA(cudaSetDevice(device)); }

    // "Polite" launch shapes, for contexts that run next to many others on the same GPU (one per
    // layer of a model): every kernel leaves half of each SM's registers and thread slots free -
    // single-CTA kernels use 512 threads, wide kernels a few CTAs per SM - so that another
    // context's latency-critical single-CTA kernel (a transcript step, a sumcheck tail) never
    // has to wait for a wide kernel to drain before it finds an SM.
    bool polite = false;
    // Tuning options (zkb_ctx_set_option): 0 = the built-in choice.
    int opt_single_threads = 0, opt_pipe_threads = 0, opt_fold2_vec = 0;
    bool opt_plain_tail = false, opt_no_fused2 = false, opt_bf_in_order = false;
    int opt_att_threads = 0;             // threads per row CTA of the attention kernels (0: chosen from the shape)
    int opt_shared_sm = 0;               // 0: hash-chain kernels reserve 200 KB of shared memory, 1: none, 16 .. 200: that many KB
    bool opt_mv_ring = false;            // forward matvec: the bulk-copy ring kernel instead of the register-staged one
    int opt_mv_prefetch = 2;             // rows per CTA whose lines a forward matvec prefetches into L2 before it waits for its input (0 .. 8 measured: 2 is best)
    // Second stream for work that does not depend on the transcript (the fold / tree chain of a Basefold
    // opening), joined to `stream` through events; created on first use.
    // Page-locked staging for results that are larger than the record buffer; grows, freed with the context.
    void* stage = nullptr;
    size_t stage_cap = 0;
    void* stage_host(size_t bytes) {
        if (bytes > stage_cap) {
            if (stage) { ZKB_CUDA(cudaStreamSynchronize(stream)); cudaFreeHost(stage); stage = nullptr; stage_cap = 0; }
            size_t cap = bytes + (bytes >> 2);
            ZKB_CUDA(cudaHostAlloc(&stage, cap, cudaHostAllocDefault));
            stage_cap = cap;
        }
        return stage;
    }
    cudaStream_t side = nullptr;
    std::vector<cudaEvent_t> side_ev;
    cudaStream_t side_stream() {
        if (!side) ZKB_CUDA(cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking));
        return side;
    }
    cudaEvent_t side_event(size_t i) {
        while (side_ev.size() <= i) {
            cudaEvent_t e;
            ZKB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            side_ev.push_back(e);
        }
        return side_ev[i];
    }
    int single_cta_threads() const { return opt_single_threads ? opt_single_threads : (polite ? 512 : 1024); }
    int pipe_threads(int full) const { return opt_pipe_threads ? opt_pipe_threads : (polite ? full / 2 : full); }
    int wide_ctas_per_sm(int greedy, int shared) const { return polite ? shared : greedy; }

    // While a stream capture is open nothing may be allocated; arena_epoch changes whenever the
    // arena's memory does, which invalidates captured graphs that hold addresses inside it.
    bool capturing = false;
    uint64_t arena_epoch = 0;

    size_t cur_chunk = 0;               // chunks before it are full (or were skipped), chunks after it are empty
    void* scratch(size_t bytes) {
        bytes = (bytes + 255) & ~size_t(255);
        for (size_t i = cur_chunk; i < chunks.size(); i++) {
            Chunk& c = chunks[i];
            if (c.used + bytes <= c.cap) { void* p = c.base + c.used; c.used += bytes; cur_chunk = i; return p; }
        }
        if (capturing) throw zkb::ArgFail{ZKB_E_TOO_LARGE, "scratch arena would have to grow during a stream capture"};
        arena_epoch++;
        size_t cap = bytes;
        if (cap < (size_t(64) << 20)) cap = size_t(64) << 20;
        char* p = nullptr;
        ZKB_CUDA(cudaMalloc(&p, cap));
        chunks.push_back(Chunk{p, cap, bytes});
        cur_chunk = chunks.size() - 1;
        return p;
    }
    // A section whose scratch is dead once its kernels have been enqueued (work on one stream runs in
    // order, so whatever is enqueued later may reuse the memory): mark, allocate, release.
    struct ScratchMark { size_t chunk, used; };
    ScratchMark scratch_mark() const { return ScratchMark{cur_chunk, chunks.empty() ? 0 : chunks[cur_chunk].used}; }
    void scratch_release(ScratchMark m) {
        if (chunks.empty()) return;
        for (size_t i = m.chunk + 1; i < chunks.size(); i++) chunks[i].used = 0;
        chunks[m.chunk].used = m.used;
        cur_chunk = m.chunk;
    }
    // Rewind everything; if the arena fragmented into several chunks, replace them by one.
    void scratch_reset() {
        cur_chunk = 0;
        if (chunks.size() > 1) {
            arena_epoch++;
            ZKB_CUDA(cudaStreamSynchronize(stream));
            size_t total = 0;
            for (auto& c : chunks) { total += c.cap; cudaFree(c.base); }
            chunks.clear();
            char* p = nullptr;
            ZKB_CUDA(cudaMalloc(&p, total));
            chunks.push_back(Chunk{p, total, 0});
        } else if (!chunks.empty()) {
            chunks[0].used = 0;
        }
    }
    // Give the arena's memory back to the device (the next proof allocates it again).
    void scratch_trim() {
        ZKB_CUDA(cudaStreamSynchronize(stream));
        for (auto& c : chunks) cudaFree(c.base);
        chunks.clear();
        cur_chunk = 0;
        arena_epoch++;
    }
    size_t scratch_capacity() const { size_t t = 0; for (auto& c : chunks) t += c.cap; return t; }
    void prof_mark() {
        if (!profile) return;
        if (prof_used == prof_events.size()) {
            cudaEvent_t e;
            ZKB_CUDA(cudaEventCreate(&e));
            prof_events.push_back(e);
        }
        ZKB_CUDA(cudaEventRecord(prof_events[prof_used++], stream));
    }
};

struct zkb_transcript {
    zkb_ctx* ctx;
    zkb::TrState* dev;
};
