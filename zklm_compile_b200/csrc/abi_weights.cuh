// C ABI, part 8: weights brought in the reference's own wire format and kept resident.
//
// The reference's server mode reads a preload block once (rust/zk_ml_prover/src/server.rs:33-94):
//   [count u32] then per matrix [name_len u32][name bytes, UTF-8][m u32][n u32][m * n u32 LE, canonical field elements]
// converts every matrix to field elements, commits it with commit_weights_fast and keeps it in a map by
// name for all later requests.  Here the block is taken as it arrives: each matrix is copied to device
// memory through two pinned staging buffers (the copy of one piece to the GPU overlaps the host copy of
// the next), its commitment is computed on the GPU from the resident copy, and the map hands out device
// pointers.  The caps are the reference's (server.rs:19-22).  Included by zkb200.cu.

struct zkb_weightset {
    struct Entry { std::string name; zkb::u32* w = nullptr; size_t m = 0, n = 0; uint8_t root[32] = {}; };
    zkb_ctx* ctx = nullptr;
    std::vector<Entry> entries;                  // in arrival order; a later entry of the same name replaces the earlier one in `by_name`
    std::map<std::string, size_t> by_name;
    size_t bytes = 0;
};

namespace {

constexpr uint32_t PRELOAD_MAX_WEIGHTS = 1u << 16;
constexpr size_t PRELOAD_MAX_DIM = size_t(1) << 24, PRELOAD_MAX_NAME_LEN = size_t(1) << 12, PRELOAD_MAX_ELEMENT_COUNT = size_t(1) << 30;
constexpr size_t PRELOAD_STAGE_BYTES = size_t(64) << 20;

bool utf8_valid(const uint8_t* s, size_t n) {
    size_t i = 0;
    while (i < n) {
        const uint8_t c = s[i];
        size_t extra;
        uint32_t cp;
        if (c < 0x80) { i++; continue; }
        else if ((c & 0xE0) == 0xC0) { extra = 1; cp = c & 0x1F; if (cp < 2) return false; }
        else if ((c & 0xF0) == 0xE0) { extra = 2; cp = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { extra = 3; cp = c & 0x07; if (cp > 4) return false; }
        else return false;
        for (size_t k = 1; k <= extra; k++) {
            if (i + k >= n || (s[i + k] & 0xC0) != 0x80) return false;
            cp = (cp << 6) | (s[i + k] & 0x3F);
        }
        if (extra == 2 && (cp < 0x800 || (cp >= 0xD800 && cp <= 0xDFFF))) return false;
        if (extra == 3 && (cp < 0x10000 || cp > 0x10FFFF)) return false;
        i += extra + 1;
    }
    return true;
}

struct PreloadReader {
    const uint8_t* p; size_t n, at = 0;
    uint32_t u32v() {
        if (at + 4 > n) throw ArgFail{ZKB_E_ARG, "preload block: unexpected end"};
        uint32_t v = (uint32_t)p[at] | ((uint32_t)p[at + 1] << 8) | ((uint32_t)p[at + 2] << 16) | ((uint32_t)p[at + 3] << 24);
        at += 4;
        return v;
    }
};

}  // namespace

extern "C" {

void zkb_weightset_destroy(zkb_weightset* ws) {
    if (!ws) return;
    if (ws->ctx) { cudaSetDevice(ws->ctx->device); cudaStreamSynchronize(ws->ctx->stream); }
    for (auto& e : ws->entries) if (e.w) cudaFree(e.w);
    delete ws;
}

int32_t zkb_weightset_preload(zkb_ctx* c, const uint8_t* block, size_t len, zkb_weightset** out, size_t* consumed) {
    if (!c || !block || !out) return ZKB_E_ARG;
    *out = nullptr;
    zkb_weightset* ws = new (std::nothrow) zkb_weightset();
    if (!ws) return ZKB_E_CUDA;
    ws->ctx = c;
    uint8_t* stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    auto cleanup = [&]() {
        for (int i = 0; i < 2; i++) { if (stage[i]) cudaFreeHost(stage[i]); if (done[i]) cudaEventDestroy(done[i]); }
    };
    int32_t rc = ZKB_OK;
    try {
        c->use();
        for (int i = 0; i < 2; i++) {
            ZKB_CUDA(cudaHostAlloc(&stage[i], PRELOAD_STAGE_BYTES, cudaHostAllocDefault));
            ZKB_CUDA(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
        PreloadReader rd{block, len};
        const uint32_t count = rd.u32v();
        if (count > PRELOAD_MAX_WEIGHTS) throw ArgFail{ZKB_E_ARG, "preload block: num_weights exceeds the cap of 65536"};
        int slot = 0;
        for (uint32_t i = 0; i < count; i++) {
            const size_t name_len = rd.u32v();
            if (name_len > PRELOAD_MAX_NAME_LEN) throw ArgFail{ZKB_E_ARG, "preload block: name_len exceeds the cap of 4096"};
            if (rd.at + name_len > len) throw ArgFail{ZKB_E_ARG, "preload block: unexpected end"};
            if (!utf8_valid(block + rd.at, name_len)) throw ArgFail{ZKB_E_ARG, "preload block: name not valid UTF-8"};
            zkb_weightset::Entry e;
            e.name.assign(reinterpret_cast<const char*>(block + rd.at), name_len);
            rd.at += name_len;
            e.m = rd.u32v(); e.n = rd.u32v();
            if (e.m > PRELOAD_MAX_DIM || e.n > PRELOAD_MAX_DIM) throw ArgFail{ZKB_E_ARG, "preload block: dimension exceeds the cap of 2^24"};
            const size_t total = e.m * e.n;                      // both below 2^24: no overflow
            if (total > PRELOAD_MAX_ELEMENT_COUNT) throw ArgFail{ZKB_E_ARG, "preload block: element count exceeds the cap of 2^30"};
            if (total > (len - rd.at) / 4) throw ArgFail{ZKB_E_ARG, "preload block: unexpected end"};
            ZKB_CUDA(cudaMalloc(&e.w, (total ? total : 1) * 4 + 16));
            ws->entries.push_back(e);                            // from here on destroy() frees it
            const uint8_t* src = block + rd.at;
            for (size_t off = 0; off < total * 4; off += PRELOAD_STAGE_BYTES) {
                const size_t piece = total * 4 - off < PRELOAD_STAGE_BYTES ? total * 4 - off : PRELOAD_STAGE_BYTES;
                ZKB_CUDA(cudaEventSynchronize(done[slot]));      // the copy that last used this staging buffer has finished
                memcpy(stage[slot], src + off, piece);
                ZKB_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(e.w) + off, stage[slot], piece, cudaMemcpyHostToDevice, c->stream));
                ZKB_CUDA(cudaEventRecord(done[slot], c->stream));
                slot ^= 1;
            }
            rd.at += total * 4;
            // commit_weights_fast(w) from the resident copy
            u32* root = (u32*)c->scratch(32);
            commit_large(c, b3_prefix("weights", 7), e.w, total, root);
            ZKB_CUDA(cudaMemcpyAsync(ws->entries.back().root, root, 32, cudaMemcpyDeviceToHost, c->stream));
            ws->bytes += total * 4;
            ws->by_name[e.name] = ws->entries.size() - 1;
        }
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
        if (consumed) *consumed = rd.at;
    } catch (const CudaFail& e) { c->err = e.msg; rc = ZKB_E_CUDA; }
    catch (const ArgFail& e) { c->err = e.msg; rc = e.code; }
    catch (const std::bad_alloc&) { c->err = "host allocation failed"; rc = ZKB_E_CUDA; }
    if (rc != ZKB_OK) {
        cudaStreamSynchronize(c->stream);
        cleanup();
        zkb_weightset_destroy(ws);
        return rc;
    }
    cleanup();
    *out = ws;
    return ZKB_OK;
}

uint32_t zkb_weightset_count(const zkb_weightset* ws) { return ws ? (uint32_t)ws->by_name.size() : 0; }
uint64_t zkb_weightset_bytes(const zkb_weightset* ws) { return ws ? ws->bytes : 0; }

int32_t zkb_weightset_get(const zkb_weightset* ws, const char* name, const uint32_t** w_dev, size_t* m, size_t* n, uint8_t root[32]) {
    if (!ws || !name) return ZKB_E_ARG;
    auto it = ws->by_name.find(name);
    if (it == ws->by_name.end()) { ws->ctx->err = std::string("no preloaded weight named '") + name + "'"; return ZKB_E_ARG; }
    const zkb_weightset::Entry& e = ws->entries[it->second];
    if (w_dev) *w_dev = e.w;
    if (m) *m = e.m;
    if (n) *n = e.n;
    if (root) memcpy(root, e.root, 32);
    return ZKB_OK;
}

}  // extern "C"
