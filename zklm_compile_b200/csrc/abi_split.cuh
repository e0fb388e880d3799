// C ABI, part 5: one sumcheck split over several GPUs (one process per GPU).  The per-round
// sums cross NVLink inside the round kernels through peer-mapped mailboxes (exchange.cuh); the
// host only sets the mailboxes up once (CUDA IPC handles, carried between the processes by the
// caller) and enqueues the same launches on every rank.  Included by zkb200.cu.

struct zkb_xch {
    zkb_ctx* ctx = nullptr;
    uint32_t world = 1, rank = 0;
    zkb::u32* local = nullptr;                       // mailbox + sticky word
    zkb::u32* peers[zkb::XCH_MAX_WORLD] = {};        // mapped peer mailboxes (peers[rank] == local)
    bool opened[zkb::XCH_MAX_WORLD] = {};
    bool loopback[zkb::XCH_MAX_WORLD] = {};
    zkb::ScXch* dev = nullptr;                       // descriptor read by the kernels
    uint32_t seq = 1;
    unsigned long long timeout_ns = 4000000000ull;
    bool connected = false;
};

extern "C" {

int32_t zkb_xch_create(zkb_ctx* c, uint32_t world, uint32_t rank, zkb_xch** out) {
    if (!c || !out || world < 1 || world > XCH_MAX_WORLD || (world & (world - 1)) || rank >= world) return ZKB_E_ARG;
    *out = nullptr;
    zkb_xch* x = new (std::nothrow) zkb_xch();
    if (!x) return ZKB_E_CUDA;
    try {
        c->use();
        x->ctx = c; x->world = world; x->rank = rank;
        ZKB_CUDA(cudaMalloc(&x->local, (XCH_BOX_WORDS + 64) * 4));
        ZKB_CUDA(cudaMemset(x->local, 0, (XCH_BOX_WORDS + 64) * 4));
        ZKB_CUDA(cudaMalloc(&x->dev, sizeof(ScXch)));
        x->peers[rank] = x->local;
        x->connected = world == 1;
    } catch (const CudaFail& e) {
        c->err = e.msg;
        if (x->local) cudaFree(x->local);
        if (x->dev) cudaFree(x->dev);
        delete x;
        return ZKB_E_CUDA;
    }
    *out = x;
    return ZKB_OK;
}

int32_t zkb_xch_handle(zkb_xch* x, uint8_t handle[64]) {
    if (!x || !handle) return ZKB_E_ARG;
    zkb_ctx* c = x->ctx;
    ZKB_TRY(c, {
        c->use();
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
        cudaIpcMemHandle_t h;
        ZKB_CUDA(cudaIpcGetMemHandle(&h, x->local));
        memcpy(handle, &h, 64);
    });
}

// handles: world x 64 bytes, entry p from rank p's zkb_xch_handle (entry `rank` is ignored).
int32_t zkb_xch_connect(zkb_xch* x, const uint8_t* handles) {
    if (!x || (!handles && x->world > 1)) return ZKB_E_ARG;
    zkb_ctx* c = x->ctx;
    ZKB_TRY(c, {
        c->use();
        for (uint32_t p = 0; p < x->world; p++) {
            if (p == x->rank || x->opened[p]) continue;
            cudaIpcMemHandle_t h;
            memcpy(&h, handles + 64 * (size_t)p, 64);
            void* ptr = nullptr;
            ZKB_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
            x->peers[p] = (u32*)ptr;
            x->opened[p] = true;
        }
        x->connected = true;
    });
}

// Loop-back wiring for a world of more than one rank inside a single process: every peer mailbox
// is a private buffer on this GPU that nobody writes, so the first exchange runs into the time
// limit.  Exists to exercise the time-out path (status ZKB_E_TIMEOUT, context still usable).
int32_t zkb_xch_connect_loopback(zkb_xch* x) {
    if (!x) return ZKB_E_ARG;
    zkb_ctx* c = x->ctx;
    ZKB_TRY(c, {
        c->use();
        for (uint32_t p = 0; p < x->world; p++) {
            if (p == x->rank || x->peers[p]) continue;
            u32* buf = nullptr;
            ZKB_CUDA(cudaMalloc(&buf, (XCH_BOX_WORDS + 64) * 4));
            ZKB_CUDA(cudaMemset(buf, 0, (XCH_BOX_WORDS + 64) * 4));
            x->peers[p] = buf;
            x->loopback[p] = true;
        }
        x->connected = true;
    });
}

int32_t zkb_xch_set_timeout_ms(zkb_xch* x, uint32_t ms) {
    if (!x || ms == 0) return ZKB_E_ARG;
    x->timeout_ns = (unsigned long long)ms * 1000000ull;
    return ZKB_OK;
}

void zkb_xch_destroy(zkb_xch* x) {
    if (!x) return;
    if (x->ctx) {
        cudaSetDevice(x->ctx->device);
        cudaStreamSynchronize(x->ctx->stream);
    }
    for (uint32_t p = 0; p < x->world; p++)
        if (x->opened[p]) cudaIpcCloseMemHandle(x->peers[p]);
        else if (x->loopback[p]) cudaFree(x->peers[p]);
    if (x->local) cudaFree(x->local);
    if (x->dev) cudaFree(x->dev);
    delete x;
}

// The sumcheck of zkb_sumcheck_prove over tables of 2^num_vars elements of which this rank
// holds the slice {j : j mod world == rank}, stored contiguously (tables[i][j'] = T_i[j' world + rank]).
// Every rank must make the same call (same kind, num_vars, transcript state); every rank gets the
// whole proof and ends with the same transcript state.
int32_t zkb_sumcheck_prove_split(zkb_ctx* c, zkb_xch* x, zkb_transcript* t, int32_t kind, const uint32_t* const* tables,
                                 uint32_t num_vars, int32_t on_device, uint32_t* round_polys, uint32_t* challenges, uint32_t* finals) {
    if (!c || !x || !t || !tables || !round_polys || !challenges || !finals || x->ctx != c) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        if (!x->connected) throw ArgFail{ZKB_E_ARG, "exchange not connected"};
        KindInfo ki = kind_info(kind);
        u32 log_world = 0;
        while ((1u << log_world) < x->world) log_world++;
        if (num_vars < log_world + 1 || num_vars > 34) throw ArgFail{ZKB_E_ARG, "num_vars out of range"};
        const u32 local_vars = num_vars - log_world;
        const size_t n = size_t(1) << local_vars;
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
        ScXch h{};
        h.world = x->world; h.rank = x->rank; h.seq = x->seq;
        for (uint32_t p = 0; p < x->world; p++) h.box[p] = x->peers[p];
        h.sticky = x->local + XCH_BOX_WORDS;
        h.timeout_ns = x->timeout_ns;
        ZKB_CUDA(cudaMemcpyAsync(x->dev, &h, sizeof(h), cudaMemcpyHostToDevice, c->stream));
        c->rec_reset();
        ScOpts o;
        o.xch = x->dev; o.xch_world = x->world;
        ScRec r = sumcheck_enqueue(c, t->dev, kind, dev_tabs, num_vars, o);
        x->seq += local_vars + 1;                 // one exchange per local round, one gather; only once the launches are queued,
                                                  // so that a call that fails before launching leaves the ranks in step
        size_t sticky_off = c->rec_alloc(1);
        ZKB_CUDA(cudaMemcpyAsync(c->rec_dev + sticky_off, h.sticky, 4, cudaMemcpyDeviceToDevice, c->stream));
        c->rec_fetch();
        const u32* rec = c->rec_host;
        c->scratch_reset();
        if (rec[sticky_off]) { c->err = "split sumcheck: a peer did not answer in time"; return ZKB_E_TIMEOUT; }
        size_t k = 0;
        for (u32 round = 0; round < num_vars; round++)
            for (u32 e = 0; e < ki.nabs; e++)
                if (ki.mask & (1u << e))
                    for (int wd = 0; wd < ki.w; wd++) round_polys[k++] = rec[r.polys + ((size_t)round * ki.nabs + e) * ki.w + wd];
        memcpy(challenges, rec + r.chal, (size_t)num_vars * ki.w * 4);
        if (ki.nt == 1) {
            memset(finals, 0, ki.w * 4);
            finals[0] = 1;
            memcpy(finals + ki.w, rec + r.fin, ki.w * 4);
        } else {
            memcpy(finals, rec + r.fin, (size_t)ki.nt * ki.w * 4);
        }
    });
}

}  // extern "C"
