// C ABI, part 6: stand-alone field helpers for callers that keep their own protocol order:
// MLE evaluation (rust/zk_ml_prover/src/field/m31_ops.rs:11-26, 155-171) and batch inversion
// (rust/zk_ml_prover/src/proving/lookup.rs:322-368, the hook the reference's GPU seam has at
// lookup.rs:491-542 / gpu/metal_kernels.rs:212-229).  Included by zkb200.cu.
//
// The reference folds the table MSB-first, one variable at a time.  The fold is linear, so the
// result equals sum_i eq(point, i) * evals[i]; with the index split into high and low bits,
// eq(point, i) = eq(point_hi, i >> kl) * eq(point_lo, i & (2^kl - 1)).  Each CTA keeps the low
// eq table (at most 1024 entries) in shared memory, so the pass costs one multiplication per
// element plus one per 1024-element block, and streams the table exactly once.  All values are
// canonical field elements: the sum does not depend on the order it is taken in.

namespace zkb {

constexpr u32 MLE_LO_BITS = 10;
constexpr int MLE_THREADS = 256;

template <class PtT, class ValT> struct MleMul;
template <> struct MleMul<Fp, Fp> { static __device__ __forceinline__ Fp mul(Fp e, Fp v) { return e * v; } };
template <> struct MleMul<Fe, Fp> { static __device__ __forceinline__ Fe mul(Fe e, Fp v) { return e * v; } };
template <> struct MleMul<Fe, Fe> { static __device__ __forceinline__ Fe mul(Fe e, Fe v) { return e * v; } };

// partials[blockIdx.x] = sum over this CTA's blocks; evals holds n_valid elements (the rest of the
// 2^k hypercube is zero).
template <class PtT, class ValT>
__global__ void __launch_bounds__(MLE_THREADS) mle_eval_partial_kernel(const ValT* __restrict__ evals, size_t n_valid,
                                                                      const PtT* __restrict__ point, u32 k, PtT* partials) {
    constexpr int W = Width<PtT>::W;
    __shared__ __align__(16) PtT eq_lo[1u << MLE_LO_BITS];
    __shared__ u32 red[32 * 16];
    const u32 kl = k < MLE_LO_BITS ? k : MLE_LO_BITS, kh = k - kl;
    const size_t lo_n = size_t(1) << kl;
    for (size_t i = threadIdx.x; i < lo_n; i += blockDim.x) st_fe(eq_lo + i, eq_at_index<PtT>(point + kh, kl, i));
    __syncthreads();
    PtT acc = zero_of<PtT>();
    const size_t blocks = (n_valid + lo_n - 1) >> kl;          // blocks that hold at least one valid element
    for (size_t h = blockIdx.x; h < blocks; h += gridDim.x) {
        PtT local = zero_of<PtT>();
        const size_t base = h << kl;
        for (size_t i = threadIdx.x; i < lo_n && base + i < n_valid; i += blockDim.x)
            local = local + MleMul<PtT, ValT>::mul(ld_fe(eq_lo + i), ld_fe(evals + base + i));
        acc = acc + eq_at_index<PtT>(point, kh, h) * local;
    }
    u32 w[W];
    to_words(acc, w);
    block_sum_words<W>(w, red);
    if (threadIdx.x == 0) {
        PtT s;
        from_words(s, w);
        st_fe(partials + blockIdx.x, s);
    }
}
template <class PtT>
__global__ void __launch_bounds__(MLE_THREADS) mle_eval_final_kernel(const PtT* __restrict__ partials, u32 n, PtT* out) {
    constexpr int W = Width<PtT>::W;
    __shared__ u32 red[32 * 16];
    PtT acc = zero_of<PtT>();
    for (u32 i = threadIdx.x; i < n; i += blockDim.x) acc = acc + ld_fe(partials + i);
    u32 w[W];
    to_words(acc, w);
    block_sum_words<W>(w, red);
    if (threadIdx.x == 0) {
        PtT s;
        from_words(s, w);
        st_fe(out, s);
    }
}

// MLE of `evals` (n_valid <= 2^k elements on the device) at `point` (k coordinates on the device)
// -> one element at `out` (device).  Nothing is waited for.
template <class PtT, class ValT>
inline void mle_eval_enqueue(zkb_ctx* c, const ValT* evals, size_t n_valid, const PtT* point, u32 k, PtT* out) {
    const u32 kl = k < MLE_LO_BITS ? k : MLE_LO_BITS;
    size_t blocks = ((n_valid ? n_valid : 1) + (size_t(1) << kl) - 1) >> kl;
    const size_t cap = (size_t)c->sm_count * 8;
    const u32 grid = (u32)(blocks < cap ? blocks : cap);
    PtT* partials = (PtT*)c->scratch((size_t)grid * sizeof(PtT));
    mle_eval_partial_kernel<PtT, ValT><<<grid, MLE_THREADS, 0, c->stream>>>(evals, n_valid, point, k, partials);
    ZKB_LAUNCHED(c);
    mle_eval_final_kernel<PtT><<<1, MLE_THREADS, 0, c->stream>>>(partials, grid, out);
    ZKB_LAUNCHED(c);
}

// out[i] = 1 / vals[i]; every thread inverts a Montgomery batch of four elements with one field
// inversion.  A zero element has no inverse (the reference's `.inverse()` panics): its slot and
// the other slots of its batch receive 0 and the status word is set to ST_DIV_ZERO.
constexpr u32 ST_DIV_ZERO = 9;
template <class T>
__global__ void batch_inverse_kernel(const T* __restrict__ vals, size_t n, T* out, u32* status) {
    const size_t stride = (size_t)gridDim.x * blockDim.x * 4;
    for (size_t base = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; base < n; base += stride) {
        T d[4], pre[4];
        const int cnt = (int)(n - base < 4 ? n - base : 4);
        bool any_zero = false;
        for (int t = 0; t < cnt; t++) { d[t] = ld_fe(vals + base + t); any_zero |= is_zero_el(d[t]); }
        if (any_zero) {
            atomicExch(status, ST_DIV_ZERO);
            for (int t = 0; t < cnt; t++) st_fe(out + base + t, zero_of<T>());
            continue;
        }
        pre[0] = d[0];
        for (int t = 1; t < cnt; t++) pre[t] = pre[t - 1] * d[t];
        T inv = LogupEnc<T>::inv(pre[cnt - 1]);
        for (int t = cnt - 1; t >= 0; t--) {
            st_fe(out + base + t, t ? inv * pre[t - 1] : inv);
            if (t) inv = inv * d[t];
        }
    }
}

}  // namespace zkb

extern "C" {

int32_t zkb_mle_eval_base(zkb_ctx* c, const uint32_t* evals, size_t n, const uint32_t* point, uint32_t k, int32_t on_device,
                          uint32_t* out) {
    if (!c || (!evals && n) || (!point && k) || !out || k > 34 || n > (size_t(1) << k)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const u32* d = on_device ? evals : up_pad(c, evals, n, n);
        u32* dp = up_pad(c, point, k, (size_t)k + 4);
        Fp* res = (Fp*)c->scratch(16);
        mle_eval_enqueue<Fp, Fp>(c, (const Fp*)d, n, (const Fp*)dp, k, res);
        ZKB_CUDA(cudaGetLastError());
        ZKB_CUDA(cudaMemcpyAsync(out, res, 4, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

int32_t zkb_mle_eval_ef(zkb_ctx* c, const uint32_t* evals, size_t n, int32_t evals_ef, const uint32_t* point, uint32_t k,
                        int32_t on_device, uint32_t out[4]) {
    if (!c || (!evals && n) || (!point && k) || !out || k > 34 || n > (size_t(1) << k)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const size_t w = evals_ef ? 4 : 1;
        if (on_device && evals_ef) need_align16(evals, "evals");
        const u32* d = on_device ? evals : up_pad(c, evals, n * w, n * w);
        u32* dp = up_pad(c, point, 4 * (size_t)k, 4 * (size_t)k + 4);
        Fe* res = (Fe*)c->scratch(16);
        if (evals_ef) mle_eval_enqueue<Fe, Fe>(c, (const Fe*)d, n, (const Fe*)dp, k, res);
        else mle_eval_enqueue<Fe, Fp>(c, (const Fp*)d, n, (const Fe*)dp, k, res);
        ZKB_CUDA(cudaGetLastError());
        ZKB_CUDA(cudaMemcpyAsync(out, res, 16, cudaMemcpyDeviceToHost, c->stream));
        ZKB_CUDA(cudaStreamSynchronize(c->stream));
        c->scratch_reset();
    });
}

static int32_t batch_inverse_impl(zkb_ctx* c, const uint32_t* vals, size_t n, int32_t on_device, uint32_t* out, bool ef) {
    if (!c || (!vals && n) || (!out && n)) return ZKB_E_ARG;
    ZKB_TRY(c, {
        c->use();
        const size_t w = ef ? 4 : 1;
        if (on_device && ef) { need_align16(vals, "vals"); need_align16(out, "out"); }
        if (n) {
            clear_status(c);
            const u32* d = on_device ? vals : up_pad(c, vals, n * w, n * w);
            u32* res = on_device ? out : (u32*)c->scratch(n * w * 4);
            const int grid = grid_for(c, (n + 3) / 4);
            if (ef) batch_inverse_kernel<Fe><<<grid, 256, 0, c->stream>>>((const Fe*)d, n, (Fe*)res, c->status);
            else batch_inverse_kernel<Fp><<<grid, 256, 0, c->stream>>>((const Fp*)d, n, (Fp*)res, c->status);
            ZKB_LAUNCHED(c);
            ZKB_CUDA(cudaGetLastError());
            if (!on_device) ZKB_CUDA(cudaMemcpyAsync(out, res, n * w * 4, cudaMemcpyDeviceToHost, c->stream));
            const uint32_t st = c->read_status();
            c->scratch_reset();
            if (st == ST_DIV_ZERO) { c->err = "batch_inverse: zero has no inverse"; return ZKB_E_DIV_ZERO; }
            if (st) return status_to_code(c, st);
        }
    });
}
int32_t zkb_batch_inverse_base(zkb_ctx* c, const uint32_t* vals, size_t n, int32_t on_device, uint32_t* out) {
    return batch_inverse_impl(c, vals, n, on_device, out, false);
}
int32_t zkb_batch_inverse_ef(zkb_ctx* c, const uint32_t* vals, size_t n, int32_t on_device, uint32_t* out) {
    return batch_inverse_impl(c, vals, n, on_device, out, true);
}

}  // extern "C"
