// Exchange of the small per-round values of one sumcheck that is split over several GPUs.
//
// Ownership is by the low bits of the table index: with W GPUs, GPU g holds the elements
// j = j' W + g as a contiguous local table indexed by j'.  Folding is MSB-first (pairs j,
// j + half), so while half >= W both partners of a pair live on the same GPU and a round is
// purely local except for its three or four partial sums.  Those are exchanged here, inside
// the kernel that produced them: one warp of the CTA that finishes the local reduction stores
// its sums into a mailbox in every peer's memory (lane p serves peer p; plain stores through
// peer mappings over NVLink, nothing broadcast by hardware), publishes a sequence number with
// release semantics, waits for the W sequence numbers in its own mailbox (lane s polls sender s),
// adds the W vectors and advances its own copy of the transcript.
// Field addition of canonical values is associative and commutative, so every GPU gets the
// same round message and therefore the same challenge; no broadcast is needed.
//
// Mailbox of one GPU: [2 slots][8 senders][XCH_WORDS words]; word XCH_FLAG of a cell is the
// sequence number, the words before it the payload.  Two slots suffice: nobody can be more
// than one exchange ahead of a peer, because every exchange needs every peer's contribution.
//
// Waits are bounded (by the GPU's nanosecond timer): on expiry the waiter sets a sticky flag
// in its own memory, every later wait on that GPU returns at once, the kernels run to their
// normal end with meaningless sums, and the host reports ZKB_E_TIMEOUT instead of a proof.
#pragma once
#include "m31.cuh"

namespace zkb {

constexpr int XCH_MAX_WORLD = 8;
constexpr int XCH_WORDS = 32;
constexpr int XCH_FLAG = 24;            // payload: up to 24 words
constexpr size_t XCH_BOX_WORDS = 2 * XCH_MAX_WORLD * XCH_WORDS;

struct ScXch {
    u32 world, rank;
    u32 seq;                            // sequence number of the first exchange of this sumcheck
    u32* box[XCH_MAX_WORLD];            // box[p]: mailbox of rank p as seen from this GPU (box[rank] is local)
    u32* sticky;                        // local word: nonzero once a wait has timed out
    unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long xch_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void xch_st_release(u32* p, u32 v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ u32 xch_ld_acquire(const u32* p) {
    u32 v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void xch_st_relaxed(u32* p, u32 v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ u32 xch_ld_relaxed(const u32* p) {
    u32 v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ u32* xch_cell(u32* box, u32 slot, u32 sender) { return box + ((size_t)slot * XCH_MAX_WORLD + sender) * XCH_WORDS; }

// Called by all 32 lanes of ONE warp; `mine` (nw <= XCH_FLAG words) is taken from lane 0.  Lane p
// sends to rank p and lane s waits for sender s, so the stores, the release and the polls of the
// up to eight peers proceed in parallel.  Afterwards lane s (s < world) holds rank s's words in
// got[0..nw).  Returns false (in every lane) after a time-out, now or earlier on this GPU.
template <int NW>
__device__ __forceinline__ bool xch_exchange_warp(const ScXch& x, u32 seq, const u32* mine_lane0, u32* got) {
    const int lane = threadIdx.x & 31;
    const u32 slot = seq & 1;
    u32 mine[NW];
#pragma unroll
    for (int k = 0; k < NW; k++) mine[k] = __shfl_sync(0xffffffffu, mine_lane0[k], 0);
    if (lane < (int)x.world) {
        u32* cell = xch_cell(x.box[lane], slot, x.rank);
#pragma unroll
        for (int k = 0; k < NW; k++) xch_st_relaxed(cell + k, mine[k]);
        xch_st_release(cell + XCH_FLAG, seq);       // orders this lane's payload stores before the flag, system scope
    }
    bool ok = xch_ld_relaxed(x.sticky) == 0;
#pragma unroll
    for (int k = 0; k < NW; k++) got[k] = 0;
    if (lane < (int)x.world) {
        const u32* cell = xch_cell(x.box[x.rank], slot, (u32)lane);
        const unsigned long long t0 = xch_now_ns();
        while (ok && xch_ld_acquire(cell + XCH_FLAG) != seq) {
            if (xch_now_ns() - t0 > x.timeout_ns) { ok = false; xch_st_relaxed(x.sticky, 1u); break; }
            __nanosleep(100);
        }
        if (ok) {
#pragma unroll
            for (int k = 0; k < NW; k++) got[k] = xch_ld_relaxed(cell + k);
        }
    }
    return __all_sync(0xffffffffu, ok);
}
// Sum of the canonical words of all ranks; input and result in lane 0's t[0..NW).
template <int NW>
__device__ __forceinline__ void xch_allreduce_warp(const ScXch& x, u32 seq, u32* t) {
    u32 got[NW];
    const bool ok = xch_exchange_warp<NW>(x, seq, t, got);
#pragma unroll
    for (int k = 0; k < NW; k++) {
        u32 v = got[k];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v = add31(v, __shfl_down_sync(0xffffffffu, v, off));
        if (ok && (threadIdx.x & 31) == 0) t[k] = v;
    }
}

}  // namespace zkb
