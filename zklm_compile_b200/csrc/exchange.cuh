// Exchange of the small per-round values of one sumcheck that is split over several GPUs.
//
// Ownership is by the low bits of the table index: with W GPUs, GPU g holds the elements
// j = j' W + g as a contiguous local table indexed by j'.  Folding is MSB-first (pairs j,
// j + half), so while half >= W both partners of a pair live on the same GPU and a round is
// purely local except for its three or four partial sums.  Those are exchanged here, inside
// the kernel that produced them: the CTA that finishes the local reduction stores its sums
// into a mailbox in every peer's memory (plain stores through peer mappings over NVLink, no
// multicast), publishes a sequence number with release semantics, waits for the W sequence
// numbers in its own mailbox, adds the W vectors and advances its own copy of the transcript.
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

// Called by ONE thread.  Sends `mine` (nw <= XCH_FLAG words) to every rank under sequence
// number `seq` and collects everybody's words into all[s * nw + k].  Returns false after a
// timeout (now or earlier on this GPU); `all` is then unspecified.
__device__ inline bool xch_allgather(const ScXch& x, u32 seq, const u32* mine, int nw, u32* all) {
    const u32 slot = seq & 1;
    for (u32 p = 0; p < x.world; p++) {
        u32* cell = xch_cell(x.box[p], slot, x.rank);
        for (int k = 0; k < nw; k++) xch_st_relaxed(cell + k, mine[k]);
    }
    // release: the payload stores above are ordered before each flag store at system scope
    for (u32 p = 0; p < x.world; p++) xch_st_release(xch_cell(x.box[p], slot, x.rank) + XCH_FLAG, seq);
    bool ok = xch_ld_relaxed(x.sticky) == 0;
    const unsigned long long t0 = xch_now_ns();
    for (u32 s = 0; s < x.world && ok; s++) {
        const u32* cell = xch_cell(x.box[x.rank], slot, s);
        while (xch_ld_acquire(cell + XCH_FLAG) != seq) {
            if (xch_now_ns() - t0 > x.timeout_ns) { ok = false; xch_st_relaxed(x.sticky, 1u); break; }
            __nanosleep(100);
        }
        if (ok) for (int k = 0; k < nw; k++) all[s * nw + k] = xch_ld_relaxed(cell + k);
    }
    return ok;
}
// Sum of the canonical words of all ranks, in place.
template <int NW>
__device__ inline void xch_allreduce(const ScXch& x, u32 seq, u32* t) {
    u32 all[XCH_MAX_WORLD * NW];
    if (!xch_allgather(x, seq, t, NW, all)) return;
#pragma unroll
    for (int k = 0; k < NW; k++) {
        u32 a = 0;
        for (u32 s = 0; s < x.world; s++) a = add31(a, all[s * NW + k]);
        t[k] = a;
    }
}

}  // namespace zkb
