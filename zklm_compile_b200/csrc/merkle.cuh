// Merkle trees with 16-byte digests over vectors of field elements
// (rust/zk_ml_prover/src/proving/pcs.rs:57-196).
//
//   leaf      u32 value, little-endian, zero-padded to 16 bytes, not hashed      pcs.rs:71-75
//   node      blake3(L || R) truncated to 16 bytes (what the reference computes   pcs.rs:125-134
//             on every target except aarch64), or the AES-based Matyas-Meyer-
//             Oseas compression it uses on aarch64                               pcs.rs:92-121
//
// A tree of height h over 2^h leaves stores layers 1..h (layer k has 2^(h-k) nodes) back to
// back: layer k starts at node offset 2^h - 2^(h-k+1); the root is node 2^h - 2.  One launch
// of mk_tile_kernel builds up to MK_TILE_LOG levels: each CTA owns MK_TILE consecutive inputs,
// keeps the running level in shared memory and writes every level it produces.  A 32-byte node
// input is a single blake3 block, so one node costs one compression; the kernel is bound by
// integer issue, not by bandwidth (16 bytes read and 8 written per compression on average).
#pragma once
#include "blake3.cuh"

namespace zkb {

enum NodeHash : int { NODE_BLAKE3 = 0, NODE_AES_MMO = 1 };

// ---- blake3 node: one block of 32 bytes, flags CHUNK_START | CHUNK_END | ROOT -------------------
// Message words 8..15 are zero, so with the schedule resolved at compile time half of the
// message additions disappear.
__device__ __forceinline__ uint4 b3_node(uint4 l, uint4 r) {
    u32 w[16] = {l.x, l.y, l.z, l.w, r.x, r.y, r.z, r.w, 0, 0, 0, 0, 0, 0, 0, 0};
    u32 s0 = 0x6a09e667u, s1 = 0xbb67ae85u, s2 = 0x3c6ef372u, s3 = 0xa54ff53au;
    u32 s4 = 0x510e527fu, s5 = 0x9b05688cu, s6 = 0x1f83d9abu, s7 = 0x5be0cd19u;
    u32 s8 = 0x6a09e667u, s9 = 0xbb67ae85u, s10 = 0x3c6ef372u, s11 = 0xa54ff53au;
    u32 s12 = 0, s13 = 0, s14 = 32, s15 = B3_CHUNK_START | B3_CHUNK_END | B3_ROOT;
#pragma unroll
    for (int rd = 0; rd < 7; rd++) {
        B3_G(s0, s4, s8, s12, w[0], w[1]);   B3_G(s1, s5, s9, s13, w[2], w[3]);
        B3_G(s2, s6, s10, s14, w[4], w[5]);  B3_G(s3, s7, s11, s15, w[6], w[7]);
        B3_G(s0, s5, s10, s15, w[8], w[9]);  B3_G(s1, s6, s11, s12, w[10], w[11]);
        B3_G(s2, s7, s8, s13, w[12], w[13]); B3_G(s3, s4, s9, s14, w[14], w[15]);
        if (rd < 6) {
            u32 t[16] = {w[2], w[6], w[3], w[10], w[7], w[0], w[4], w[13], w[1], w[11], w[12], w[5], w[9], w[14], w[15], w[8]};
#pragma unroll
            for (int i = 0; i < 16; i++) w[i] = t[i];
        }
    }
    return make_uint4(s0 ^ s8, s1 ^ s9, s2 ^ s10, s3 ^ s11);
}

// ---- AES-MMO node -------------------------------------------------------------------------------
// ARM's AESE is AddRoundKey, SubBytes, ShiftRows (in that order) and AESMC is MixColumns; the
// reference runs ten AESE steps keyed L, R, L, R, ... on the state L^R, MixColumns after the
// first nine, and XORs L^R back in.  SubBytes + ShiftRows + MixColumns of one column is four
// lookups in a table T0[x] = (2 S[x], S[x], S[x], 3 S[x]) and byte rotations of it.
__constant__ u32 AES_T0[256];
__constant__ unsigned char AES_SBOX[256];

struct AesTables { u32 t0[256]; unsigned char sbox[256]; };
// S-box from its definition (FIPS-197 5.1.1): inverse in GF(2^8) mod x^8+x^4+x^3+x+1, then the affine map.
inline AesTables aes_make_tables() {
    AesTables t;
    auto xt = [](unsigned a) { return ((a << 1) ^ ((a & 0x80) ? 0x11b : 0)) & 0xff; };
    auto mul = [&](unsigned a, unsigned b) { unsigned r = 0; while (b) { if (b & 1) r ^= a; a = xt(a); b >>= 1; } return r; };
    for (unsigned x = 0; x < 256; x++) {
        unsigned inv = 0;
        if (x) { inv = 1; for (int i = 0; i < 254; i++) inv = mul(inv, x); }
        unsigned s = inv;
        for (int i = 1; i <= 4; i++) s ^= ((inv << i) | (inv >> (8 - i))) & 0xff;
        s ^= 0x63;
        t.sbox[x] = (unsigned char)s;
        unsigned s2 = xt(s), s3 = s2 ^ s;
        t.t0[x] = s2 | (s << 8) | (s << 16) | (s3 << 24);
    }
    return t;
}

__device__ __forceinline__ u32 rotl8(u32 x, int bytes) { return __funnelshift_l(x, x, 8 * bytes); }
__device__ __forceinline__ uint4 aes_node(uint4 l, uint4 r, const u32* __restrict__ T0, const unsigned char* __restrict__ S) {
    const u32 x0 = l.x ^ r.x, x1 = l.y ^ r.y, x2 = l.z ^ r.z, x3 = l.w ^ r.w;
    u32 c0 = x0, c1 = x1, c2 = x2, c3 = x3;
#pragma unroll
    for (int rd = 0; rd < 10; rd++) {
        const uint4 k = (rd & 1) ? r : l;
        c0 ^= k.x; c1 ^= k.y; c2 ^= k.z; c3 ^= k.w;
        u32 n0, n1, n2, n3;
        if (rd < 9) {
            n0 = T0[c0 & 255] ^ rotl8(T0[(c1 >> 8) & 255], 1) ^ rotl8(T0[(c2 >> 16) & 255], 2) ^ rotl8(T0[c3 >> 24], 3);
            n1 = T0[c1 & 255] ^ rotl8(T0[(c2 >> 8) & 255], 1) ^ rotl8(T0[(c3 >> 16) & 255], 2) ^ rotl8(T0[c0 >> 24], 3);
            n2 = T0[c2 & 255] ^ rotl8(T0[(c3 >> 8) & 255], 1) ^ rotl8(T0[(c0 >> 16) & 255], 2) ^ rotl8(T0[c1 >> 24], 3);
            n3 = T0[c3 & 255] ^ rotl8(T0[(c0 >> 8) & 255], 1) ^ rotl8(T0[(c1 >> 16) & 255], 2) ^ rotl8(T0[c2 >> 24], 3);
        } else {
            n0 = (u32)S[c0 & 255] | ((u32)S[(c1 >> 8) & 255] << 8) | ((u32)S[(c2 >> 16) & 255] << 16) | ((u32)S[c3 >> 24] << 24);
            n1 = (u32)S[c1 & 255] | ((u32)S[(c2 >> 8) & 255] << 8) | ((u32)S[(c3 >> 16) & 255] << 16) | ((u32)S[c0 >> 24] << 24);
            n2 = (u32)S[c2 & 255] | ((u32)S[(c3 >> 8) & 255] << 8) | ((u32)S[(c0 >> 16) & 255] << 16) | ((u32)S[c1 >> 24] << 24);
            n3 = (u32)S[c3 & 255] | ((u32)S[(c0 >> 8) & 255] << 8) | ((u32)S[(c1 >> 16) & 255] << 16) | ((u32)S[c2 >> 24] << 24);
        }
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    }
    return make_uint4(c0 ^ x0, c1 ^ x1, c2 ^ x2, c3 ^ x3);
}

// ---- tree storage ---------------------------------------------------------------------------------
__host__ __device__ __forceinline__ size_t mk_layer_offset(u32 h, u32 k) { return (size_t(1) << h) - (size_t(1) << (h - k + 1)); }
__host__ __device__ __forceinline__ size_t mk_node_count(u32 h) { return (size_t(1) << h) - 1; }

constexpr int MK_TILE_LOG = 10;
constexpr int MK_TILE = 1 << MK_TILE_LOG;
constexpr int MK_THREADS = 256;

// How a CTA obtains its MK_TILE inputs.
enum MkMode : int {
    MK_VALUES = 0,   // u32 leaves (zero beyond n_valid)
    MK_DIGESTS = 1,  // nodes of layer k0 of the same tree
    MK_FOLD = 2      // leaves produced on the fly by a Basefold codeword fold (see basefold.cuh)
};

struct MkFold {
    const u32* prev;      // previous codeword, 2 * half values
    u32* out;             // folded codeword, half values
    const u32* weights;   // w_level of this fold, w_len values
    const u32* alpha;     // device-resident challenge
    u32* eval_src;        // coefficient buffer being evaluated (eval_half * 2 live values), or null
    u32* eval_dst;        // where the folded coefficients go (may equal eval_src)
    size_t w_len, eval_half;
    // first round only: coefficients are read through a row-padded view of a matrix
    const u32* coef; u32 coef_rows, coef_cols, coef_log_cols_pad; int eval_from_coef;
    // batch openings: values added to the folded codeword before it is stored and hashed (the already scaled sum of the
    // codewords that join the chain at this length), or null
    const u32* add;
};

__device__ __forceinline__ u32 coef_at(const u32* __restrict__ p, u32 rows, u32 cols, u32 log_cols_pad, size_t i) {
    size_t r = i >> log_cols_pad, c = i & ((size_t(1) << log_cols_pad) - 1);
    return (r < rows && c < cols) ? p[r * cols + c] : 0u;
}

// One CTA: MK_TILE inputs (fewer when the whole level is smaller) -> up to MK_TILE_LOG layers.
// n_in = number of inputs at level k0 (a power of two); h = height of the tree.
template <int KIND, int MODE>
__global__ void __launch_bounds__(MK_THREADS) mk_tile_kernel(const u32* __restrict__ values, size_t n_valid, size_t n_in, u32 k0, u32 h,
                                                            uint4* __restrict__ nodes, MkFold fold) {
    __shared__ uint4 bufA[MK_TILE];
    __shared__ uint4 bufB[MK_TILE / 2];
    __shared__ u32 t0_s[KIND == NODE_AES_MMO ? 256 : 1];
    __shared__ unsigned char sb_s[KIND == NODE_AES_MMO ? 256 : 1];
    if (KIND == NODE_AES_MMO) {
        for (int i = threadIdx.x; i < 256; i += MK_THREADS) { t0_s[i] = AES_T0[i]; sb_s[i] = AES_SBOX[i]; }
    }
    const size_t tile = n_in < (size_t)MK_TILE ? n_in : (size_t)MK_TILE;
    const size_t base = (size_t)blockIdx.x * tile;

    if (MODE == MK_DIGESTS) {
        const uint4* in = nodes + mk_layer_offset(h, k0) + base;
        for (size_t i = threadIdx.x; i < tile; i += MK_THREADS) bufA[i] = in[i];
    } else if (MODE == MK_VALUES) {
        for (size_t i = threadIdx.x; i < tile; i += MK_THREADS) {
            size_t g = base + i;
            bufA[i] = make_uint4(g < n_valid ? values[g] : 0u, 0, 0, 0);
        }
    } else {
        const size_t half = n_in;
        const Fp alpha{*fold.alpha};
        const Fp two_inv{1073741824u};
        for (size_t i = threadIdx.x; i < tile; i += MK_THREADS) {
            size_t j = base + i;
            Fp l{fold.prev[j]}, r{fold.prev[j + half]};
            Fp w{fold.weights[j & (fold.w_len - 1)]};
            Fp f = (l + r) * two_inv + alpha * ((l - r) * w);
            if (fold.add) f = f + Fp{fold.add[j]};
            fold.out[j] = f.v;
            bufA[i] = make_uint4(f.v, 0, 0, 0);
            if (fold.eval_dst && j < fold.eval_half) {
                Fp a, b;
                if (fold.eval_from_coef) {
                    a.v = coef_at(fold.coef, fold.coef_rows, fold.coef_cols, fold.coef_log_cols_pad, j);
                    b.v = coef_at(fold.coef, fold.coef_rows, fold.coef_cols, fold.coef_log_cols_pad, j + fold.eval_half);
                } else {
                    a.v = fold.eval_src[j]; b.v = fold.eval_src[j + fold.eval_half];
                }
                fold.eval_dst[j] = ((fp_one() - alpha) * a + alpha * b).v;
            }
        }
    }
    __syncthreads();

    uint4* cur = bufA;
    uint4* nxt = bufB;
    size_t cnt = tile;
    u32 k = k0;
    while (cnt > 1 && k < h) {
        const size_t out_cnt = cnt >> 1;
        k++;
        uint4* layer = nodes + mk_layer_offset(h, k) + (size_t)blockIdx.x * out_cnt;
        for (size_t i = threadIdx.x; i < out_cnt; i += MK_THREADS) {
            uint4 d = KIND == NODE_AES_MMO ? aes_node(cur[2 * i], cur[2 * i + 1], t0_s, sb_s) : b3_node(cur[2 * i], cur[2 * i + 1]);
            nxt[i] = d;
            layer[i] = d;
        }
        __syncthreads();
        uint4* t = cur; cur = nxt; nxt = t;
        cnt = out_cnt;
    }
}

// Raw authentication data of opened positions: for position p of a tree of height h over
// `values`, out = [value, sibling value, sibling digest at level 1, ..., level h-1] (2 + 4 (h-1)
// words).  The host drops the digests a batch proof does not need (pcs.rs:290-337).
__device__ inline void mk_gather_path(const u32* __restrict__ values, size_t n_valid, const uint4* __restrict__ nodes, u32 h, size_t p,
                                      u32* out, int lane, int nlanes) {
    for (u32 k = lane; k <= h; k += nlanes) {
        if (k == 0) {
            out[0] = p < n_valid ? values[p] : 0u;
        } else if (k == 1) {
            size_t s = p ^ 1;
            out[1] = s < n_valid ? values[s] : 0u;
        } else {
            size_t s = (p >> (k - 1)) ^ 1;
            uint4 d = nodes[mk_layer_offset(h, k - 1) + s];
            u32* o = out + 2 + 4 * (size_t)(k - 2);
            o[0] = d.x; o[1] = d.y; o[2] = d.z; o[3] = d.w;
        }
    }
}
// Positions given by the host (the stand-alone Merkle entry points).
__global__ void mk_open_kernel(const u32* __restrict__ values, size_t n_valid, const uint4* __restrict__ nodes, u32 h,
                               const unsigned long long* __restrict__ pos, u32 n_pos, u32* out) {
    for (u32 q = blockIdx.x; q < n_pos; q += gridDim.x)
        mk_gather_path(values, n_valid, nodes, h, (size_t)pos[q], out + (size_t)q * (2 + 4 * (size_t)(h - 1)), threadIdx.x, blockDim.x);
}

}  // namespace zkb
