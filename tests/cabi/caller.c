/* A caller of the C ABI written in plain C (what a cgo / bindgen / FFI user of include/zkb200.h sees):
 * it proves one product sumcheck with EF challenges (prove_product_ef, sumcheck.rs:1204-1258), one
 * succinct matmul proof (matmul.rs:963-997), checks a Basefold opening with the verifier
 * (basefold.rs:368-396, 611-748), opens two polynomials of different sizes with one batch Basefold
 * (basefold.rs:1183-1378, 959-1137) and proves and verifies a small row attention (attention.rs:116-385),
 * and prints everything as hex so that the test can compare it with what the oracle computes from the
 * same seeded inputs.
 *
 *   caller <num_vars> <m> <n>
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "zkb200.h"

#define P 2147483647u

static uint32_t lcg_state = 12345u;
static uint32_t next_u32(void) {           /* numerical-recipes LCG, reduced into [0, p) */
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return (lcg_state >> 1) % P;
}
static void hex(const char* name, const void* p, size_t n) {
    const unsigned char* b = (const unsigned char*)p;
    printf("%s ", name);
    for (size_t i = 0; i < n; i++) printf("%02x", b[i]);
    printf("\n");
}
#define CHECK(call)                                                                   \
    do {                                                                              \
        int32_t rc_ = (call);                                                         \
        if (rc_ != ZKB_OK) { fprintf(stderr, "%s -> %d: %s\n", #call, rc_, zkb_last_error(ctx)); return 1; } \
    } while (0)

int main(int argc, char** argv) {
    if (argc < 4) return 2;
    const uint32_t nv = (uint32_t)atoi(argv[1]);
    const size_t m = (size_t)atoi(argv[2]), n = (size_t)atoi(argv[3]);
    zkb_ctx* ctx = NULL;
    if (zkb_ctx_create(0, &ctx) != ZKB_OK) { fprintf(stderr, "no CUDA device\n"); return 3; }

    /* product sumcheck, EF challenges */
    const size_t len = (size_t)1 << nv;
    uint32_t* f = (uint32_t*)malloc(len * 4);
    uint32_t* g = (uint32_t*)malloc(len * 4);
    for (size_t i = 0; i < len; i++) f[i] = next_u32();
    for (size_t i = 0; i < len; i++) g[i] = next_u32();
    zkb_transcript* tr = NULL;
    CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-caller", 8, &tr));
    uint32_t* polys = (uint32_t*)calloc((size_t)nv * 2 * 4, 4);
    uint32_t* chal = (uint32_t*)calloc((size_t)nv * 4, 4);
    uint32_t fin[8];
    const uint32_t* tabs[2] = {f, g};
    CHECK(zkb_sumcheck_prove(ctx, tr, ZKB_SC_PRODUCT_EF, tabs, nv, 0, polys, chal, fin));
    hex("polys", polys, (size_t)nv * 2 * 16);
    hex("chal", chal, (size_t)nv * 16);
    hex("finals", fin, 32);

    /* succinct matmul proof on the same transcript */
    uint32_t* W = (uint32_t*)malloc(m * n * 4);
    uint32_t* x = (uint32_t*)malloc(n * 4);
    uint32_t* y = (uint32_t*)malloc(m * 4);
    for (size_t i = 0; i < m * n; i++) W[i] = next_u32();
    for (size_t i = 0; i < n; i++) x[i] = next_u32();
    CHECK(zkb_matvec_forward(ctx, W, x, m, n, 0, y));
    hex("y", y, m * 4);
    size_t cap = (size_t)1 << 20, plen = 0;
    uint8_t* out = (uint8_t*)malloc(cap);
    CHECK(zkb_prove_matmul_succinct_ef(ctx, tr, W, x, y, m, n, 0, out, cap, &plen));
    hex("matmul", out, plen);

    /* Basefold commitment + opening of f, then the verifier on the bytes */
    uint32_t point[32];
    for (uint32_t i = 0; i < nv; i++) point[i] = next_u32();
    CHECK(zkb_basefold_commit_and_prove(ctx, tr, f, len, point, nv, 0, ZKB_NODE_BLAKE3, out, cap, &plen));
    hex("basefold", out, plen);
    zkb_transcript* tv = NULL;
    CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-verify", 8, &tv));
    CHECK(zkb_tr_absorb_bytes(tv, out, 16));
    uint32_t claimed = 0;
    memcpy(&claimed, out + plen - 12, 4);
    int32_t ok = 0;
    /* the opening was made on `tr` after other traffic, so under a fresh transcript it must be rejected ... */
    CHECK(zkb_basefold_verify_opening(ctx, tv, out, plen, point, nv, claimed, ZKB_NODE_BLAKE3, &ok));
    printf("verify_other_transcript %d\n", ok);
    /* ... and a proof made on a transcript in the same state is accepted */
    zkb_transcript* tp = NULL;
    CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-verify", 8, &tp));
    CHECK(zkb_basefold_commit_and_prove(ctx, tp, f, len, point, nv, 0, ZKB_NODE_BLAKE3, out, cap, &plen));
    zkb_transcript* tv2 = NULL;
    CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-verify", 8, &tv2));
    CHECK(zkb_tr_absorb_bytes(tv2, out, 16));
    memcpy(&claimed, out + plen - 12, 4);
    CHECK(zkb_basefold_verify_opening(ctx, tv2, out, plen, point, nv, claimed, ZKB_NODE_BLAKE3, &ok));
    printf("verify_same_transcript %d\n", ok);

    /* batch Basefold: f (2^nv coefficients) and the first 2^(nv-2) - 3 values of g, one fold chain; then its verifier */
    {
        const uint32_t* polys2[2] = {f, g};
        const size_t ns[2] = {len, (len >> 2) - 3};
        const uint32_t lns[2] = {nv, nv - 2};
        zkb_bf_batch* batch = NULL;
        CHECK(zkb_basefold_batch_precommit(ctx, polys2, ns, lns, 2, 0, ZKB_NODE_BLAKE3, &batch));
        zkb_transcript* tb = NULL;
        CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-batch", 7, &tb));
        CHECK(zkb_basefold_batch_prove(batch, tb, 0, out, cap, &plen));
        hex("batch", out, plen);
        zkb_transcript* tbv = NULL;
        CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-batch", 7, &tbv));
        CHECK(zkb_basefold_batch_verify_opening(ctx, tbv, out, plen, ZKB_NODE_BLAKE3, &ok));
        printf("batch_verify %d\n", ok);
        zkb_basefold_batch_destroy(batch);
        zkb_tr_free(tb); zkb_tr_free(tbv);
    }

    /* row attention, 2 heads x 4 positions x d_head 4, over a 256-entry table (any table of positive outputs serves the protocol) */
    {
        uint32_t table[256], q[32], k[32], v[32], att[32];
        for (uint32_t i = 0; i < 256; i++) table[i] = (i * 7u + 1u) % 1000u + 1u;
        for (int i = 0; i < 32; i++) { q[i] = next_u32() % 3u; k[i] = next_u32() % 3u; v[i] = next_u32(); }
        zkb_transcript* ta = NULL;
        CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-attn", 6, &ta));
        CHECK(zkb_prove_row_attention(ctx, ta, q, k, v, 2, 4, 4, table, 256, 0, att, out, cap, &plen));
        hex("attention", out, plen);
        hex("attention_out", att, sizeof att);
        zkb_transcript* tav = NULL;
        CHECK(zkb_tr_new(ctx, (const uint8_t*)"c-attn", 6, &tav));
        CHECK(zkb_verify_row_attention(ctx, tav, out, plen, k, v, 2, 0, 4, 4, 0, &ok));
        printf("attention_verify %d\n", ok);
        zkb_tr_free(ta); zkb_tr_free(tav);
    }

    zkb_tr_free(tr); zkb_tr_free(tv); zkb_tr_free(tp); zkb_tr_free(tv2);
    zkb_ctx_destroy(ctx);
    free(f); free(g); free(polys); free(chal); free(W); free(x); free(y); free(out);
    return 0;
}
