"""Stand-alone field helpers of the C ABI against the oracle: MLE evaluation (m31_ops.rs:11-26,
155-171), batch inversion (lookup.rs:322-368), and the host-side alignment checks on device
pointers that kernels read with 16-byte loads."""
import ctypes as C

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import _lib, protocols as zp
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1
u32p = C.POINTER(C.c_uint32)


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def _rand(rng, n):
    return rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)


def _shifted(buf, words):
    """Device pointer `words` u32 past the start of a DeviceBuffer."""
    return C.cast(C.c_void_p(C.addressof(buf.ptr.contents) + 4 * words), u32p)


@pytest.mark.parametrize("k", [0, 1, 2, 5, 10, 11, 13, 17])
def test_mle_evaluate_matches_oracle(ctx, k):
    rng = np.random.default_rng(100 + k)
    n = 1 << k
    ev, pt = _rand(rng, n), _rand(rng, k)
    pt_ef = _rand(rng, 4 * k).reshape(k, 4)
    ev_ef = _rand(rng, 4 * n).reshape(n, 4)
    assert zp.mle_evaluate(ctx, ev, pt) == O.mle_evaluate(ev, pt)
    assert zp.mle_evaluate_ef(ctx, ev, pt_ef).tolist() == O.mle_evaluate_ef(ev, pt_ef).tolist()
    assert zp.mle_evaluate_ef(ctx, ev_ef, pt_ef, evals_ef=True).tolist() == O.mle_evaluate_efef(ev_ef, pt_ef).tolist()
    # device-resident table, and extreme values
    assert zp.mle_evaluate(ctx, ctx.upload(ev), pt) == O.mle_evaluate(ev, pt)
    top = np.full(n, P - 1, np.uint32)
    assert zp.mle_evaluate_ef(ctx, ctx.upload(top), np.full((k, 4), P - 1, np.uint32)).tolist() == \
        O.mle_evaluate_ef(top, np.full((k, 4), P - 1, np.uint32)).tolist()


def test_mle_evaluate_ragged_table_is_zero_padded(ctx):
    """n < 2^k: the missing entries count as zero (the reference pads before calling)."""
    rng = np.random.default_rng(7)
    for k, n in [(12, 2560), (14, 9728), (11, 1025), (3, 5), (4, 0)]:
        ev, pt = _rand(rng, n), _rand(rng, 4 * k).reshape(k, 4)
        full = np.zeros(1 << k, np.uint32)
        full[:n] = ev
        assert zp.mle_evaluate_ef(ctx, ev, pt).tolist() == O.mle_evaluate_ef(full, pt).tolist()
        ptb = _rand(rng, k)
        assert zp.mle_evaluate(ctx, ev, ptb) == O.mle_evaluate(full, ptb)


def test_mle_evaluate_literal_of_the_reference(ctx):
    """m31_ops.rs:198-214 (test_mle_evaluate): evals [1,2,3,4] at (0,0)=1, (1,1)=4, and the linear mix."""
    ev = np.array([1, 2, 3, 4], np.uint32)
    assert zp.mle_evaluate(ctx, ev, [0, 0]) == 1 and zp.mle_evaluate(ctx, ev, [1, 1]) == 4
    assert zp.mle_evaluate(ctx, ev, [1, 0]) == 3 and zp.mle_evaluate(ctx, ev, [0, 1]) == 2


@pytest.mark.parametrize("n", [1, 3, 4, 5, 1000, 13825])
def test_batch_inverse_matches_oracle(ctx, n):
    rng = np.random.default_rng(n)
    v = rng.integers(1, P, n, dtype=np.int64).astype(np.uint32)
    got = zp.batch_inverse(ctx, v)
    assert got.tolist() == [O.f_inv(int(a)) for a in v]
    ve = _rand(rng, 4 * n).reshape(n, 4)
    ve[0] = [0, 0, 0, 5]                      # only one coordinate nonzero: still invertible
    gote = zp.batch_inverse(ctx, ve, ef=True)
    assert gote.tolist() == [O.ef_inv(a).tolist() for a in ve]
    assert all(O.ef_mul(a, b).tolist() == [1, 0, 0, 0] for a, b in zip(ve[:16], gote[:16]))
    # in place on the device, as the reference's Metal hook does
    d = ctx.upload(ve)
    zp.batch_inverse(ctx, d, ef=True)
    assert d.download().tolist() == gote.tolist()


def test_batch_inverse_of_zero_is_an_error_and_context_survives(ctx):
    v = np.array([3, 0, 7, 9, 11], np.uint32)
    with pytest.raises(zk.ZkbError) as e:
        zp.batch_inverse(ctx, v)
    assert e.value.code == 9
    with pytest.raises(zk.ZkbError) as e:
        zp.batch_inverse(ctx, np.zeros((2, 4), np.uint32), ef=True)
    assert e.value.code == 9
    assert zp.batch_inverse(ctx, np.array([2], np.uint32)).tolist() == [O.f_inv(2)]
    assert zp.batch_inverse(ctx, np.zeros(0, np.uint32)).size == 0


def test_misaligned_device_pointers_are_refused_on_the_host(ctx):
    """A device pointer that kernels read with 16-byte loads but that is only 4-byte aligned must
    come back as ZKB_E_ARG before any launch (on the GPU it would fault the whole context)."""
    L = _lib.lib()
    rng = np.random.default_rng(3)
    m, n = 8, 16
    buf = ctx.upload(_rand(rng, m * n + 8))
    w_off = _shifted(buf, 1)
    r = _rand(rng, 4 * 3)
    out = np.zeros(4 * n, np.uint32)
    st = L.zkb_fold_eq_matvec(ctx.h, w_off, C.c_size_t(m), C.c_size_t(n), r.ctypes.data_as(u32p), C.c_uint32(3), C.c_int32(1), C.c_int32(1),
                              out.ctypes.data_as(u32p))
    assert st == 2 and b"16-byte" in L.zkb_last_error(ctx.h)
    x = _rand(rng, n)
    y = np.zeros(m, np.uint32)
    assert L.zkb_matvec_forward(ctx.h, w_off, x.ctypes.data_as(u32p), C.c_size_t(m), C.c_size_t(n), C.c_int32(1), y.ctypes.data_as(u32p)) == 2
    # an odd column count is read with scalar loads: the same pointer is fine there
    n_odd = 15
    w_host = buf.download()[1:1 + m * n_odd]
    assert L.zkb_matvec_forward(ctx.h, w_off, x.ctypes.data_as(u32p), C.c_size_t(m), C.c_size_t(n_odd), C.c_int32(1), y.ctypes.data_as(u32p)) == 0
    assert y.tolist() == O.matmul_forward(w_host, x[:n_odd], m, n_odd).tolist()
    # EF tables of a sumcheck on the device
    tr = zk.Transcript(ctx, b"align")
    tabs = (u32p * 3)(_shifted(buf, 1), _shifted(buf, 1), None)
    o = np.zeros(64, np.uint32).ctypes.data_as(u32p)
    assert L.zkb_sumcheck_prove(ctx.h, tr.h, C.c_int32(zk.SC_PRODUCT_EF_FULL), tabs, C.c_uint32(2), C.c_int32(1), o, o, o) == 2
    # base-field tables only need 4-byte alignment (the scalar launches take over): same proof as from the host
    nv = 14                                    # large enough for the multi-CTA round launches
    big_h = _rand(rng, (1 << nv) + 8)
    big = ctx.upload(big_h)
    f, g = big_h[1:1 + (1 << nv)], big_h[3:3 + (1 << nv)]
    tabs = (u32p * 3)(_shifted(big, 1), _shifted(big, 3), None)
    polys, chal, fin = np.zeros((nv, 2, 4), np.uint32), np.zeros((nv, 4), np.uint32), np.zeros((2, 4), np.uint32)
    t1 = zk.Transcript(ctx, b"align2")
    assert L.zkb_sumcheck_prove(ctx.h, t1.h, C.c_int32(zk.SC_PRODUCT_EF), tabs, C.c_uint32(nv), C.c_int32(1), polys.ctypes.data_as(u32p),
                                chal.ctypes.data_as(u32p), fin.ctypes.data_as(u32p)) == 0
    ep, ec, ef_ = O.prove("product_ef", O.Transcript(b"align2"), [f, g], nv)
    assert polys.reshape(nv, -1).tolist() == ep.tolist() and chal.tolist() == ec.tolist() and fin.tolist() == ef_.tolist()
    # the allocation-free fold names the pointer in its own error buffer
    err = C.create_string_buffer(256)
    eq = ctx.upload(_rand(rng, 4 * m))
    dst = ctx.upload(np.zeros(4 * n, np.uint32))
    st = L.zkb_fold_eq_matvec_ef_noalloc(w_off, C.c_size_t(m), C.c_size_t(n), eq.ptr, dst.ptr, C.c_void_p(ctx.stream), err, C.c_size_t(256))
    assert st == 2 and b"16-byte" in err.value


def test_context_options_keep_the_proof_bytes(ctx):
    """The tuning options change launch shapes only: the plain tail and other thread counts give the same proof."""
    rng = np.random.default_rng(5)
    nv = 13
    f, g = _rand(rng, 4 << nv).reshape(-1, 4), _rand(rng, 4 << nv).reshape(-1, 4)
    ref = O.prove("product_ef_full", O.Transcript(b"opt"), [f, g], nv)
    c2 = zk.Context(0)
    try:
        for opt, val in [(None, 0), (c2.OPT_PLAIN_TAIL, 1), (c2.OPT_PLAIN_TAIL, 0), (c2.OPT_PIPE_THREADS, 256), (c2.OPT_SINGLE_CTA_THREADS, 512)]:
            if opt is not None:
                c2.set_option(opt, val)
            proof, fs, gs = zk.prove_product_ef_full(f, g, nv, zk.Transcript(c2, b"opt"))
            assert proof.round_polys.reshape(nv, -1).tolist() == ref[0].tolist()
            assert fs.tolist() == ref[2][0].tolist() and gs.tolist() == ref[2][1].tolist()
        # product sumcheck over base-field tables: two challenges folded per pass (default), one per pass, and
        # the vector widths of the two-challenge pass all give the same proof
        nv2 = 17
        fb, gb = _rand(rng, 1 << nv2), _rand(rng, 1 << nv2)
        refb = O.prove("product_ef", O.Transcript(b"opt2"), [fb, gb], nv2)
        for opt, val in [(c2.OPT_NO_FUSED_FOLD, 1), (c2.OPT_NO_FUSED_FOLD, 0), (c2.OPT_FOLD2_VEC, 1), (c2.OPT_FOLD2_VEC, 4), (c2.OPT_FOLD2_VEC, 2)]:
            c2.set_option(opt, val)
            proof, fs, gs = zk.prove_product_ef(fb, gb, nv2, zk.Transcript(c2, b"opt2"))
            assert proof.round_polys.reshape(nv2, -1).tolist() == refb[0].tolist() and proof.challenges.tolist() == refb[1].tolist()
            assert fs.tolist() == refb[2][0].tolist() and gs.tolist() == refb[2][1].tolist()
        with pytest.raises(zk.ZkbError):
            c2.set_option(c2.OPT_PIPE_THREADS, 100)
        with pytest.raises(zk.ZkbError):
            c2.set_option(77, 1)
    finally:
        c2.close()


def test_requantize_lookup_matches_host_statement(ctx):
    """zkb_requantize_lookup against the numpy statement of requantize_to_i16_field
    (transformer/mod.rs:293-324) and a table lookup: small values pass through, large ones are scaled."""
    from zklm_compile_b200 import tables
    rng = np.random.default_rng(31)
    gelu = tables.build_gelu_table(1000)
    tdev = ctx.upload(gelu)
    for n, lim in [(1, 5), (1000, 100), (1024, 1 << 20), (4099, 1 << 30)]:
        v = np.mod(rng.integers(-lim, lim + 1, n), P).astype(np.uint32)
        q, t = zp.requantize_lookup(ctx, v, tdev)
        exp = tables.requantize_to_i16_field(v)
        assert q.tolist() == exp.tolist()
        s = np.where(exp > P // 2, exp.astype(np.int64) - P, exp.astype(np.int64))
        assert t.tolist() == gelu[np.mod(s, gelu.size)].tolist()
        assert zp.requantize_lookup(ctx, v).tolist() == exp.tolist()
    tdev.free()


@pytest.mark.parametrize("m,n", [(1, 128), (5, 132), (77, 1024), (300, 2560), (1030, 768), (37, 9728), (9, 12288), (2051, 256), (64, 16384), (3, 20000), (50, 130)])
def test_matvec_forward_ring_and_register_kernels(ctx, m, n):
    """y = W x through both forward-matvec kernels: the register-staged one (the default) and the
    shared-memory ring filled by bulk copies (ZKB_OPT_MATVEC_RING; rows of a multiple of 16 bytes up to
    64 KB, tiles of 16 .. 1 rows, ragged last tile, more tiles than SMs; n = 130 and n = 20000 fall back)."""
    rng = np.random.default_rng(m * 7 + n)
    w = rng.integers(0, P, m * n, dtype=np.int64).astype(np.uint32)
    x = rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)
    exp = O.matmul_forward(w, x, m, n)
    for ring in (0, 1):
        ctx.set_option(ctx.OPT_MATVEC_RING, ring)
        try:
            assert zp.matmul_forward(ctx, w, x, m, n).tolist() == exp.tolist()
        finally:
            ctx.set_option(ctx.OPT_MATVEC_RING, 0)
