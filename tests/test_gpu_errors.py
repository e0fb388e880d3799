"""Error behaviour of the C ABI on a GPU: bad arguments come back as status codes with a message,
short output buffers report the needed length, and the context keeps working afterwards."""
import ctypes as C

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import _lib, pcs as zpc, protocols as zp
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1
u32p = C.POINTER(C.c_uint32)


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def test_bad_arguments_are_status_codes(ctx):
    L = _lib.lib()
    tr = zk.Transcript(ctx, b"e")
    buf = (C.c_uint8 * 64)()
    n = C.c_size_t()
    one = np.ones(4, np.uint32)
    p1 = one.ctypes.data_as(u32p)
    # unknown sumcheck kind, zero rounds
    tabs = (u32p * 3)(p1, p1, p1)
    out = np.zeros(64, np.uint32).ctypes.data_as(u32p)
    assert L.zkb_sumcheck_prove(ctx.h, tr.h, C.c_int32(99), tabs, C.c_uint32(2), C.c_int32(0), out, out, out) == 2
    assert L.zkb_sumcheck_prove(ctx.h, tr.h, C.c_int32(0), tabs, C.c_uint32(0), C.c_int32(0), out, out, out) == 2
    # lookup table of an unsupported size, empty lookup
    assert L.zkb_prove_lookup_ef(ctx.h, tr.h, p1, C.c_size_t(100), p1, p1, C.c_size_t(4), buf, C.c_size_t(64), C.byref(n)) == 2
    assert L.zkb_prove_lookup(ctx.h, tr.h, p1, C.c_size_t(256), p1, p1, C.c_size_t(0), buf, C.c_size_t(64), C.byref(n)) == 2
    # unknown node hash / binding mode
    root = (C.c_uint8 * 16)()
    assert L.zkb_merkle_root(ctx.h, p1, C.c_size_t(4), C.c_int32(0), C.c_int32(7), root) == 2
    assert b"node hash" in L.zkb_last_error(ctx.h)
    assert L.zkb_prove_matmul_succinct_ef_bind(ctx.h, tr.h, p1, p1, p1, C.c_size_t(2), C.c_size_t(2), C.c_int32(0), C.c_int32(5), C.c_int32(0),
                                               buf, C.c_size_t(64), C.byref(n)) == 2
    # opened position outside the tree
    idx = (C.c_uint64 * 1)(9)
    assert L.zkb_merkle_batch_open(ctx.h, p1, C.c_size_t(4), C.c_int32(0), C.c_int32(0), idx, C.c_size_t(1), buf, C.c_size_t(64), C.byref(n)) == 2
    # exchange with a world that is not a power of two
    x = C.c_void_p()
    assert L.zkb_xch_create(ctx.h, C.c_uint32(3), C.c_uint32(0), C.byref(x)) == 2


def test_short_output_buffer_reports_length_and_context_survives(ctx):
    L = _lib.lib()
    rng = np.random.default_rng(0)
    w = rng.integers(0, P, 64, dtype=np.int64).astype(np.uint32)
    x = rng.integers(0, P, 8, dtype=np.int64).astype(np.uint32)
    y = O.matmul_forward(w, x, 8, 8)
    tr = zk.Transcript(ctx, b"short")
    buf = (C.c_uint8 * 16)()
    n = C.c_size_t()
    st = L.zkb_prove_matmul_succinct_ef(ctx.h, tr.h, w.ctypes.data_as(u32p), x.ctypes.data_as(u32p), y.ctypes.data_as(u32p),
                                        C.c_size_t(8), C.c_size_t(8), C.c_int32(0), buf, C.c_size_t(16), C.byref(n))
    assert st == 7 and n.value > 16
    # the same context still proves correctly (fresh transcripts on both sides)
    t2, o2 = zk.Transcript(ctx, b"again"), O.Transcript(b"again")
    assert zp.prove_matmul_succinct_ef(w, x, y, 8, 8, t2) == O.prove_matmul_succinct(o2, w, x, y, 8, 8, ef=True)
    # and the Merkle / Basefold entry points accept the smallest inputs
    assert zpc.merkle_root(ctx, np.array([5], np.uint32)) == O.merkle_root(np.array([5], np.uint32), 0)


def test_verifier_entry_points_refuse_bad_arguments(ctx):
    """The verifiers answer malformed input with a status code, never with a verdict: null pointers, bytes
    that do not decode, an unknown node hash, a layer that has no forward trace yet, an end without a begin."""
    import hashlib
    from zklm_compile_b200 import qwen as zq
    from tests.util import load_qwen_golden, rand_layer
    L = _lib.lib()
    ok = C.c_int32(7)
    tr = zk.Transcript(ctx, b"v")
    pt = np.ones(4, np.uint32)
    junk = (C.c_uint8 * 40)(*range(40))
    assert L.zkb_basefold_verify_opening(ctx.h, tr.h, None, C.c_size_t(0), pt.ctypes.data_as(u32p), C.c_uint32(4), C.c_uint32(0), C.c_int32(0), C.byref(ok)) == 2
    assert L.zkb_basefold_verify_opening(ctx.h, tr.h, junk, C.c_size_t(40), pt.ctypes.data_as(u32p), C.c_uint32(4), C.c_uint32(0), C.c_int32(0), C.byref(ok)) == 2
    assert ok.value == 0 and b"decode" in L.zkb_last_error(ctx.h)
    c = np.arange(1, 65, dtype=np.uint32)
    point = np.arange(3, 9, dtype=np.uint32)
    blob = zpc.basefold_commit_and_prove(ctx, zk.Transcript(ctx, b"v"), c, point)
    buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
    assert L.zkb_basefold_verify_opening(ctx.h, tr.h, buf, C.c_size_t(len(blob)), point.ctypes.data_as(u32p), C.c_uint32(6), C.c_uint32(0), C.c_int32(5),
                                         C.byref(ok)) == 2                     # unknown node hash

    G = load_qwen_golden()
    cfg, weights, x = rand_layer(1, d_model=64, d_ff=96, heads=2, kv=2, d_head=16, v_heads=4, v_d_head=16)
    layer = zq.QwenLayer(ctx, cfg, weights, ctx.upload(G["silu"]), ctx.upload(G["sigmoid"]))
    ih = hashlib.sha256(b"e").digest()
    with pytest.raises(zk.ZkbError) as e:
        layer.verify(0, ih, bytes(100))                                          # no forward pass yet
    assert e.value.code == 2
    y = layer.forward(x)
    with pytest.raises(zk.ZkbError) as e:
        layer.verify(0, ih, bytes(100), y)                                       # a hundred zero bytes are not a proof
    assert e.value.code == 2
    with pytest.raises(zk.ZkbError):
        layer.verify_end()                                                       # nothing was begun
    proof = layer.prove(0, ih)
    assert layer.verify(0, ih, proof, y) is True                                 # and the layer is still usable
    layer.close()
