"""Batch Basefold on the GPU against the CPU restatement: bincode bytes and the transcript state afterwards, on the reference's
own test polynomials (basefold.rs:1849-1960), ragged multi-height batches, both node hashes, device-resident polynomials, the
in-order schedule, repeated proofs from one precommit, and argument errors."""
import struct

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import pcs
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def both(ctx, polys, log_ns, individual=False, kind=0, label=b"batch"):
    b = pcs.BasefoldBatch(ctx, polys, log_ns, kind)
    tg = zk.Transcript(ctx, label)
    got = b.prove(tg, individual)
    to = O.Transcript(label)
    exp = O.basefold_batch_prove(to, polys, log_ns, individual, kind)
    return b, got, exp, tg.squeeze(), to.squeeze()


@pytest.mark.parametrize("kind", [0, 1])
def test_same_size_batch_is_batch_commit_and_prove(ctx, kind):
    polys = [np.array([((i + seed * 100) * 17 + 3) % P for i in range(256)], dtype=np.uint32) for seed in range(4)]
    b, got, exp, sg, so = both(ctx, polys, [8] * 4, True, kind, b"batch-basefold-test")
    assert got == exp and sg == so
    root, n, ln = b.commitment(2)
    assert (n, ln) == (256, 8) and root == exp[8 + 64:8 + 80]
    b.close()


@pytest.mark.parametrize("kind", [0, 1])
def test_multi_height_batch(ctx, kind):
    p1 = np.array([(i * 17 + 3) % P for i in range(256)], np.uint32)
    p2 = np.array([(i * 31 + 7) % P for i in range(64)], np.uint32)
    p3 = np.array([(i * 43 + 11) % P for i in range(16)], np.uint32)
    b, got, exp, sg, so = both(ctx, [p1, p2, p3], [8, 6, 4], False, kind, b"multi-height-test")
    assert got == exp and sg == so
    # a second proof from the same precommit, on another transcript
    tg = zk.Transcript(ctx, b"again")
    assert b.prove(tg) == O.basefold_batch_prove(O.Transcript(b"again"), [p1, p2, p3], [8, 6, 4], False, kind)
    b.close()


@pytest.mark.parametrize("sizes,log_ns", [((16, 200, 64, 256, 50, 9), (4, 8, 6, 8, 6, 4)), ((3, 1, 2), (2, 1, 1)), ((5000, 4096, 100, 100, 7), (13, 12, 7, 7, 3)),
                                          ((1 << 15, 1 << 14, 1 << 15), (15, 14, 15)), ((70000,), (17,))])
def test_ragged_batches(ctx, sizes, log_ns):
    rng = np.random.default_rng(sum(sizes))
    polys = [rng.integers(0, P, n).astype(np.uint32) for n in sizes]
    b, got, exp, sg, so = both(ctx, polys, list(log_ns))
    assert len(got) == len(exp) and got == exp and sg == so
    assert b.device_bytes > 0
    b.close()


def test_device_resident_polynomials_and_in_order_schedule(ctx):
    rng = np.random.default_rng(8)
    sizes, log_ns = (3000, 1000, 1024), [12, 10, 10]
    polys = [rng.integers(0, P, n).astype(np.uint32) for n in sizes]
    dev = [ctx.upload(p) for p in polys]
    b = pcs.BasefoldBatch(ctx, dev, log_ns)
    exp = O.basefold_batch_prove(O.Transcript(b"dev"), polys, log_ns)
    assert b.prove(zk.Transcript(ctx, b"dev")) == exp
    ctx.set_option(zk.Context.OPT_BASEFOLD_IN_ORDER, 1)
    try:
        assert b.prove(zk.Transcript(ctx, b"dev")) == exp
    finally:
        ctx.set_option(zk.Context.OPT_BASEFOLD_IN_ORDER, 0)
    b.close()


def test_argument_errors(ctx):
    p = np.arange(10, dtype=np.uint32)
    with pytest.raises(zk.ZkbError):
        pcs.BasefoldBatch(ctx, [p], [3])                       # 10 coefficients do not fit 2^3
    with pytest.raises(zk.ZkbError):
        pcs.BasefoldBatch(ctx, [p], [0])
    with pytest.raises(zk.ZkbError):
        pcs.BasefoldBatch(ctx, [], [])
    with pytest.raises(zk.ZkbError):
        pcs.BasefoldBatch(ctx, [p], [4], 7)                    # unknown node hash
    b = pcs.BasefoldBatch(ctx, [p, p[:4]], [4, 2])
    with pytest.raises(zk.ZkbError, match="one size"):
        b.prove(zk.Transcript(ctx, b"x"), True)
    assert b.prove(zk.Transcript(ctx, b"x")) == O.basefold_batch_prove(O.Transcript(b"x"), [p, p[:4]], [4, 2])
    b.close()


# ---- the verifier (basefold.rs:959-1137) ------------------------------------------------------------------------
def _gpu_decision(ctx, blob, kind, label):
    try:
        return int(pcs.basefold_batch_verify_opening(ctx, zk.Transcript(ctx, label), blob, kind))
    except zk.ZkbError as e:
        assert e.code == 2
        return -1


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("case", ["multi", "same"])
def test_batch_verifier_decides_like_the_restated_one(ctx, kind, case):
    rng = np.random.default_rng(77)
    if case == "multi":
        polys = [rng.integers(0, P, n).astype(np.uint32) for n in (200, 64, 256, 50, 9)]
        log_ns, individual = [8, 6, 8, 6, 4], False
    else:
        polys = [rng.integers(0, P, 128).astype(np.uint32) for _ in range(3)]
        log_ns, individual = [7, 7, 7], True
    b = pcs.BasefoldBatch(ctx, polys, log_ns, kind)
    blob = b.prove(zk.Transcript(ctx, b"bv"), individual)
    b.close()
    tg, to = zk.Transcript(ctx, b"bv"), O.Transcript(b"bv")
    assert pcs.basefold_batch_verify_opening(ctx, tg, blob, kind) is True
    assert O.basefold_batch_verify_bytes(to, blob, kind)[0] == 1
    assert tg.squeeze() == to.squeeze()
    assert pcs.basefold_batch_verify_opening(ctx, zk.Transcript(ctx, b"other"), blob, kind) is False
    # single low-bit changes all over the proof part (the commitments in front are not read by either verifier except for the
    # individual openings' roots; their length fields are left alone): the two verifiers agree on every one
    start = 8 + 32 * len(polys)
    n_rejected = 0
    for at in list(range(start, len(blob), 61)) + list(range(8, start, 32)):
        bad = bytearray(blob)
        bad[at] ^= 1
        exp = O.basefold_batch_verify_bytes(O.Transcript(b"bv"), bytes(bad), kind)[0]
        got = _gpu_decision(ctx, bytes(bad), kind, b"bv")
        assert got == exp, (at, got, exp)
        n_rejected += exp != 1
    assert n_rejected > 100
    assert _gpu_decision(ctx, blob[:-5], kind, b"bv") == -1 and _gpu_decision(ctx, blob + b"\\0", kind, b"bv") == -1


def test_batch_verifier_at_2_17(ctx):
    rng = np.random.default_rng(3)
    polys = [rng.integers(0, P, n).astype(np.uint32) for n in (100000, 30000, 131072, 5)]
    log_ns = [17, 15, 17, 3]
    b = pcs.BasefoldBatch(ctx, polys, log_ns)
    blob = b.prove(zk.Transcript(ctx, b"big"))
    b.close()
    assert pcs.basefold_batch_verify_opening(ctx, zk.Transcript(ctx, b"big"), blob) is True
    assert O.basefold_batch_verify_bytes(O.Transcript(b"big"), blob)[0] == 1
