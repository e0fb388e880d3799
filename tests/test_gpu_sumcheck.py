"""GPU parity: device transcript and every sumcheck prover kind against the CPU oracle,
bit-exact (integer field arithmetic), through the C ABI."""
import numpy as np
import pytest

import zklm_compile_b200 as zk
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1

KIND_NAMES = {
    zk.SC_PRODUCT: "product",
    zk.SC_TRIPLE: "triple",
    zk.SC_PRODUCT_ONES: "product_ones",
    zk.SC_PRODUCT_EF: "product_ef",
    zk.SC_PRODUCT_EF_FULL: "product_ef_full",
    zk.SC_PRODUCT_EF_MIXED: "product_ef_mixed",
    zk.SC_TRIPLE_EF_FULL: "triple_ef_full",
    zk.SC_PRODUCT_ONES_EF_FULL: "product_ones_ef_full",
}


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def rand_tables(kind, nv, seed):
    rng = np.random.default_rng(seed)
    widths = O.SUMCHECKS[KIND_NAMES[kind]][1]
    n = 1 << nv
    return [rng.integers(0, P, (n, w) if w == 4 else n, dtype=np.int64).astype(np.uint32) for w in widths]


def test_transcript_matches_oracle(ctx):
    for label in (b"", b"x", b"qwen-layer-12", b"a" * 55, b"b" * 56, b"c" * 64, b"d" * 300):
        t, o = zk.Transcript(ctx, label), O.Transcript(label)
        for step in range(3):
            t.absorb(0x12345678 + step); o.absorb(0x12345678 + step)
            t.absorb_bytes(b"hello" * (step + 1)); o.absorb_bytes(b"hello" * (step + 1))
            vals = np.arange(1, 70 + 37 * step, dtype=np.uint32)
            t.absorb_many(vals); o.absorb_many(vals)
            assert t.squeeze() == o.squeeze()
            assert t.squeeze_ef().tolist() == o.squeeze_ef().tolist()
        # large absorb from a device buffer
        big = np.random.default_rng(1).integers(0, P, 5000, dtype=np.int64).astype(np.uint32)
        t.absorb_many(ctx.upload(big)); o.absorb_many(big)
        assert [t.squeeze() for _ in range(5)] == [o.squeeze() for _ in range(5)]


def test_transcript_export_import(ctx):
    t = zk.Transcript(ctx, b"exp")
    t.absorb_bytes(b"abcdefg")
    st = t.export_state()
    a = t.squeeze()
    t2 = zk.Transcript(ctx, b"other")
    t2.import_state(st)
    assert t2.squeeze() == a


@pytest.mark.parametrize("kind", sorted(KIND_NAMES))
@pytest.mark.parametrize("nv", [1, 2, 3, 7, 11, 12, 13, 15, 18])
def test_sumcheck_matches_oracle(ctx, kind, nv):
    if nv >= 18 and kind in (zk.SC_TRIPLE_EF_FULL,):
        nv = 16
    tables = rand_tables(kind, nv, 1000 * kind + nv)
    label = b"parity-%d-%d" % (kind, nv)
    tr = zk.Transcript(ctx, label)
    tr.absorb(nv)
    proof, *fin = zk.sumcheck_prove(kind, tables, nv, tr)
    otr = O.Transcript(label)
    otr.absorb(nv)
    polys, chal, ofin = O.prove(KIND_NAMES[kind], otr, tables, nv)
    assert proof.round_polys.reshape(nv, -1).tolist() == polys.tolist()
    assert proof.challenges.reshape(nv, -1).tolist() == chal.tolist()
    got = np.array([np.asarray(f, dtype=np.uint32).reshape(-1) for f in fin])
    assert got.tolist() == ofin.tolist()
    # the transcripts stay in step afterwards
    assert tr.squeeze() == otr.squeeze()


@pytest.mark.parametrize("kind", [zk.SC_PRODUCT_EF, zk.SC_PRODUCT, zk.SC_TRIPLE_EF_FULL])
def test_sumcheck_device_tables_untouched_and_verifies(ctx, kind):
    nv = 14
    tables = rand_tables(kind, nv, 77 + kind)
    dev = [ctx.upload(t) for t in tables]
    tr = zk.Transcript(ctx, b"dev")
    proof, *fin = zk.sumcheck_prove(kind, dev, nv, tr)
    for d, t in zip(dev, tables):
        assert np.array_equal(d.download().reshape(t.shape), t)
    # the oracle's restatement of the reference verifier accepts the GPU proof
    name = KIND_NAMES[kind]
    polys = proof.round_polys.reshape(nv, -1)
    first = polys[0].reshape(-1, 4 if name.endswith(("ef", "full")) else 1)
    otr = O.Transcript(b"dev")
    oracle_polys, _, _ = O.prove(name, otr, tables, nv)
    assert polys.tolist() == oracle_polys.tolist()
    finarr = np.array([np.asarray(f, dtype=np.uint32).reshape(-1) for f in fin])
    if kind == zk.SC_PRODUCT:
        claimed = (int(first[0, 0]) + int(first[1, 0])) % P
        assert O.verify(name, O.Transcript(b"dev"), claimed, polys, proof.challenges, finarr)
        assert O.verify(name, O.Transcript(b"dev"), claimed, polys, np.zeros(0, np.uint32), finarr)


def test_large_product_ef_roundtrip_property(ctx):
    """At a size the oracle does not finish quickly (2^24) check size-independent properties:
    round-0 message equals the directly computed sums, every later round satisfies
    s0 + s1 == interpolated claim, and the final evaluations close the chain."""
    nv = 24
    rng = np.random.default_rng(5)
    f = rng.integers(0, P, 1 << nv, dtype=np.int64).astype(np.uint32)
    g = rng.integers(0, P, 1 << nv, dtype=np.int64).astype(np.uint32)
    tr = zk.Transcript(ctx, b"big")
    proof, f_s, g_s = zk.prove_product_ef(f, g, nv, tr)
    half = 1 << (nv - 1)
    fo, go = f.astype(object), g.astype(object)
    s0 = int(np.sum(fo[:half] * go[:half]) % P)
    s1 = int(np.sum(fo[half:] * go[half:]) % P)
    assert proof.round_polys[0, 0].tolist() == [s0, 0, 0, 0]
    claimed = np.array([(s0 + s1) % P, 0, 0, 0], np.uint32)
    # the verifier restatement re-derives every challenge from the transcript and checks the chain
    assert O.verify("product_ef", O.Transcript(b"big"), claimed, proof.round_polys.reshape(nv, -1),
                    proof.challenges, np.array([f_s, g_s]))
    # the final values are the MLEs of f and g at the challenge point
    assert O.mle_evaluate_ef(f, proof.challenges).tolist() == f_s.tolist()
    assert O.mle_evaluate_ef(g, proof.challenges).tolist() == g_s.tolist()
