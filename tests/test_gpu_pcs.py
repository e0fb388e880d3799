"""GPU parity of the Merkle tree and the Basefold commitment against the CPU oracle: roots,
layers, codewords and whole proofs are compared bit for bit, for both node hashes."""
import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import pcs as zp
from oracle import pyoracle as O
from tests.util import P

pytestmark = pytest.mark.gpu
KINDS = [zp.NODE_BLAKE3, zp.NODE_AES_MMO]


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def rnd(seed, n):
    return np.random.default_rng(seed).integers(0, P, n, dtype=np.int64).astype(np.uint32)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("n", [1, 2, 3, 5, 64, 1000, 1024, 1025, 2048, 5000, 1 << 16, (1 << 20) + 7])
def test_merkle_root_and_layers(ctx, kind, n):
    v = rnd(n, n)
    assert zp.merkle_root(ctx, v, kind) == O.merkle_root(v, kind)
    if n <= 5000:
        assert zp.merkle_layers(ctx, v, kind) == O.merkle_layers(v, kind)


@pytest.mark.parametrize("kind", KINDS)
def test_merkle_batch_open_bytes(ctx, kind):
    v = rnd(7, 3000)
    for idx in ([3, 3, 2, 2999, 4095, 2048, 0, 1], [17], list(range(40)), [4095, 0]):
        assert zp.merkle_batch_open(ctx, v, idx, kind) == O.merkle_batch_open(v, kind, idx)
    v2 = rnd(8, 2)
    assert zp.merkle_batch_open(ctx, v2, [1, 0, 1], kind) == O.merkle_batch_open(v2, kind, [1, 0, 1])


@pytest.mark.parametrize("log_n", [1, 2, 5, 11, 14])
def test_basefold_tables(ctx, log_n):
    t, w = zp.basefold_tables(ctx, log_n)
    to, wo = O.basefold_tables(log_n)
    assert t.tolist() == to.tolist() and w.tolist() == wo.tolist()


@pytest.mark.parametrize("n", [1, 2, 3, 100, 4096, 5000, 1 << 13, 1 << 16, (1 << 18) - 5, 1 << 19])
def test_basefold_encode(ctx, n):
    c = rnd(100 + n, n)
    log_n = 1 if n <= 1 else (n - 1).bit_length()
    padded = np.zeros(1 << log_n, np.uint32)
    padded[:n] = c
    assert np.array_equal(zp.basefold_encode(ctx, c), O.basefold_encode(padded, log_n))


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("n", [1, 2, 5, 64, 300, 1024, 3000, 1 << 14])
def test_basefold_commit_and_prove_bytes(ctx, kind, n):
    c = rnd(200 + n, n)
    log_n = 1 if n <= 1 else (n - 1).bit_length()
    pt = rnd(300 + n, log_n)
    tg = zk.Transcript(ctx, b"bf-parity")
    to = O.Transcript(b"bf-parity")
    assert zp.basefold_commit_and_prove(ctx, tg, c, pt, kind) == O.basefold_commit_and_prove(to, c, pt, kind)
    assert tg.squeeze() == to.squeeze()          # transcripts left in the same state


@pytest.mark.parametrize("kind", KINDS)
def test_basefold_in_order_and_run_ahead_schedules_agree(ctx, kind):
    """The opening normally runs its folds and trees ahead of the transcript chain on a second stream;
    with ZKB_OPT_BASEFOLD_IN_ORDER everything stays on one stream.  Same bytes, same transcript state,
    also when openings follow one another on the same context (buffers reused)."""
    n = (1 << 17) - 3
    c, pt = rnd(41, n), rnd(42, 17)
    exp = O.basefold_commit_and_prove(O.Transcript(b"bf-sched"), c, pt, kind)
    for in_order in (0, 1, 0):
        ctx.set_option(ctx.OPT_BASEFOLD_IN_ORDER, in_order)
        tg = zk.Transcript(ctx, b"bf-sched")
        try:
            assert zp.basefold_commit_and_prove(ctx, tg, c, pt, kind) == exp
        finally:
            ctx.set_option(ctx.OPT_BASEFOLD_IN_ORDER, 0)


def _verify_both(ctx, blob, point, claimed, kind, label=b"bf-verify"):
    """(GPU decision, oracle decision); undecodable bytes are -1 on both sides."""
    to = O.Transcript(label)
    to.absorb_bytes(blob[:16])
    exp = O.basefold_verify_bytes(to, blob, point, claimed, kind)
    tg = zk.Transcript(ctx, label)
    tg.absorb_bytes(blob[:16])
    try:
        got = int(zp.basefold_verify_opening(ctx, tg, blob, point, claimed, kind))
    except zk.ZkbError as e:
        assert e.code == 2
        got = -1
    return got, exp, tg, to


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("n", [2, 5, 300, 1 << 14, (1 << 17) - 3])
def test_basefold_verifier_accepts_what_the_prover_emits(ctx, kind, n):
    """verify_opening on the GPU (basefold.rs:611-748) accepts the prover's proofs, leaves the transcript
    where the prover's is, and agrees with the oracle's verifier; wrong claims and points are rejected."""
    c = rnd(500 + n, n)
    log_n = 1 if n <= 1 else (n - 1).bit_length()
    pt = rnd(600 + n, log_n)
    tp = zk.Transcript(ctx, b"bf-verify")
    blob = zp.basefold_commit_and_prove(ctx, tp, c, pt, kind)
    padded = np.zeros(1 << log_n, np.uint32)
    padded[:n] = c
    claimed = O.mle_evaluate(padded, pt)
    assert int.from_bytes(blob[-12:-8], "little") == claimed
    got, exp, tg, to = _verify_both(ctx, blob, pt, claimed, kind)
    assert (got, exp) == (1, 1)
    assert tg.squeeze() == tp.squeeze() == to.squeeze()
    assert _verify_both(ctx, blob, pt, (claimed + 1) % P, kind)[:2] == (0, 0)
    # another point: rejected through the fold relation, except for coordinate 0, which the relation cannot see
    # (round 0 folds the two identical halves of [c || c], so l - r = 0 there) - the oracle says the same
    pt2 = pt.copy()
    pt2[log_n // 2] = (int(pt2[log_n // 2]) + 1) % P
    got, exp = _verify_both(ctx, blob, pt2, claimed, kind)[:2]
    assert got == exp == (0 if log_n // 2 >= 1 else 1)
    # a proof made with the other node hash does not verify
    assert _verify_both(ctx, blob, pt, claimed, 1 - kind)[:2] == (0, 0)


@pytest.mark.parametrize("kind", KINDS)
def test_basefold_verifier_rejects_tampered_proofs_like_the_oracle(ctx, kind):
    """Every single-byte change of a proof is decided as the oracle's restatement of the reference
    verifier decides it: changed roots, opened values, sibling digests, indices, lengths, final value."""
    n, log_n = 3000, 12
    c, pt = rnd(71, n), rnd(72, log_n)
    blob = zp.basefold_commit_and_prove(ctx, zk.Transcript(ctx, b"bf-verify"), c, pt, kind)
    claimed = int.from_bytes(blob[-12:-8], "little")
    assert _verify_both(ctx, blob, pt, claimed, kind)[:2] == (1, 1)
    rng = np.random.default_rng(5)
    spots = [0, 15, 16, 24, 32, 40, 41, 60, len(blob) - 1, len(blob) - 9, len(blob) - 12]
    spots += [int(v) for v in rng.integers(0, len(blob), 120)]
    seen = set()
    for pos in spots:
        bad = bytearray(blob)
        bad[pos] ^= 1 << int(rng.integers(0, 8))
        bad = bytes(bad)
        got, exp, _, _ = _verify_both(ctx, bad, pt, claimed, kind)
        assert got == exp, f"byte {pos}: GPU {got}, oracle {exp}"
        seen.add(exp)
    assert 0 in seen and -1 in seen            # both rejected and undecodable cases were met
    # dropping the last fold round: rejected, not an error
    assert _verify_both(ctx, blob[:-1], pt, claimed, kind)[:2] == (-1, -1)


def test_basefold_verifier_short_point(ctx):
    c, pt = rnd(5, 700), rnd(6, 4)
    tp = zk.Transcript(ctx, b"bf-verify")
    blob = zp.basefold_commit_and_prove(ctx, tp, c, pt)
    claimed = int.from_bytes(blob[-12:-8], "little")
    got, exp, tg, to = _verify_both(ctx, blob, pt, claimed, O.NODE_BLAKE3)
    assert (got, exp) == (1, 1) and tg.squeeze() == tp.squeeze()


def test_basefold_short_point_squeezes_challenges(ctx):
    c = rnd(5, 700)
    pt = rnd(6, 4)
    tg = zk.Transcript(ctx, b"bf-short")
    to = O.Transcript(b"bf-short")
    assert zp.basefold_commit_and_prove(ctx, tg, c, pt) == O.basefold_commit_and_prove(to, c, pt, O.NODE_BLAKE3)
    assert tg.squeeze() == to.squeeze()


def test_basefold_large_final_value_is_mle_evaluation(ctx):
    # size-independent property at 2^22 coefficients: the proof's final value is the multilinear
    # evaluation, which for a point of zeros and ones is a single coefficient
    n = 1 << 22
    c = rnd(9, n)
    log_n = 22
    bits = [1, 0, 1, 1, 0, 0, 1, 0, 1, 1, 1, 0, 0, 1, 0, 1, 0, 0, 1, 1, 0, 1]
    idx = int("".join(map(str, bits)), 2)
    tg = zk.Transcript(ctx, b"bf-large")
    blob = zp.basefold_commit_and_prove(ctx, tg, c, np.array(bits, np.uint32))
    assert int.from_bytes(blob[16:24], "little") == n and int.from_bytes(blob[24:32], "little") == log_n
    final_value = int.from_bytes(blob[-12:-8], "little")
    assert final_value == int(c[idx])
    assert blob[-8:] == bytes(8)
    # commitment root = Merkle root of the codeword
    cw = zp.basefold_encode(ctx, c)
    assert blob[:16] == zp.merkle_root(ctx, cw)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("m,n", [(4, 4), (5, 7), (33, 100), (128, 64)])
def test_matmul_binding_modes_bytes(ctx, kind, mode, m, n):
    from zklm_compile_b200 import protocols as zpr
    rng = np.random.default_rng(m * 1000 + n)
    w = rng.integers(0, P, m * n, dtype=np.int64).astype(np.uint32)
    x = rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)
    y = O.matmul_forward(w, x, m, n)
    tg = zk.Transcript(ctx, b"mm-bind")
    to = O.Transcript(b"mm-bind")
    got = zpr.prove_matmul_succinct_ef(w, x, y, m, n, tg, bind_mode=mode, node_hash=kind)
    with O.features(mode, kind):
        assert got == O.prove_matmul_succinct(to, w, x, y, m, n, ef=True)
    assert tg.squeeze() == to.squeeze()


@pytest.mark.parametrize("mode,kind", [(1, 0), (2, 0), (2, 1)])
def test_qwen_layer_with_basefold_binding_bytes(ctx, mode, kind):
    import hashlib
    from zklm_compile_b200 import qwen as zq
    from tests.util import load_qwen_golden, rand_layer
    G = load_qwen_golden()
    cfg, weights, x = rand_layer(31, d_model=64, d_ff=96, heads=2, kv=2, d_head=16, v_heads=4, v_d_head=16)
    ih = hashlib.sha256(b"model-input").digest()
    layer = zq.QwenLayer(ctx, cfg, weights, ctx.upload(G["silu"]), ctx.upload(G["sigmoid"]))
    layer.set_binding(mode, kind)
    y = layer.forward(x)
    with O.features(mode, kind):
        ey, eproof, ok = O.qwen_layer_prove(cfg, weights, x, G["silu"], G["sigmoid"], 3, ih, verify=True)
    assert ok and y.tolist() == ey.tolist()
    proof = layer.prove(3, ih)
    assert len(proof) == len(eproof) and proof == eproof
    assert layer.prove(3, ih) == eproof
    layer.close()


def test_qwen_model_shared_contexts_prove_in_waves_pcs_full():
    """Five layers on two contexts (layer i uses context i mod 2), pcs-full binding: the layers are
    proved in waves of two, the Basefold scratch of one matmul is reused by the next, and every
    proof equals the oracle's; afterwards the arenas can be given back."""
    from zklm_compile_b200 import qwen as zq
    from tests.util import load_qwen_golden, rand_layer
    G = load_qwen_golden()
    shapes = [dict(d_model=64, d_ff=96, heads=2, kv=2, d_head=16, v_heads=4, v_d_head=16), dict(d_model=64, d_ff=96, heads=4, kv=2, d_head=16)]
    layers = [rand_layer(50 + i, **shapes[i % 2]) for i in range(5)]
    x = layers[0][2]
    model = zq.QwenModel(0, [l[0] for l in layers], [l[1] for l in layers], G["silu"], G["sigmoid"], first_layer=7, n_contexts=2)
    assert len(model._own_ctxs) == 2 and model.ctxs[0] is model.ctxs[2] is model.ctxs[4]
    for l in model.layers:
        l.set_binding(2, 0)
        l.use_graph(False)
    ih = zq.hash_values(x)
    cur, exp = x, []
    with O.features(2, 0):
        for i, (cfg, w, _) in enumerate(layers):
            cur, pr, ok = O.qwen_layer_prove(cfg, w, cur, G["silu"], G["sigmoid"], 7 + i, ih, verify=True)
            assert ok
            exp.append(pr)
    for _ in range(2):
        assert model.forward_and_prove(x) == exp[::-1]
    assert model.output().tolist() == cur.tolist()
    assert all(c.scratch_bytes > 0 for c in model._own_ctxs)
    for c in model._own_ctxs:
        c.trim()
        assert c.scratch_bytes == 0
    assert model.forward_and_prove(x) == exp[::-1]      # the arena grows again
    model.close()
