"""Row attention at seq_len >= 2 on the GPU against the CPU restatement: the proof bytes, the transcript state
afterwards, the op's output, ragged shapes, both table sizes, device-resident inputs, and the reference's
two panics as error codes."""
import hashlib

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import attention as za, tables
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def small_exp_table(scale=100):
    x = np.arange(256, dtype=np.uint8).astype(np.int8).astype(np.float64) / scale
    return tables.i16_to_field(tables.quantize_i16(np.exp(x), float(scale)))


def qkv(rng, nh, s, d, lo=-3, hi=4):
    """Small signed entries: scores stay inside the table and reach its negative half; V is any field value."""
    n = nh * s * d
    q = np.mod(rng.integers(lo, hi, n), P).astype(np.uint32)
    k = np.mod(rng.integers(lo, hi, n), P).astype(np.uint32)
    v = rng.integers(0, P, n).astype(np.uint32)
    return q, k, v


def both(ctx, q, k, v, nh, s, d, t, label=b"attn"):
    tg = zk.Transcript(ctx, label)
    got, out = za.prove_row_attention(q, k, v, nh, s, d, t, tg, want_output=True)
    to = O.Transcript(label)
    exp, st = O.prove_row_attention(to, q, k, v, nh, s, d, t)
    assert st == 0
    return got, out, tg.squeeze(), exp, to.squeeze()


@pytest.mark.parametrize("nh,s,d", [(2, 4, 4), (4, 16, 8), (1, 64, 16), (3, 5, 3), (2, 2, 1), (1, 33, 7), (2, 128, 64), (1, 3, 200)])
def test_proof_bytes_equal_the_oracle(ctx, nh, s, d):
    rng = np.random.default_rng(nh * 1000 + s * 10 + d)
    t = tables.build_exp_table(100)
    hi = 4 if d <= 16 else 2                                  # |score| <= d * 9 (or d) stays far inside i16
    q, k, v = qkv(rng, nh, s, d, -hi + 1, hi)
    got, out, sg, exp, so = both(ctx, q, k, v, nh, s, d, t)
    assert len(got) == len(exp)
    assert hashlib.sha256(got).digest() == hashlib.sha256(exp).digest()
    assert sg == so
    fwd, st = O.row_attention_forward(q, k, v, nh, s, d, t)
    assert st == 0 and np.array_equal(out, fwd)
    assert np.array_equal(za.row_attention_forward(ctx, q, k, v, nh, s, d, t), fwd)


def test_forward_against_the_reference_python_restatement(ctx):
    """tests/golden/attention_forward.json: outputs of the reference's own attention_full (tests/reference/attention.py)."""
    import json, os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "attention_forward.json")))
    for c in g["cases"]:
        q, k, v = (np.array(c[x], np.uint32) for x in "qkv")
        nh, s, d = c["num_heads"], c["seq_len"], c["d_head"]
        t = tables.build_exp_table(c["exp_scale"])
        assert za.row_attention_forward(ctx, q, k, v, nh, s, d, t).tolist() == c["out"]
        proof, out = za.prove_row_attention(q, k, v, nh, s, d, t, zk.Transcript(ctx, b"g"), want_output=True)
        assert out.tolist() == c["out"]
        for r in range(nh * s):                                  # the rows' outputs inside the proof are those values
            assert np.array(c["out"][r * d:(r + 1) * d], "<u4").tobytes() in proof


def test_the_reference_test_inputs_with_the_256_entry_table(ctx):
    """attention.rs:632-671: q = i % 3 + 1, k = i % 2 + 1, v = i % 4 + 1 on (2, 4, 4)."""
    t = small_exp_table()
    i = np.arange(2 * 4 * 4)
    q, k, v = ((i % 3) + 1).astype(np.uint32), ((i % 2) + 1).astype(np.uint32), ((i % 4) + 1).astype(np.uint32)
    got, out, sg, exp, so = both(ctx, q, k, v, 2, 4, 4, t, b"row-attn-test")
    assert got == exp and sg == so


def test_repeated_scores_give_one_active_entry(ctx):
    """All scores equal: one active table entry with multiplicity seq_len."""
    t = tables.build_exp_table(100)
    nh, s, d = 1, 16, 4
    q = np.ones(nh * s * d, np.uint32); k = np.ones(nh * s * d, np.uint32)
    v = np.arange(nh * s * d, dtype=np.uint32)
    got, out, sg, exp, so = both(ctx, q, k, v, nh, s, d, t)
    assert got == exp and sg == so


def test_longest_supported_row(ctx):
    rng = np.random.default_rng(9)
    t = tables.build_exp_table(100)
    nh, s, d = 1, 1024, 8
    q, k, v = qkv(rng, nh, s, d)
    # two rows only would not exercise less: every row has 1024 lookups; keep the oracle's work bounded by one head
    got, out, sg, exp, so = both(ctx, q, k, v, nh, s, d, t)
    assert hashlib.sha256(got).digest() == hashlib.sha256(exp).digest() and sg == so


def test_threads_per_row_and_stream_order_do_not_change_the_bytes(ctx):
    rng = np.random.default_rng(6)
    t = tables.build_exp_table(100)
    nh, s, d = 3, 40, 24
    q, k, v = qkv(rng, nh, s, d, -1, 2)
    exp, st = O.prove_row_attention(O.Transcript(b"opt"), q, k, v, nh, s, d, t)
    try:
        for threads, in_order in [(64, 0), (128, 0), (256, 0), (0, 1)]:
            ctx.set_option(zk.Context.OPT_ATTENTION_THREADS, threads)
            ctx.set_option(zk.Context.OPT_BASEFOLD_IN_ORDER, in_order)
            assert za.prove_row_attention(q, k, v, nh, s, d, t, zk.Transcript(ctx, b"opt")) == exp, (threads, in_order)
        with pytest.raises(zk.ZkbError):
            ctx.set_option(zk.Context.OPT_ATTENTION_THREADS, 96)
    finally:
        ctx.set_option(zk.Context.OPT_ATTENTION_THREADS, 0)
        ctx.set_option(zk.Context.OPT_BASEFOLD_IN_ORDER, 0)


def test_device_resident_inputs(ctx):
    rng = np.random.default_rng(4)
    t = tables.build_exp_table(100)
    nh, s, d = 2, 8, 4
    q, k, v = qkv(rng, nh, s, d)
    dq, dk, dv, dt = (ctx.upload(a) for a in (q, k, v, t))
    tg = zk.Transcript(ctx, b"dev")
    got, out = za.prove_row_attention(dq, dk, dv, nh, s, d, dt, tg, want_output=True)
    exp, st = O.prove_row_attention(O.Transcript(b"dev"), q, k, v, nh, s, d, t)
    assert got == exp
    assert np.array_equal(out.download().reshape(-1), O.row_attention_forward(q, k, v, nh, s, d, t)[0])
    assert np.array_equal(za.row_attention_forward(ctx, dq, dk, dv, nh, s, d, dt).download().reshape(-1), out.download().reshape(-1))


def test_errors(ctx):
    t = small_exp_table()
    q = np.full(8, 20, np.uint32); k = np.full(8, 20, np.uint32); v = np.ones(8, np.uint32)
    with pytest.raises(zk.ZkbError, match="not an input of the exp table"):
        za.row_attention_forward(ctx, q, k, v, 1, 2, 4, t)
    with pytest.raises(zk.ZkbError, match="not an input of the exp table"):
        za.prove_row_attention(q, k, v, 1, 2, 4, t, zk.Transcript(ctx, b"e"))
    zero = np.zeros(256, np.uint32)                           # a table whose outputs are all zero: sum e = 0
    with pytest.raises(zk.ZkbError, match="denominator is zero"):
        za.row_attention_forward(ctx, np.ones(8, np.uint32), np.ones(8, np.uint32), v, 1, 2, 4, zero)
    with pytest.raises(zk.ZkbError):
        za.prove_row_attention(q[:4], k[:4], v[:4], 1, 1, 4, t, zk.Transcript(ctx, b"e"))      # seq_len = 1
    with pytest.raises(zk.ZkbError):
        za.row_attention_forward(ctx, q, k, v, 1, 2, 4, t[:100])                               # not a table size
    with pytest.raises(zk.ZkbError, match="1024"):
        za.row_attention_forward(ctx, np.ones(2050, np.uint32), np.ones(2050, np.uint32), np.ones(2050, np.uint32), 1, 1025, 2, t)
    # the context is still usable
    got, out, sg, exp, so = both(ctx, *qkv(np.random.default_rng(1), 1, 4, 4), 1, 4, 4, tables.build_exp_table(100))
    assert got == exp


# ---- the op-list driver with an attention op at seq_len >= 2 (pipeline/prove.rs:419-432) -----------------------
def _small_linear(rng, m, n, nnz=2):
    """Rows with `nnz` entries of +-1: with inputs in {0, 1} every output stays within +-nnz."""
    w = np.zeros((m, n), np.int64)
    for i in range(m):
        cols = rng.choice(n, nnz, replace=False)
        w[i, cols] = rng.choice([-1, 1], nnz)
    return np.mod(w, P).astype(np.uint32)


@pytest.mark.parametrize("external_kv", [False, True])
def test_oplist_with_row_attention(ctx, external_kv):
    from zklm_compile_b200 import oplist as zo
    rng = np.random.default_rng(21)
    nh, s, d, d_in, d_out = 2, 8, 4, 24, 10
    total = nh * s * d
    t = tables.build_exp_table(100)
    dt = ctx.upload(t)
    x = rng.integers(0, 2, d_in).astype(np.uint32)
    m1 = total if external_kv else 3 * total
    w1 = _small_linear(rng, m1, d_in)
    b1 = np.mod(rng.integers(-1, 2, m1), P).astype(np.uint32)
    w2 = rng.integers(0, P, (d_out, total)).astype(np.uint32)
    kv = (np.mod(rng.integers(-3, 4, total), P).astype(np.uint32), rng.integers(0, P, total).astype(np.uint32)) if external_kv else (None, None)
    g = zo.OpList(ctx, d_in); o = O.OpList()
    g.linear("c_attn", w1, b1, m1, d_in); o.linear("c_attn", w1, b1, m1, d_in)
    g.save("save_res", "res"); o.simple("save", "save_res", "res")
    g.attention("attn", nh, s, d, dt, *kv); o.attention("attn", nh, s, d, t, *kv)
    g.linear("c_proj", w2, None, d_out, total); o.linear("c_proj", w2, None, d_out, total)
    g.forward(x)
    assert np.array_equal(g.activation(2), o.forward(x, 2))
    assert np.array_equal(g.activation(), o.forward(x))
    got, exp = g.prove(x), o.prove(x)
    assert got == exp
    assert g.prove(x) == exp                                  # a second proof on the same list (staging and scratch reused)
    if external_kv:                                           # the next request brings other K and V
        kv2 = (np.mod(rng.integers(-3, 4, total), P).astype(np.uint32), rng.integers(0, P, total).astype(np.uint32))
        g.set_attention_kv(2, *kv2)
        o2 = O.OpList()
        o2.linear("c_attn", w1, b1, m1, d_in); o2.simple("save", "save_res", "res"); o2.attention("attn", nh, s, d, t, *kv2)
        o2.linear("c_proj", w2, None, d_out, total)
        assert g.prove(x) == o2.prove(x)
    else:
        with pytest.raises(zk.ZkbError):
            g.set_attention_kv(2, np.zeros(total, np.uint32), np.zeros(total, np.uint32))
    g.close()


def test_oplist_attention_length_checks(ctx):
    from zklm_compile_b200 import oplist as zo
    dt = ctx.upload(tables.build_exp_table(100))
    g = zo.OpList(ctx, 50)
    with pytest.raises(zk.ZkbError, match="Q . K . V"):
        g.attention("a", 2, 4, 2, dt)                          # 50 != 3 * 16
    with pytest.raises(zk.ZkbError):
        g.attention("a", 2, 1, 2, dt)                          # seq_len = 1 is the other op
    with pytest.raises(zk.ZkbError, match="Q . K . V"):
        g.attention("a", 2, 8, 4, dt, np.zeros(64, np.uint32), np.zeros(64, np.uint32))   # 50 < 64 words of Q
    g.attention("a", 2, 4, 2, dt, np.ones(16, np.uint32), np.ones(16, np.uint32))           # Q = the first 16 words
    g.close()


# ---- grouped-query attention (attention.rs:386-500) -------------------------------------------------------------
@pytest.mark.parametrize("nq,nkv,s,d", [(4, 2, 4, 4), (4, 1, 8, 4), (2, 2, 5, 3), (12, 4, 64, 16)])
def test_gqa_proof_bytes_equal_the_oracle(ctx, nq, nkv, s, d):
    rng = np.random.default_rng(nq * 100 + nkv * 10 + s)
    t = tables.build_exp_table(100)
    q = np.mod(rng.integers(-2, 3, nq * s * d), P).astype(np.uint32)
    k = np.mod(rng.integers(-2, 3, nkv * s * d), P).astype(np.uint32)
    v = rng.integers(0, P, nkv * s * d).astype(np.uint32)
    tg = zk.Transcript(ctx, b"gqa")
    got, out = za.prove_row_attention_gqa(q, k, v, nq, nkv, s, d, t, tg, want_output=True)
    to = O.Transcript(b"gqa")
    exp, st = O.prove_row_attention(to, q, k, v, nq, s, d, t, nkv)
    assert st == 0 and got == exp and tg.squeeze() == to.squeeze()
    fwd, st = O.row_attention_forward(q, k, v, nq, s, d, t, nkv)
    assert np.array_equal(out, fwd)
    assert np.array_equal(za.row_attention_forward(ctx, q, k, v, nq, s, d, t, nkv), fwd)


def test_gqa_head_counts_must_divide(ctx):
    t = tables.build_exp_table(100)
    with pytest.raises(zk.ZkbError, match="divisible"):
        za.row_attention_forward(ctx, np.ones(3 * 8, np.uint32), np.ones(2 * 8, np.uint32), np.ones(2 * 8, np.uint32), 3, 2, 4, t, 2)


def test_oplist_with_gqa_attention(ctx):
    from zklm_compile_b200 import oplist as zo
    rng = np.random.default_rng(23)
    nq, nkv, s, d, d_in = 4, 2, 4, 4, 20
    tq, tkv = nq * s * d, nkv * s * d
    t = tables.build_exp_table(100)
    dt = ctx.upload(t)
    x = rng.integers(0, 2, d_in).astype(np.uint32)
    m1 = tq + 2 * tkv
    w1 = _small_linear(rng, m1, d_in)
    w2 = rng.integers(0, P, (7, tq)).astype(np.uint32)
    g = zo.OpList(ctx, d_in); o = O.OpList()
    g.linear("qkv", w1, None, m1, d_in); o.linear("qkv", w1, None, m1, d_in)
    g.attention("gqa", nq, s, d, dt, num_kv_heads=nkv); o.attention("gqa", nq, s, d, t, num_kv_heads=nkv)
    g.linear("o_proj", w2, None, 7, tq); o.linear("o_proj", w2, None, 7, tq)
    assert g.prove(x) == o.prove(x)
    g.close()


# ---- the verifier (attention.rs:279-385, 503-590) -----------------------------------------------------------------
def _decision(ctx, blob, k, v, nh, s, d, nkv, label):
    try:
        return int(za.verify_row_attention(blob, k, v, nh, s, d, zk.Transcript(ctx, label), nkv))
    except zk.ZkbError as e:
        assert e.code == 2
        return -1


@pytest.mark.parametrize("nh,nkv,s,d,n_table", [(2, 0, 6, 4, 65536), (4, 2, 5, 3, 65536), (1, 0, 16, 8, 256)])
def test_verifier_decides_like_the_restated_one(ctx, nh, nkv, s, d, n_table):
    rng = np.random.default_rng(nh + s + d)
    t = tables.build_exp_table(100) if n_table == 65536 else small_exp_table()
    kvh = nkv or nh
    q = np.mod(rng.integers(-2, 3, nh * s * d), P).astype(np.uint32)
    k = np.mod(rng.integers(-2, 3, kvh * s * d), P).astype(np.uint32)
    v = rng.integers(0, P, kvh * s * d).astype(np.uint32)
    proof = za.prove_row_attention(q, k, v, nh, s, d, t, zk.Transcript(ctx, b"av"), num_kv_heads=nkv)
    tg, to = zk.Transcript(ctx, b"av"), O.Transcript(b"av")
    assert za.verify_row_attention(proof, k, v, nh, s, d, tg, nkv) is True
    assert O.row_attention_verify_bytes(to, proof, k, v, nh, s, d, nkv) == 1
    assert tg.squeeze() == to.squeeze()
    # other K / V, other head grouping, other dimensions: rejected by both
    k2 = k.copy(); k2[3] = (int(k2[3]) + 1) % P
    v2 = v.copy(); v2[-1] ^= 1
    for kk, vv in ((k2, v), (k, v2)):
        assert _decision(ctx, proof, kk, vv, nh, s, d, nkv, b"av") == O.row_attention_verify_bytes(O.Transcript(b"av"), proof, kk, vv, nh, s, d, nkv) == 0
    assert _decision(ctx, proof, k, v, nh, s, d, nkv, b"av2") == 1        # rows have transcripts of their own: the caller's label does not enter them
    # one low bit changed, all over the proof: the two verifiers agree on every position
    n_rej = n_acc = 0
    for at in range(0, len(proof), 7):
        bad = bytearray(proof)
        bad[at] ^= 1
        exp = O.row_attention_verify_bytes(O.Transcript(b"av"), bytes(bad), k, v, nh, s, d, nkv)
        got = _decision(ctx, bytes(bad), k, v, nh, s, d, nkv, b"av")
        assert got == exp, (at, got, exp)
        n_rej += exp == 0
        n_acc += exp == 1
    assert n_rej > 300 and n_acc > 10       # accepted: fields the reference's verifier does not read (challenges of the plain sumchecks, y_values, ...)


def test_verifier_at_the_bench_shape(ctx):
    rng = np.random.default_rng(12)
    t = tables.build_exp_table(100)
    nh, s, d = 12, 128, 64
    n = nh * s * d
    q = np.mod(rng.integers(-1, 2, n), P).astype(np.uint32); k = np.mod(rng.integers(-1, 2, n), P).astype(np.uint32)
    v = rng.integers(0, P, n).astype(np.uint32)
    proof = za.prove_row_attention(q, k, v, nh, s, d, t, zk.Transcript(ctx, b"big"))
    dk, dv = ctx.upload(k), ctx.upload(v)
    assert za.verify_row_attention(proof, dk, dv, nh, s, d, zk.Transcript(ctx, b"big")) is True
    bad = bytearray(proof)
    bad[len(bad) // 2] ^= 1
    assert _decision(ctx, bytes(bad), dk, dv, nh, s, d, 0, b"big") == O.row_attention_verify_bytes(O.Transcript(b"big"), bytes(bad), k, v, nh, s, d)


def test_caller_keeps_its_transcript(ctx):
    """tr = NULL: only the rows are proved / checked; the proof is the same bytes, and a caller that absorbs the dimensions and the
    rows' scores and outputs itself ends in the state the library's transcript ends in."""
    rng = np.random.default_rng(17)
    t = tables.build_exp_table(100)
    for nh, nkv, s, d in [(3, 0, 9, 5), (4, 2, 6, 4)]:
        kvh = nkv or nh
        q = np.mod(rng.integers(-2, 3, nh * s * d), P).astype(np.uint32)
        k = np.mod(rng.integers(-2, 3, kvh * s * d), P).astype(np.uint32)
        v = rng.integers(0, P, kvh * s * d).astype(np.uint32)
        tg = zk.Transcript(ctx, b"own")
        full = za.prove_row_attention(q, k, v, nh, s, d, t, tg, num_kv_heads=nkv)
        rows_only, out = za.prove_row_attention(q, k, v, nh, s, d, t, ctx, want_output=True, num_kv_heads=nkv)
        assert rows_only == full
        assert np.array_equal(out, O.row_attention_forward(q, k, v, nh, s, d, t, nkv)[0])
        mine = zk.Transcript(ctx, b"own")
        mine.absorb_bytes(za.caller_transcript_stream(rows_only, nh, s, d, nkv))
        assert mine.squeeze() == tg.squeeze()
        assert za.verify_row_attention(full, k, v, nh, s, d, ctx, nkv) is True
        bad = bytearray(full)
        bad[len(bad) // 3] ^= 1
        exp = O.row_attention_verify_bytes(O.Transcript(b"own"), bytes(bad), k, v, nh, s, d, nkv)
        try:
            got = int(za.verify_row_attention(bytes(bad), k, v, nh, s, d, ctx, nkv))
        except zk.ZkbError:
            got = -1
        assert got == exp
