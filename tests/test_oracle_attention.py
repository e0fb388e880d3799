"""Row attention at seq_len >= 2: the CPU restatement against the reference's own tests
(rust/zk_ml_prover/src/proving/attention.rs:651-870: prove -> verify round trips on the same shapes and
inputs, tampered proofs rejected) and against an independent numpy forward pass."""
import numpy as np
import pytest

from oracle import pyoracle as po
from zklm_compile_b200 import tables

P = (1 << 31) - 1


def golden():
    import json, os
    return json.load(open(os.path.join(os.path.dirname(__file__), "golden", "attention_forward.json")))


def test_forward_and_exp_table_against_the_reference_python_restatement():
    """tests/golden/attention_forward.json was produced by the reference's own attention_full / exp_table
    (tests/reference/attention.py, reference.py; generator: tests/golden/make_golden_attention.py)."""
    import hashlib
    g = golden()
    for scale, rec in g["exp_tables"].items():
        t = tables.build_exp_table(int(scale))
        assert t.size == rec["rows"]
        assert hashlib.sha256(t.astype("<u4").tobytes()).hexdigest() == rec["sha256_outputs_le_u32"]
        assert hashlib.sha256(tables.table_inputs(65536).astype("<u4").tobytes()).hexdigest() == rec["sha256_inputs_le_u32"]
    for c in g["cases"]:
        q, k, v = (np.array(c[x], np.uint32) for x in "qkv")
        out, st = po.row_attention_forward(q, k, v, c["num_heads"], c["seq_len"], c["d_head"], tables.build_exp_table(c["exp_scale"]))
        assert st == 0 and out.tolist() == c["out"]


def small_exp_table(scale=100):
    """attention.rs:605-629: 256 entries, input raw as i8."""
    x = np.arange(256, dtype=np.uint8).astype(np.int8).astype(np.float64) / scale
    return tables.i16_to_field(tables.quantize_i16(np.exp(x), float(scale)))


def make_qkv(nh, s, d, mq=3, mk=2, mv=4):
    """attention.rs:632-649"""
    n = nh * s * d
    i = np.arange(n)
    return ((i % mq) + 1).astype(np.uint32), ((i % mk) + 1).astype(np.uint32), ((i % mv) + 1).astype(np.uint32)


def numpy_forward(q, k, v, nh, s, d, table):
    n_table = table.size
    q = q.reshape(nh, s, d).astype(object); k = k.reshape(nh, s, d).astype(object); v = v.reshape(nh, s, d).astype(object)
    out = np.zeros((nh, s, d), dtype=np.uint32)
    for h in range(nh):
        for i in range(s):
            sc = [int(sum(k[h, j, l] * q[h, i, l] for l in range(d)) % P) for j in range(s)]
            e = [int(table[x if x < n_table // 2 else x + n_table - P]) for x in sc]
            inv = pow(sum(e) % P, P - 2, P)
            y = [ei * inv % P for ei in e]
            for c in range(d):
                out[h, i, c] = sum(y[l] * int(v[h, l, c]) for l in range(s)) % P
    return out.reshape(-1)


@pytest.mark.parametrize("nh,s,d,mods", [(2, 4, 4, (3, 2, 4)), (4, 16, 8, (2, 2, 3)), (1, 64, 16, (1, 1, 3)), (3, 5, 3, (2, 2, 5))])
def test_round_trip_on_the_reference_test_shapes(nh, s, d, mods):
    t = small_exp_table()
    q, k, v = make_qkv(nh, s, d, *mods)
    assert po.row_attention_roundtrip(q, k, v, nh, s, d, t) == 1
    for tamper in (1, 2, 3, 4):
        assert po.row_attention_roundtrip(q, k, v, nh, s, d, t, tamper) == 0, tamper


def test_forward_matches_numpy_and_the_proof_carries_it():
    nh, s, d = 2, 6, 4
    t = tables.build_exp_table(100)
    rng = np.random.default_rng(5)
    q = rng.integers(0, 7, nh * s * d).astype(np.uint32)
    k = np.mod(rng.integers(-6, 7, nh * s * d), P).astype(np.uint32)     # negative scores reach the table's upper half
    v = rng.integers(0, P, nh * s * d).astype(np.uint32)
    out, st = po.row_attention_forward(q, k, v, nh, s, d, t)
    assert st == 0
    assert np.array_equal(out, numpy_forward(q, k, v, nh, s, d, t))
    proof, st = po.prove_row_attention(po.Transcript(b"x"), q, k, v, nh, s, d, t)
    assert st == 0
    # every row's output words appear in the proof, in order
    for r in range(nh * s):
        assert out[r * d:(r + 1) * d].astype("<u4").tobytes() in proof
    assert po.row_attention_roundtrip(q, k, v, nh, s, d, t) == 1


def test_score_outside_the_table_is_reported():
    t = small_exp_table()
    q = np.full(8, 20, np.uint32); k = np.full(8, 20, np.uint32); v = np.ones(8, np.uint32)   # score 800 > 127
    _, st = po.row_attention_forward(q, k, v, 1, 2, 4, t)
    assert st == 8
    proof, st = po.prove_row_attention(po.Transcript(b"x"), q, k, v, 1, 2, 4, t)
    assert st == 8 and proof == b""


def test_gqa_round_trips():
    """attention.rs:737-820: 4 query heads over 2 KV heads, MQA (1 KV head), and GQA with equal head counts."""
    t = small_exp_table()
    s, d = 4, 4
    for nq, nkv in [(4, 2), (4, 1), (2, 2)]:
        i = np.arange(nq * s * d); j = np.arange(nkv * s * d)
        q = ((i % 3) + 1).astype(np.uint32); k = ((j % 2) + 1).astype(np.uint32); v = ((j % 4) + 1).astype(np.uint32)
        assert po.row_attention_roundtrip(q, k, v, nq, s, d, t, 0, nkv) == 1
        for tamper in (1, 2, 3, 4):
            assert po.row_attention_roundtrip(q, k, v, nq, s, d, t, tamper, nkv) == 0
    # with equal head counts GQA computes what MHA computes (attention.rs:799-819); labels and the absorbed header differ
    i = np.arange(2 * s * d)
    q = ((i % 3) + 1).astype(np.uint32); k = ((i % 2) + 1).astype(np.uint32); v = ((i % 4) + 1).astype(np.uint32)
    assert np.array_equal(po.row_attention_forward(q, k, v, 2, s, d, t, 2)[0], po.row_attention_forward(q, k, v, 2, s, d, t)[0])
    a, _ = po.prove_row_attention(po.Transcript(b"x"), q, k, v, 2, s, d, t, 2)
    b, _ = po.prove_row_attention(po.Transcript(b"x"), q, k, v, 2, s, d, t)
    assert len(a) == len(b) and a != b


def test_caller_transcript_stream_is_what_the_prover_absorbs():
    """zklm_compile_b200.attention.caller_transcript_stream (host helper for callers that keep their transcript): absorbing its bytes
    leaves a transcript where prove_row_attention leaves it (attention.rs:140-143, 254-265; GQA :403-406)."""
    from zklm_compile_b200 import attention as za
    t = tables.build_exp_table(100)
    rng = np.random.default_rng(3)
    for nh, nkv, s, d in [(2, 0, 6, 4), (4, 2, 5, 3), (1, 0, 2, 1)]:
        kvh = nkv or nh
        q = np.mod(rng.integers(-2, 3, nh * s * d), P).astype(np.uint32)
        k = np.mod(rng.integers(-2, 3, kvh * s * d), P).astype(np.uint32)
        v = rng.integers(0, P, kvh * s * d).astype(np.uint32)
        tr = po.Transcript(b"x")
        proof, st = po.prove_row_attention(tr, q, k, v, nh, s, d, t, nkv)
        assert st == 0
        mine = po.Transcript(b"x")
        mine.absorb_bytes(za.caller_transcript_stream(proof, nh, s, d, nkv))
        assert mine.squeeze() == tr.squeeze()
