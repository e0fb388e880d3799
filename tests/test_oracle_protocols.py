"""CPU checks of the oracle's protocol layer: forward pieces against the reference's numpy
restatement (tests/golden/qwen_forward.json, produced by tests/golden/make_golden_qwen.py),
and prove -> verify round trips plus tamper rejection for every sub-protocol, mirroring the
reference's own unit-test pattern (e.g. rust/zk_ml_prover/src/proving/matmul.rs:1123-1311,
rmsnorm.rs:905-1009, lookup.rs:979-1569, transformer/qwen.rs tests)."""
import hashlib

import numpy as np
import pytest

from oracle import pyoracle as O
from tests.util import P, load_qwen_golden, rand_layer, small_table

G = load_qwen_golden()


@pytest.mark.parametrize("ci", range(len(G["cases"])))
def test_forward_pieces_match_numpy_reference(ci):
    case = G["cases"][ci]
    cfg, t, w = case["config"], case["trace"], case["weights"]
    x = np.array(case["x"], np.uint32)
    out, xu, delta = O.rmsnorm_forward(x, w["norm1_gamma"])
    assert delta == t["norm1_delta"] and out.tolist() == t["norm1_out"] and xu.tolist() == t["norm1_x"]
    q_dim = cfg["num_q_heads"] * cfg["d_head"]
    assert O.matmul_forward(w["w_q"], t["norm1_out"], q_dim, cfg["d_model"]).tolist() == t["q"]
    assert O.requantize(t["g_proj_out_raw"]).tolist() == t["g_proj_out"]
    assert O.requantize(t["gate_out_raw"]).tolist() == t["gate_out"]
    out2, xu2, d2 = O.rmsnorm_forward(t["h"], w["norm2_gamma"])
    assert d2 == t["norm2_delta"] and out2.tolist() == t["norm2_out"] and xu2.tolist() == t["norm2_x"]


@pytest.mark.parametrize("ci", range(len(G["cases"])))
def test_layer_output_matches_numpy_reference_and_proof_verifies(ci):
    case = G["cases"][ci]
    ih = hashlib.sha256(b"input").digest()
    y, proof, ok = O.qwen_layer_prove(case["config"], case["weights"], case["x"], G["silu"], G["sigmoid"], ci, ih, verify=True)
    assert y.tolist() == case["trace"]["output"]
    assert ok is True
    assert len(proof) > 1000
    # deterministic
    y2, proof2, _ = O.qwen_layer_prove(case["config"], case["weights"], case["x"], G["silu"], G["sigmoid"], ci, ih)
    assert proof2 == proof
    # a different layer index (transcript seed) changes the proof
    _, proof3, _ = O.qwen_layer_prove(case["config"], case["weights"], case["x"], G["silu"], G["sigmoid"], ci + 1, ih)
    assert proof3 != proof


def test_tables_follow_rust_rounding():
    """The package's host-side table builder differs from the numpy reference only where
    x.5 rounds differently (the numpy reference documents a +-1 LSB allowance)."""
    from zklm_compile_b200 import tables
    mine = tables.build_silu_table(G["silu_scale"]).astype(np.int64)
    ref = G["silu"].astype(np.int64)
    diff = np.abs(np.where(mine > P // 2, mine - P, mine) - np.where(ref > P // 2, ref - P, ref))
    assert diff.max() <= 1 and (diff != 0).mean() < 0.01
    assert tables.table_inputs()[[0, 1, 32767, 32768, 65535]].tolist() == [0, 1, 32767, P - 32768, P - 1]


@pytest.mark.parametrize("m,n", [(2, 2), (3, 5), (8, 8), (17, 9), (33, 64)])
@pytest.mark.parametrize("ef", [False, True])
def test_matmul_roundtrip(m, n, ef):
    rng = np.random.default_rng(m * 100 + n)
    w = rng.integers(0, P, m * n, dtype=np.int64).astype(np.uint32)
    x = rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)
    y = O.matmul_forward(w, x, m, n)
    assert O.matmul_succinct_roundtrip(w, x, y, m, n, ef)
    assert not O.matmul_succinct_roundtrip(w, x, y, m, n, ef, tamper=True)
    y_bad = y.copy(); y_bad[0] = (int(y_bad[0]) + 1) % P
    assert not O.matmul_succinct_roundtrip(w, x, y_bad, m, n, ef)


def test_matmul_literal_2x2():
    # rust/zk_ml_prover/src/proving/matmul.rs:1123-1148: W=[3,5,7,11], x=[2,4], y=[26,58]
    assert O.matmul_forward([3, 5, 7, 11], [2, 4], 2, 2).tolist() == [26, 58]
    assert O.matmul_succinct_roundtrip([3, 5, 7, 11], [2, 4], [26, 58], 2, 2, False)


def test_fold_eq_matvec_is_mle_partial_eval():
    rng = np.random.default_rng(3)
    m, n = 6, 5
    w = rng.integers(0, P, m * n, dtype=np.int64).astype(np.uint32)
    r = rng.integers(0, P, 3, dtype=np.int64).astype(np.uint32)
    got = O.fold_eq_matvec(w, m, n, r)
    wp = np.zeros((8, 8), np.uint32); wp[:m, :n] = w.reshape(m, n)
    for j in range(8):
        assert got[j] == O.mle_evaluate(wp[:, j], r)
    r_ef = rng.integers(0, P, 12, dtype=np.int64).astype(np.uint32)
    got_ef = O.fold_eq_matvec_ef(w, m, n, r_ef)
    for j in range(8):
        assert got_ef[j].tolist() == O.mle_evaluate_ef(wp[:, j], r_ef).tolist()


@pytest.mark.parametrize("n", [4, 7, 16])
@pytest.mark.parametrize("add", [False, True])
def test_elementwise_roundtrip(n, add):
    rng = np.random.default_rng(n)
    a = rng.integers(0, P, n, dtype=np.int64); b = rng.integers(0, P, n, dtype=np.int64)
    c = ((a + b) % P if add else (a * b) % P).astype(np.uint32)
    assert O.elementwise_roundtrip(a, b, c, add)
    assert not O.elementwise_roundtrip(a, b, c, add, tamper=True)
    c_bad = c.copy(); c_bad[1] = (int(c_bad[1]) + 1) % P
    assert not O.elementwise_roundtrip(a, b, c_bad, add)


@pytest.mark.parametrize("d", [4, 12, 16])
def test_rmsnorm_roundtrip(d):
    rng = np.random.default_rng(d)
    x = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    gamma = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    y, xu, delta = O.rmsnorm_forward(x, gamma)
    assert O.rmsnorm_roundtrip(xu, gamma, y, delta)
    assert not O.rmsnorm_roundtrip(xu, gamma, y, delta, tamper=True)
    y_bad = y.copy(); y_bad[0] = (int(y_bad[0]) + 1) % P
    assert not O.rmsnorm_roundtrip(xu, gamma, y_bad, delta)


@pytest.mark.parametrize("n_table", [256, 65536])
def test_lookup_roundtrip_and_panics(n_table):
    tab_in, tab_out = small_table(n_table)
    rng = np.random.default_rng(n_table)
    idx = rng.integers(0, n_table, 50)
    ins, outs = tab_in[idx], tab_out[idx]
    assert O.lookup_roundtrip(tab_out, ins, outs)
    assert not O.lookup_roundtrip(tab_out, ins, outs, tamper=True)
    # a wrong output breaks the LogUp identity: the reference panics (lookup.rs:733-738)
    bad = outs.copy(); bad[3] = (int(bad[3]) + 1) % P
    proof, status = O.prove_lookup_ef(O.Transcript(b"x"), tab_out, ins, bad)
    assert status == 3 and proof == b""
    proof, status = O.prove_lookup_ef(O.Transcript(b"x"), tab_out, ins, outs)
    assert status == 0 and len(proof) > 100


def test_layer_tamper_by_wrong_witness():
    cfg, w, x = rand_layer(5, d_model=8, d_ff=12, heads=2, kv=2, d_head=4)
    tab_in, silu = small_table(65536, seed=1)
    _, sigm = small_table(65536, seed=2)
    ih = bytes(32)
    y, proof, ok = O.qwen_layer_prove(cfg, w, x, silu, sigm, 0, ih, verify=True)
    assert ok


@pytest.mark.parametrize("n", [2, 5, 64, 300])
@pytest.mark.parametrize("add", [False, True])
def test_base_field_elementwise_roundtrip(n, add):
    # elementwise.rs base-field tests (prove -> verify, tamper rejected)
    rng = np.random.default_rng(n)
    a = rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)
    b = rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)
    c = ((a.astype(np.int64) + b) % P if add else (a.astype(object) * b.astype(object)) % P).astype(np.uint32)
    k = 1 if n <= 1 else (n - 1).bit_length()
    point = rng.integers(0, P, k, dtype=np.int64).astype(np.uint32)
    assert O.elementwise_base_roundtrip(a, b, c, point, add)
    assert not O.elementwise_base_roundtrip(a, b, c, point, add, tamper=True)
    wrong = c.copy(); wrong[0] = (int(wrong[0]) + 1) % P
    assert not O.elementwise_base_roundtrip(a, b, wrong, point, add)


@pytest.mark.parametrize("n_table,n", [(256, 10), (256, 300), (65536, 500)])
def test_base_field_lookup_roundtrip(n_table, n):
    tab_in, tab_out = small_table(n_table, seed=4)
    rng = np.random.default_rng(n)
    idx = rng.integers(0, n_table, n)
    assert O.lookup_base_roundtrip(tab_out, tab_in[idx], tab_out[idx])
    assert not O.lookup_base_roundtrip(tab_out, tab_in[idx], tab_out[idx], tamper=1)
    assert not O.lookup_base_roundtrip(tab_out, tab_in[idx], tab_out[idx], tamper=2)
    bad = tab_out[idx].copy()
    bad[3] = (int(bad[3]) + 1) % P
    proof, st = O.prove_lookup(O.Transcript(b"x"), tab_out, tab_in[idx], bad)
    assert st == 3 and proof == b""


@pytest.mark.parametrize("d", [4, 12, 100])
def test_base_field_rmsnorm_roundtrip(d):
    rng = np.random.default_rng(d)
    x = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    gamma = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    y, xu, delta = O.rmsnorm_forward(x, gamma)
    assert O.rmsnorm_base_roundtrip(xu, gamma, y, delta)
    assert not O.rmsnorm_base_roundtrip(xu, gamma, y, delta, tamper=1)
    wrong = y.copy(); wrong[1] = (int(wrong[1]) + 1) % P
    assert not O.rmsnorm_base_roundtrip(xu, gamma, wrong, delta)


def test_layer_proof_bytes_decode_and_verify():
    """oracle/unbincode.hpp is the inverse of oracle/bincode.hpp for QwenLayerProofEF: the restated verifier
    accepts the decoded bytes of its own prover, rejects another layer index, and a truncated or extended
    byte string does not decode."""
    import hashlib
    from tests.util import load_qwen_golden, rand_layer
    G = load_qwen_golden()
    cfg, weights, x = rand_layer(1, d_model=64, d_ff=96, heads=2, kv=2, d_head=16, v_heads=4, v_d_head=16)
    ih = hashlib.sha256(b"decode").digest()
    L = O.QwenLayer(cfg, weights, G["silu"], G["sigmoid"])
    y, proof, ok = L.prove(x, 2, ih, verify=True)
    assert ok
    assert L.verify_bytes(x, 2, ih, y, proof) == 1
    assert L.verify_bytes(x, 3, ih, y, proof) == 0
    assert L.verify_bytes(x, 2, ih, y, proof[:-1]) == -1 and L.verify_bytes(x, 2, ih, y, proof + b"\0") == -1
    bad = bytearray(proof)
    bad[40] ^= 1                               # inside the first round polynomial of the first norm's variance sumcheck
    assert L.verify_bytes(x, 2, ih, y, bytes(bad)) == 0
