"""GPU parity of the protocol layer against the CPU oracle: every proof is compared as
bincode bytes (bit-exact; all arithmetic is integer field arithmetic)."""
import hashlib

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import protocols as zp
from zklm_compile_b200 import qwen as zq
from oracle import pyoracle as O
from tests.util import P, load_qwen_golden, rand_layer, small_table

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def rnd(rng, n):
    return rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)


@pytest.mark.parametrize("n", [0, 1, 3, 250, 254, 255, 256, 257, 511, 512, 513, 1000, 4096, 70001, 1 << 20])
def test_blake3_commit_matches_oracle(ctx, n):
    w = rnd(np.random.default_rng(n), n)
    assert zp.commit_weights_fast(ctx, w) == O.commit_weights_fast(w)


@pytest.mark.parametrize("k", [1, 2, 5, 12])
def test_eq_evals(ctx, k):
    rng = np.random.default_rng(k)
    r = rnd(rng, k)
    assert zp.eq_evals(ctx, r).tolist() == O.eq_evals(r).tolist()
    r4 = rnd(rng, 4 * k).reshape(k, 4)
    assert zp.eq_evals_ef(ctx, r4).tolist() == O.eq_evals_ef(r4).tolist()


def test_eq_evals_literal(ctx):
    # rust/zk_ml_prover/src/field/m31_ops.rs:212-228
    assert zp.eq_evals(ctx, [2, 3]).tolist() == [2, P - 3, P - 4, 6]


@pytest.mark.parametrize("m,n", [(2, 2), (3, 5), (17, 9), (64, 64), (100, 260), (513, 1028), (700, 33)])
@pytest.mark.parametrize("ef", [False, True])
def test_fold_eq_matvec_and_forward(ctx, m, n, ef):
    rng = np.random.default_rng(m * 1000 + n)
    w = rnd(rng, m * n)
    log_m = zp.log2_ceil(m)
    r = rnd(rng, log_m * (4 if ef else 1))
    got = zp.fold_eq_matvec(ctx, w, m, n, r, ef=ef)
    exp = O.fold_eq_matvec_ef(w, m, n, r) if ef else O.fold_eq_matvec(w, m, n, r)
    assert got.tolist() == exp.tolist()
    x = rnd(rng, n)
    assert zp.matmul_forward(ctx, w, x, m, n).tolist() == O.matmul_forward(w, x, m, n).tolist()


def test_matmul_forward_extreme_values(ctx):
    m, n = 8, 4096
    w = np.full(m * n, P - 1, np.uint32)
    x = np.full(n, P - 1, np.uint32)
    assert zp.matmul_forward(ctx, w, x, m, n).tolist() == O.matmul_forward(w, x, m, n).tolist()
    r = np.full(3, P - 1, np.uint32)
    assert zp.fold_eq_matvec(ctx, w, m, n, r).tolist() == O.fold_eq_matvec(w, m, n, r).tolist()


@pytest.mark.parametrize("m,n", [(2, 2), (3, 5), (17, 9), (64, 40), (300, 2100)])
def test_matmul_succinct_ef_bytes(ctx, m, n):
    rng = np.random.default_rng(m + n)
    w, x = rnd(rng, m * n), rnd(rng, n)
    y = O.matmul_forward(w, x, m, n)
    t, o = zk.Transcript(ctx, b"mm"), O.Transcript(b"mm")
    got = zp.prove_matmul_succinct_ef(w, x, y, m, n, t)
    exp = O.prove_matmul_succinct(o, w, x, y, m, n, ef=True)
    assert got == exp
    assert t.squeeze() == o.squeeze()


@pytest.mark.parametrize("m,n", [(2, 2), (3, 5), (17, 9), (64, 40), (300, 2100), (1024, 1024)])
def test_matmul_succinct_base_bytes(ctx, m, n):
    rng = np.random.default_rng(m + 3 * n)
    w, x = rnd(rng, m * n), rnd(rng, n)
    y = O.matmul_forward(w, x, m, n)
    t, o = zk.Transcript(ctx, b"mm-base"), O.Transcript(b"mm-base")
    got = zp.prove_matmul_succinct(w, x, y, m, n, t)
    exp = O.prove_matmul_succinct(o, w, x, y, m, n, ef=False)
    assert got == exp
    assert t.squeeze() == o.squeeze()


@pytest.mark.parametrize("n,k", [(2, 1), (5, 3), (100, 7), (4096, 12), (5000, 13)])
def test_mle_eval_bound_base_bytes(ctx, n, k):
    rng = np.random.default_rng(n)
    w, point = rnd(rng, n), rnd(rng, k)
    padded = np.zeros(1 << k, np.uint32)
    padded[:n] = w
    root = O.commit_weights_fast(padded)
    t, o = zk.Transcript(ctx, b"ev"), O.Transcript(b"ev")
    got = zp.prove_mle_eval_bound(w, point, b"some-label", root, t)
    exp, _ = O.prove_mle_eval_bound(o, w, point, b"some-label", ef=False)
    assert got == exp
    assert t.squeeze() == o.squeeze()


@pytest.mark.parametrize("n", [2, 7, 16, 100, 5000])
@pytest.mark.parametrize("add", [False, True])
def test_elementwise_ef_bytes(ctx, n, add):
    rng = np.random.default_rng(n)
    a, b = rnd(rng, n), rnd(rng, n)
    c = ((a.astype(np.int64) + b) % P if add else (a.astype(object) * b.astype(object)) % P).astype(np.uint32)
    k = zp.log2_ceil(n)
    point = rnd(rng, 4 * k).reshape(k, 4)
    t, o = zk.Transcript(ctx, b"ew"), O.Transcript(b"ew")
    got = (zp.prove_add_ef if add else zp.prove_hadamard_ef)(a, b, c, point, t)
    exp = O.prove_elementwise_ef(o, a, b, c, point, add)
    assert got == exp
    assert t.squeeze() == o.squeeze()


@pytest.mark.parametrize("n", [2, 7, 16, 100, 5000, 20000])
@pytest.mark.parametrize("add", [False, True])
def test_elementwise_base_bytes(ctx, n, add):
    rng = np.random.default_rng(n + 1)
    a, b = rnd(rng, n), rnd(rng, n)
    c = ((a.astype(np.int64) + b) % P if add else (a.astype(object) * b.astype(object)) % P).astype(np.uint32)
    k = zp.log2_ceil(n)
    point = rnd(rng, k)
    t, o = zk.Transcript(ctx, b"ewb"), O.Transcript(b"ewb")
    got = (zp.prove_add if add else zp.prove_hadamard)(a, b, c, point, t)
    exp = O.prove_elementwise(o, a, b, c, point, add)
    assert got == exp
    assert t.squeeze() == o.squeeze()


@pytest.mark.parametrize("d", [4, 12, 16, 100, 2560])
def test_rmsnorm_forward_and_proof_bytes(ctx, d):
    rng = np.random.default_rng(d)
    x = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    gamma = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    y, xu, delta = zp.rmsnorm_forward(ctx, x, gamma)
    ey, exu, edelta = O.rmsnorm_forward(x, gamma)
    assert delta == edelta and y.tolist() == ey.tolist() and xu.tolist() == exu.tolist()
    t, o = zk.Transcript(ctx, b"rn"), O.Transcript(b"rn")
    got = zp.prove_rmsnorm_ef(xu, gamma, y, delta, t)
    exp = O.prove_rmsnorm_ef(o, xu, gamma, y, delta)
    assert got == exp
    assert t.squeeze() == o.squeeze()


@pytest.mark.parametrize("d", [4, 12, 100, 768, 2560])
def test_rmsnorm_base_proof_bytes(ctx, d):
    rng = np.random.default_rng(d + 11)
    x = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    gamma = np.mod(rng.integers(-127, 128, d), P).astype(np.uint32)
    y, xu, delta = O.rmsnorm_forward(x, gamma)
    t, o = zk.Transcript(ctx, b"rnb"), O.Transcript(b"rnb")
    assert zp.prove_rmsnorm(xu, gamma, y, delta, t) == O.prove_rmsnorm(o, xu, gamma, y, delta)
    assert t.squeeze() == o.squeeze()


def test_rmsnorm_forward_needs_perturbation(ctx):
    """Find seeded inputs whose d / sum_sq is not a residue, so the +-delta search runs."""
    found = 0
    for seed in range(60):
        rng = np.random.default_rng(seed)
        x = np.mod(rng.integers(-127, 128, 8), P).astype(np.uint32)
        g = np.ones(8, np.uint32)
        ey, exu, edelta = O.rmsnorm_forward(x, g)
        y, xu, delta = zp.rmsnorm_forward(ctx, x, g)
        assert delta == edelta and y.tolist() == ey.tolist() and xu.tolist() == exu.tolist()
        found += delta != 0
    assert found > 5


@pytest.mark.parametrize("n_table,n", [(256, 10), (256, 300), (65536, 50), (65536, 4096), (65536, 9728)])
def test_lookup_ef_bytes(ctx, n_table, n):
    tab_in, tab_out = small_table(n_table, seed=3)
    rng = np.random.default_rng(n)
    idx = rng.integers(0, n_table, n)
    ins, outs = tab_in[idx], tab_out[idx]
    t, o = zk.Transcript(ctx, b"lk"), O.Transcript(b"lk")
    got = zp.prove_lookup_ef(tab_out, ins, outs, t)
    exp, st = O.prove_lookup_ef(o, tab_out, ins, outs)
    assert st == 0 and got == exp
    assert t.squeeze() == o.squeeze()


@pytest.mark.parametrize("n_table,n", [(256, 10), (256, 300), (65536, 50), (65536, 4096), (65536, 3072)])
def test_lookup_base_bytes(ctx, n_table, n):
    tab_in, tab_out = small_table(n_table, seed=5)
    rng = np.random.default_rng(n + 7)
    idx = rng.integers(0, n_table, n)
    ins, outs = tab_in[idx], tab_out[idx]
    t, o = zk.Transcript(ctx, b"lkb"), O.Transcript(b"lkb")
    got = zp.prove_lookup(tab_out, ins, outs, t)
    exp, st = O.prove_lookup(o, tab_out, ins, outs)
    assert st == 0 and got == exp
    assert t.squeeze() == o.squeeze()
    bad = outs.copy()
    bad[0] = (int(bad[0]) + 1) % P
    with pytest.raises(zk.ZkbError) as e:
        zp.prove_lookup(tab_out, ins, bad, zk.Transcript(ctx, b"lkb"))
    assert e.value.code == 3


def test_lookup_invalid_witness_is_an_error(ctx):
    """The reference panics with "LogUp identity failed" (lookup.rs:733-738); the library returns
    the matching status instead of a proof."""
    tab_in, tab_out = small_table(256)
    idx = np.arange(20)
    outs = tab_out[idx].copy()
    outs[5] = (int(outs[5]) + 1) % P
    with pytest.raises(zk.ZkbError) as e:
        zp.prove_lookup_ef(tab_out, tab_in[idx], outs, zk.Transcript(ctx, b"bad"))
    assert e.value.code == 3


def _check_layer(ctx, cfg, weights, x, silu, sigm, idx):
    ih = hashlib.sha256(b"model-input").digest()
    td = (ctx.upload(silu), ctx.upload(sigm))
    layer = zq.QwenLayer(ctx, cfg, weights, *td)
    y = layer.forward(x)
    ey, eproof, ok = O.qwen_layer_prove(cfg, weights, x, silu, sigm, idx, ih, verify=True)
    assert y.tolist() == ey.tolist()
    roots = layer.commitments()
    assert roots[0] == O.commit_weights_fast(weights["w_q"]) and roots[7] == O.commit_weights_fast(weights["w_down"])
    proof = layer.prove(idx, ih)
    assert ok, "oracle verifier rejected the oracle proof"
    assert len(proof) == len(eproof)
    assert proof == eproof, "layer proof bytes differ from the oracle"
    # proving twice gives the same bytes (buffers are reused, nothing stale leaks); the second
    # proof captures the launch sequence into a graph, later ones replay it
    assert layer.prove(idx, ih) == eproof
    assert layer.prove(idx, ih) == eproof
    # a replay with another layer index and input hash (the transcript seed is device-resident)
    ih2 = hashlib.sha256(b"another-input").digest()
    _, eproof2, _ = O.qwen_layer_prove(cfg, weights, x, silu, sigm, idx + 12, ih2)
    assert layer.prove(idx + 12, ih2) == eproof2
    # and launch-by-launch enqueueing still agrees
    layer.use_graph(False)
    assert layer.prove(idx, ih) == eproof
    layer.close()


def test_launch_trace_of_a_replayed_layer_graph(tmp_path):
    """With the launch trace on, a layer proof has the same bytes, and the dump holds one line per
    traced launch of the captured graph with non-decreasing times (the events are event-record
    nodes of the graph, refreshed by every replay)."""
    G = load_qwen_golden()
    case = G["cases"][0]
    c = zk.Context(0)
    c.trace(True)
    ih = hashlib.sha256(b"model-input").digest()
    layer = zq.QwenLayer(c, case["config"], case["weights"], c.upload(G["silu"]), c.upload(G["sigmoid"]))
    x = np.array(case["x"], np.uint32)
    layer.forward(x)
    _, eproof, _ = O.qwen_layer_prove(case["config"], case["weights"], x, G["silu"], G["sigmoid"], 0, ih)
    for _ in range(3):                      # launch by launch, captured, replayed
        assert layer.prove(0, ih) == eproof
    path = str(tmp_path / "trace.csv")
    c.trace_dump(path)
    lines = open(path).read().strip().split("\n")
    assert lines[0] == "index,site,ms"
    rows = [l.split(",") for l in lines[1:]]
    assert len(rows) > 50 and all(".cuh:" in r[1] or ".cu:" in r[1] for r in rows)
    proof_rows = [float(r[2]) for r in rows if float(r[2]) >= 0]
    assert proof_rows == sorted(proof_rows) and proof_rows[-1] > proof_rows[0]
    c.trace(False)
    layer.close()
    c.close()


def test_qwen_layer_golden_cases(ctx):
    G = load_qwen_golden()
    for ci, case in enumerate(G["cases"]):
        _check_layer(ctx, case["config"], case["weights"], np.array(case["x"], np.uint32), G["silu"], G["sigmoid"], ci)


@pytest.mark.parametrize("shape", [
    dict(d_model=64, d_ff=96, heads=2, kv=2, d_head=16, v_heads=4, v_d_head=16),     # GDN-style, asymmetric V
    dict(d_model=80, d_ff=200, heads=8, kv=2, d_head=8),                               # GQA full attention
    dict(d_model=320, d_ff=1216, heads=2, kv=2, d_head=128, v_heads=4, v_d_head=128),  # 1/8-scale 4B GDN layer
])
def test_qwen_layer_random(ctx, shape):
    cfg, weights, x = rand_layer(11, **shape)
    G = load_qwen_golden()
    _check_layer(ctx, cfg, weights, x, G["silu"], G["sigmoid"], 7)


def test_qwen_model_two_layers_reverse_order(ctx):
    G = load_qwen_golden()
    shapes = [dict(d_model=64, d_ff=96, heads=2, kv=2, d_head=16, v_heads=4, v_d_head=16),
              dict(d_model=64, d_ff=96, heads=4, kv=2, d_head=16)]
    layers = [rand_layer(20 + i, **s) for i, s in enumerate(shapes)]
    x = layers[0][2]
    model = zq.QwenModel(0, [l[0] for l in layers], [l[1] for l in layers], G["silu"], G["sigmoid"])
    model.forward(x)
    y = model.output()
    proofs = model.prove()
    ih = zq.hash_values(x)
    assert ih == O.hash_values(x)
    cur, exp = x, []
    for i, (cfg, w, _) in enumerate(layers):
        cur, pr, ok = O.qwen_layer_prove(cfg, w, cur, G["silu"], G["sigmoid"], i, ih, verify=True)
        assert ok
        exp.append(pr)
    assert y.tolist() == cur.tolist()
    assert proofs == exp[::-1]
    # the overlapped path (forward of layer i+1 behind an event, proofs enqueued right away) gives the same bytes
    assert model.forward_and_prove(x) == exp[::-1]
    assert model.forward_and_prove(model.ctxs[0].upload(x), ih) == exp[::-1]
    model.close()


@pytest.mark.parametrize("ef", [True, False])
def test_dense_chain_matches_oracle(ctx, ef):
    """The Dense-4M shape of the reference's benchmark at 1/16 scale: four linears with a lookup
    activation between them, proved on one transcript; every proof byte-identical to the oracle's."""
    from zklm_compile_b200 import mlp, tables
    dims = [64, 64, 64, 64, 64]
    rng = np.random.default_rng(17)
    weights = [np.mod(rng.integers(-127, 128, dims[l + 1] * dims[l]), P).astype(np.uint32) for l in range(4)]
    x = np.mod(rng.integers(-127, 128, dims[0]), P).astype(np.uint32)
    table_out = tables.build_gelu_table(1000)
    chain = mlp.DenseChain(ctx, weights, dims, table_out)
    trace = chain.forward(x)
    t, o = zk.Transcript(ctx, b"structured-ml-proof"), O.Transcript(b"structured-ml-proof")
    proofs = chain.prove(trace, t, ef=ef)
    cur, k = x, 0
    for l in range(4):
        m, n = dims[l + 1], dims[l]
        y = O.matmul_forward(weights[l], cur, m, n)
        assert y.tolist() == trace[l][1].tolist()
        assert proofs[k] == O.prove_matmul_succinct(o, weights[l], cur, y, m, n, ef=ef); k += 1
        if l < 3:
            q = O.requantize(y)
            assert q.tolist() == trace[l][2].tolist()
            a = trace[l][3]
            exp, st = (O.prove_lookup_ef if ef else O.prove_lookup)(o, table_out, q, a)
            assert st == 0 and proofs[k] == exp; k += 1
            cur = a
    assert t.squeeze() == o.squeeze()
    chain.close()
