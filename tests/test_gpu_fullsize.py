"""GPU proofs against the oracle at the sizes the benchmark configurations name, byte for byte:
one GatedDeltaNet-shape and one GQA-shape layer of the Qwen3.5-4B shape (d_model 2560, d_ff 9728)
with exactly the benchmark's seeded weights and input, one layer of the 9B shape (4096 / 12288),
and one 9728 x 2560 matmul proof with the Basefold commitment of the whole padded matrix
(feature pcs-full, 2^26 coefficients).  The oracle side takes a few seconds per case."""
import hashlib
import os

import numpy as np
import pytest

import bench
import zklm_compile_b200 as zk
from zklm_compile_b200 import protocols as zp, qwen as zq, tables
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1


@pytest.fixture(scope="module")
def env():
    c = zk.Context(0)
    silu, sigm = tables.build_silu_table(1000), tables.build_sigmoid_table(1000)
    yield c, silu, sigm, c.upload(silu), c.upload(sigm)
    c.close()


def _layer_case(env, cfg, weights, x, layer_idx):
    c, silu, sigm, silu_d, sigm_d = env
    ih = zq.hash_values(x)
    layer = zq.QwenLayer(c, cfg, weights, silu_d, sigm_d)
    try:
        y = layer.forward(x)
        ol = O.QwenLayer(cfg, weights, silu, sigm)
        O.set_threads(8)
        ey, eproof, ok = ol.prove(x, layer_idx, ih, verify=True)
        O.set_threads(1)
        assert ok, "the oracle's verifier rejects the oracle's proof"
        assert y.tolist() == ey.tolist(), "forward output differs from the oracle"
        for attempt in range(3):                # launch by launch, captured, replayed
            got = layer.prove(layer_idx, ih)
            assert len(got) == len(eproof) and got == eproof, f"layer proof differs from the oracle (attempt {attempt})"
        # the GPU verifier at the real size: accepts the proof, rejects it for another layer index and with one bit changed
        assert layer.verify(layer_idx, ih, got, y) is True
        assert layer.verify(layer_idx + 1, ih, got, y) is False
        bad = bytearray(got)
        bad[len(bad) // 2] ^= 4
        try:
            assert layer.verify(layer_idx, ih, bytes(bad), y) is False
        except zk.ZkbError as e:
            assert e.code == 2
        return hashlib.sha256(eproof).hexdigest()
    finally:
        layer.close()


@pytest.mark.parametrize("layer_idx", [0, 3])      # 0: GatedDeltaNet structure, 3: GQA full attention
def test_qwen4b_shape_layer_bytes(env, layer_idx):
    cfg = bench.qwen4b_layer_config(layer_idx)
    _layer_case(env, cfg, bench.synth_weights(cfg, layer_idx), bench.synth_input(2560), layer_idx)


def test_qwen9b_shape_layer_bytes(env):
    cfg = dict(d_model=4096, d_ff=12288, num_q_heads=16, num_kv_heads=16, d_head=128, v_num_heads=32, v_d_head=128)
    rng = np.random.default_rng(9)
    _layer_case(env, cfg, bench.synth_weights(cfg, 40), np.mod(rng.integers(-127, 128, 4096), P).astype(np.uint32), 5)


def _pcs_full_case(c, m, n, node_hash, label):
    rng = np.random.default_rng(m + n)
    w = np.mod(rng.integers(-127, 128, m * n, dtype=np.int32), P).astype(np.uint32)
    x = np.mod(rng.integers(-127, 128, n), P).astype(np.uint32)
    O.set_threads(8)
    try:
        y = O.matmul_forward(w, x, m, n)
        with O.features(O.BIND_PCS_FULL, node_hash):
            exp = O.prove_matmul_succinct(O.Transcript(label), w, x, y, m, n, ef=True)
    finally:
        O.set_threads(1)
    w_dev = c.upload(w)
    got = zp.prove_matmul_succinct_ef(w_dev, x, y, m, n, zk.Transcript(c, label), bind_mode=zp.BIND_PCS_FULL, node_hash=node_hash)
    w_dev.free()
    assert len(got) == len(exp) and got == exp


@pytest.mark.parametrize("node_hash", [0, 1])
def test_pcs_full_matmul_half_scale_bytes(env, node_hash):
    """bind_weights_ef, pcs-full branch (matmul.rs:372-419) at half the 4B shape's largest matrix:
    4864 x 1280, a Basefold commitment over 2^13 x 2^11 = 2^24 coefficients (the oracle needs a few
    seconds for it; the full 9728 x 2560 case below needs about a minute of CPU and is opt-in)."""
    _pcs_full_case(env[0], 4864, 1280, node_hash, b"pcs-full-half")


@pytest.mark.skipif(not os.environ.get("ZKB_SLOW_TESTS"), reason="about a minute of oracle CPU time; set ZKB_SLOW_TESTS=1")
def test_pcs_full_matmul_9728x2560_bytes(env):
    """The same at full size: 9728 x 2560 padded to 2^14 x 2^12 = 2^26 coefficients."""
    _pcs_full_case(env[0], 9728, 2560, 0, b"pcs-full-9728")


def test_basefold_2_26_properties(env):
    """Size-independent checks of the Basefold commitment at the pcs-full size of the 4B shape
    (2^26 coefficients = the row-padded 9728 x 2560 matrix): the opening's final value is the
    multilinear evaluation of the coefficients at the point (computed by the separately tested MLE
    kernel at a random point), and the committed root is the Merkle root of the codeword."""
    from zklm_compile_b200 import pcs as zpc
    c = env[0]
    log_n = 26
    rng = np.random.default_rng(2626)
    coeffs = c.upload(np.mod(rng.integers(-127, 128, 1 << log_n, dtype=np.int32), P).astype(np.uint32))
    point_h = rng.integers(0, P, log_n, dtype=np.int64).astype(np.uint32)
    point = c.upload(point_h)
    blob = zpc.basefold_commit_and_prove(c, zk.Transcript(c, b"bf-2-26"), coeffs, point)
    assert int.from_bytes(blob[16:24], "little") == 1 << log_n and int.from_bytes(blob[24:32], "little") == log_n
    final_value = int.from_bytes(blob[-12:-8], "little")
    assert final_value == zp.mle_evaluate(c, coeffs, point_h)
    cw = c.alloc(2 << log_n)
    zpc.basefold_encode(c, coeffs, out=cw)
    assert blob[:16] == zpc.merkle_root(c, cw)
    for b in (coeffs, point, cw):
        b.free()


def test_batch_basefold_of_a_4b_layer_is_accepted_by_the_restated_verifier(env):
    """Batch Basefold at the real size (the eight weight matrices of a 4B-shape attention layer, 2^22 .. 2^25 coefficients, far beyond
    what the CPU prover restatement does in test time): the restated batch_verify_opening accepts the GPU's bytes and ends in the same
    transcript state, rejects them with one opened value changed, and the final value is the rho-weighted sum of the polynomials'
    multilinear evaluations (computed with the separately tested MLE kernel; the reference's verifier does not check it)."""
    from zklm_compile_b200 import pcs as zpc
    c = env[0]
    cfg = bench.qwen4b_layer_config(3)
    sizes = bench.layer_sizes(cfg)
    names = ["w_q", "w_k", "w_v", "w_o", "w_g_proj", "w_gate", "w_up", "w_down"]
    w = bench.synth_weights(cfg, 3)
    log_ns = [max(1, (sizes[n] - 1).bit_length()) for n in names]
    polys = [c.upload(w[n]) for n in names]
    b = zpc.BasefoldBatch(c, polys, log_ns)
    tg = zk.Transcript(c, b"batch-4b")
    blob = b.prove(tg)
    to = O.Transcript(b"batch-4b")
    O.set_threads(8)
    rc, final_value = O.basefold_batch_verify_bytes(to, blob)
    O.set_threads(1)
    assert rc == 1 and tg.squeeze() == to.squeeze()
    # the transcript gives rho and the fold point back: replay the public part on the oracle's transcript type
    k = len(names)
    order = sorted(range(k), key=lambda i: -log_ns[i])            # stable, like the prover's sort
    tr = O.Transcript(b"batch-4b")
    for i in order:
        tr.absorb_bytes(b.commitment(i)[0])
    rho = tr.squeeze()
    at = 8 + 32 * k + 8 + 8 + 8 * k + 8 + 16 * k
    tr.absorb_bytes(blob[at:at + 16])
    point = [tr.squeeze() for _ in range(max(log_ns))]
    acc, pw = 0, 1
    for i in order:
        acc = (acc + pw * zp.mle_evaluate(c, polys[i], np.array(point[:log_ns[i]], np.uint32))) % P
        pw = pw * rho % P
    assert acc == final_value
    bad = bytearray(blob)
    at_values = blob.index((48).to_bytes(8, "little"), at + 16 + 8 + 16 * max(log_ns)) + 8 + 4 * 48 + 8     # first opened value of round 0
    bad[at_values] ^= 1
    assert O.basefold_batch_verify_bytes(O.Transcript(b"batch-4b"), bytes(bad))[0] == 0
    b.close()
    for x in polys:
        x.free()
