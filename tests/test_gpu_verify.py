"""The layer verifier on the GPU (verify_qwen_layer_ef_indexed, transformer/qwen.rs:932-1097): it accepts
every proof the prover emits, and decides on tampered bytes exactly as the oracle's restatement of the
reference verifier does (which decodes the same bytes and replays the transcript on the CPU)."""
import hashlib

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import qwen as zq
from oracle import pyoracle as O
from tests.util import load_qwen_golden, rand_layer

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1
SHAPES = {
    "gdn": dict(d_model=64, d_ff=96, heads=2, kv=2, d_head=16, v_heads=4, v_d_head=16),
    "gqa": dict(d_model=64, d_ff=96, heads=4, kv=2, d_head=16, v_heads=2, v_d_head=16),
    "ragged": dict(d_model=80, d_ff=200, heads=4, kv=2, d_head=24, v_heads=2, v_d_head=24),
}


@pytest.fixture(scope="module")
def env():
    G = load_qwen_golden()
    c = zk.Context(0)
    yield c, G, c.upload(G["silu"]), c.upload(G["sigmoid"])
    c.close()


def _layer(env, shape, seed=1):
    c, G, silu, sigm = env
    cfg, weights, x = rand_layer(seed, **SHAPES[shape])
    return zq.QwenLayer(c, cfg, weights, silu, sigm), O.QwenLayer(cfg, weights, G["silu"], G["sigmoid"]), x


def _both(gl, ol, x, idx, ih, y, proof):
    exp = ol.verify_bytes(x, idx, ih, y, proof)
    try:
        got = int(gl.verify(idx, ih, proof, y))
    except zk.ZkbError as e:
        assert e.code == 2
        got = -1
    return got, exp


@pytest.mark.parametrize("shape", list(SHAPES))
def test_layer_verifier_accepts_honest_proofs_and_rejects_wrong_statements(env, shape):
    gl, ol, x = _layer(env, shape)
    ih = hashlib.sha256(b"verify-" + shape.encode()).digest()
    y = gl.forward(x)
    proof = gl.prove(5, ih)
    assert _both(gl, ol, x, 5, ih, y, proof) == (1, 1)
    assert gl.verify(5, ih, proof) is True                       # without the claimed output
    assert _both(gl, ol, x, 6, ih, y, proof) == (0, 0)           # another layer index: another transcript
    assert _both(gl, ol, x, 5, hashlib.sha256(b"other").digest(), y, proof) == (0, 0)
    y2 = y.copy(); y2[3] = (int(y2[3]) + 1) % P
    assert _both(gl, ol, x, 5, ih, y2, proof) == (0, 0)
    # a proof about another input does not verify against this layer's trace
    x2 = x.copy(); x2[0] = (int(x2[0]) + 1) % P
    y_other = gl.forward(x2)
    other = gl.prove(5, ih)
    gl.forward(x)
    assert _both(gl, ol, x, 5, ih, y, other)[0] == 0
    assert gl.verify(5, ih, proof, y) is True                    # and the verifier left the layer usable
    assert not np.array_equal(y_other, y)
    gl.close()


@pytest.mark.parametrize("shape", ["gdn", "gqa"])
def test_layer_verifier_decides_tampered_bytes_like_the_oracle(env, shape):
    gl, ol, x = _layer(env, shape, seed=3)
    ih = hashlib.sha256(b"tamper").digest()
    y = gl.forward(x)
    proof = gl.prove(0, ih)
    rng = np.random.default_rng(11)
    spots = [0, 3, 4, 11, 12, 100, len(proof) - 1, len(proof) - 5, len(proof) - 52, len(proof) - 416]
    spots += [int(v) for v in rng.integers(0, len(proof), 170)]
    seen = {}
    for pos in spots:
        bad = bytearray(proof)
        bad[pos] ^= 1 << int(rng.integers(0, 8))
        got, exp = _both(gl, ol, x, 0, ih, y, bytes(bad))
        assert got == exp, f"byte {pos}: GPU {got}, oracle {exp}"
        seen[exp] = seen.get(exp, 0) + 1
    assert seen.get(0, 0) > 100 and seen.get(-1, 0) > 5        # most changes are caught by a check, some break the encoding
    assert _both(gl, ol, x, 0, ih, y, proof[:-1]) == (-1, -1)
    assert _both(gl, ol, x, 0, ih, y, proof + b"\0") == (-1, -1)
    gl.close()


@pytest.mark.parametrize("bind,kind", [(1, 0), (1, 1), (2, 0), (2, 1)])
def test_layer_verifier_with_basefold_bound_matmuls(env, bind, kind):
    """Layer proofs whose matmuls carry a Basefold opening (features pcs / pcs-full, either node hash): the
    opening is checked by the GPU Basefold verifier inside the layer verifier."""
    gl, ol, x = _layer(env, "gdn", seed=4)
    ih = hashlib.sha256(b"pcs").digest()
    gl.set_binding(bind, kind)
    y = gl.forward(x)
    proof = gl.prove(1, ih)
    with O.features(bind, kind):
        assert _both(gl, ol, x, 1, ih, y, proof) == (1, 1)
        rng = np.random.default_rng(bind * 2 + kind)
        for pos in rng.integers(0, len(proof), 40):
            bad = bytearray(proof)
            bad[int(pos)] ^= 1 << int(rng.integers(0, 8))
            got, exp = _both(gl, ol, x, 1, ih, y, bytes(bad))
            assert got == exp, f"byte {int(pos)}: GPU {got}, oracle {exp}"
    gl.close()


def test_model_verifier_checks_all_layers_side_by_side(env):
    """QwenModel.forward_and_verify: the proofs of a three-layer stack as forward_and_prove returns them are
    accepted; one changed proof, a swapped order or a wrong claimed output are rejected."""
    c, G, _, _ = env
    cfgs, ws = [], []
    for i in range(3):
        cfg, w, x = rand_layer(20 + i, **SHAPES["gdn" if i % 2 == 0 else "gqa"])
        cfgs.append(cfg); ws.append(w)
    _, _, x = rand_layer(19, **SHAPES["gdn"])
    model = zq.QwenModel(0, cfgs, ws, G["silu"], G["sigmoid"])
    ih = zq.hash_values(x)
    proofs = model.forward_and_prove(x, ih)
    y = model.output()
    assert model.forward_and_verify(x, proofs, ih, y) is True
    assert model.forward_and_verify(x, proofs, ih) is True
    assert model.forward_and_verify(x, proofs[::-1], ih, y) is False
    y2 = y.copy(); y2[0] = (int(y2[0]) + 1) % P
    assert model.forward_and_verify(x, proofs, ih, y2) is False
    bad = bytearray(proofs[1]); bad[200] ^= 1
    try:
        assert model.forward_and_verify(x, [proofs[0], bytes(bad), proofs[2]], ih, y) is False
    except zk.ZkbError as e:
        assert e.code == 2
    assert model.forward_and_verify(x, proofs, ih, y) is True
    assert model.forward_and_prove(x, ih) == proofs               # and the prover still works on the same model
    model.close()


def test_graph_replay_comes_back_after_the_arena_was_trimmed(env):
    """zkb_ctx_trim frees the scratch arena; the next proofs let it grow back launch by launch, then the launch
    sequence is captured again and replayed (graph state 2), with the same proof bytes throughout."""
    gl, ol, x = _layer(env, "gdn", seed=6)
    c = env[0]
    ih = hashlib.sha256(b"trim").digest()
    gl.forward(x)
    ref = gl.prove(0, ih)
    for _ in range(4):
        assert gl.prove(0, ih) == ref
    assert gl.graph_state() == 2
    c.trim()
    assert gl.graph_state() != 2
    states = []
    for _ in range(5):
        assert gl.prove(0, ih) == ref
        states.append(gl.graph_state())
    assert states[-1] == 2, states
    gl.close()
