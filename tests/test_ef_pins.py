"""The oracle and the CUDA kernels against vectors that come from neither: tests/golden/ef_pins.json
is produced by tests/golden/make_golden_ef.py from the field definition and the reference's
Transcript / prove_product_ef source in exact Python integers (hashlib for SHA-256)."""
import json
import os

import numpy as np
import pytest

from oracle import pyoracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
P = (1 << 31) - 1


@pytest.fixture(scope="module")
def pins():
    with open(os.path.join(HERE, "golden", "ef_pins.json")) as fh:
        return json.load(fh)


def _replay(t, case):
    out = []
    for op, arg in case["ops"]:
        if op == "absorb":
            t.absorb_many(np.array(arg, np.uint32))
        else:
            out.append([t.squeeze() for _ in range(arg)])
    return out


# ---- the oracle (CPU) -------------------------------------------------------------------------
def test_oracle_ef_tower_matches_the_definition(pins):
    for c in pins["ef_cases"]:
        assert O.ef_mul(c["a"], c["b"]).tolist() == c["mul"]
        assert O.ef_inv(c["a"]).tolist() == c["inv_a"]


def test_oracle_transcript_matches_hashlib_restatement(pins):
    for c in pins["transcripts"]:
        assert _replay(O.Transcript(c["label"].encode()), c) == c["squeezed"]


def test_oracle_product_ef_bytes_match_the_python_restatement(pins):
    for c in pins["product_ef"]:
        nv = c["num_vars"]
        polys, chal, fin = O.prove("product_ef", O.Transcript(c["label"].encode()), [np.array(c["f"], np.uint32), np.array(c["g"], np.uint32)], nv)
        assert polys.reshape(nv, 2, 4).tolist() == c["round_polys"]
        assert chal.tolist() == c["challenges"]
        assert fin[0].tolist() == c["f_at_s"] and fin[1].tolist() == c["g_at_s"]


# ---- the kernels (GPU), through the C ABI --------------------------------------------------------
@pytest.fixture(scope="module")
def ctx():
    import zklm_compile_b200 as zk
    c = zk.Context(0)
    yield c
    c.close()


@pytest.mark.gpu
def test_gpu_ef_tower_matches_the_definition(ctx, pins):
    from zklm_compile_b200 import protocols as zp
    a = np.array([c["a"] for c in pins["ef_cases"]], np.uint32)
    # inverse: zkb_batch_inverse_ef
    assert zp.batch_inverse(ctx, a, ef=True).tolist() == [c["inv_a"] for c in pins["ef_cases"]]
    # product: the MLE of the two-entry table [0, b] at the point (a) is a * b
    for c in pins["ef_cases"]:
        table = np.array([[0, 0, 0, 0], c["b"]], np.uint32)
        assert zp.mle_evaluate_ef(ctx, table, np.array([c["a"]], np.uint32), evals_ef=True).tolist() == c["mul"]


@pytest.mark.gpu
def test_gpu_transcript_matches_hashlib_restatement(ctx, pins):
    import zklm_compile_b200 as zk
    for c in pins["transcripts"]:
        assert _replay(zk.Transcript(ctx, c["label"].encode()), c) == c["squeezed"]


@pytest.mark.gpu
def test_gpu_product_ef_bytes_match_the_python_restatement(ctx, pins):
    import zklm_compile_b200 as zk
    for c in pins["product_ef"]:
        nv = c["num_vars"]
        proof, fs, gs = zk.prove_product_ef(np.array(c["f"], np.uint32), np.array(c["g"], np.uint32), nv, zk.Transcript(ctx, c["label"].encode()))
        assert proof.round_polys.tolist() == c["round_polys"]
        assert proof.challenges.tolist() == c["challenges"]
        assert fs.tolist() == c["f_at_s"] and gs.tolist() == c["g_at_s"]
