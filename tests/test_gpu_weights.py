"""Weights taken in the reference's preload format (server.rs:33-94) and kept on the GPU: contents and
commit_weights_fast roots against the oracle, use of the resident matrices by a proof, and the reference's
caps and error cases."""
import struct

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import protocols as zp, weights as zw
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1


@pytest.fixture(scope="module")
def ctx():
    c = zk.Context(0)
    yield c
    c.close()


def _mat(rng, m, n):
    return rng.integers(0, P, (m, n), dtype=np.int64).astype(np.uint32)


def test_preload_block_round_trip_and_commitments(ctx):
    rng = np.random.default_rng(3)
    mats = [("layers.0.q_proj", _mat(rng, 33, 100)), ("layers.0.down_proj", _mat(rng, 64, 4096)), ("naïve-ünïcode", _mat(rng, 1, 7)),
            ("big", _mat(rng, 4100, 4099)),                     # 67 MB: more than one 64 MiB staging piece
            ("empty", np.zeros((0, 5), np.uint32))]
    block = zw.preload_block(mats) + b"REQUESTS FOLLOW"
    ws = zw.WeightSet(ctx, block)
    assert len(ws) == len(mats) and ws.consumed == len(block) - 15
    assert ws.nbytes == sum(w.size * 4 for _, w in mats)
    for name, w in mats:
        buf, m, n, root = ws.get(name)
        assert (m, n) == w.shape
        if w.size:
            assert np.array_equal(buf.download(), w.reshape(-1))
        assert root == O.commit_weights_fast(w.reshape(-1)), name
    # the resident copy is what a proof runs on: a matmul proof from the device pointer equals the oracle's
    name, w = mats[0]
    buf, m, n, _ = ws.get(name)
    x = rng.integers(0, P, n, dtype=np.int64).astype(np.uint32)
    y = O.matmul_forward(w.reshape(-1), x, m, n)
    assert zp.matmul_forward(ctx, buf, x, m, n).tolist() == y.tolist()
    t, o = zk.Transcript(ctx, b"resident"), O.Transcript(b"resident")
    assert zp.prove_matmul_succinct_ef(buf, x, y, m, n, t) == O.prove_matmul_succinct(o, w.reshape(-1), x, y, m, n, ef=True)
    with pytest.raises(zk.ZkbError):
        ws.get("no such matrix")
    ws.close()


def test_later_matrix_of_the_same_name_replaces_the_earlier_one(ctx):
    rng = np.random.default_rng(4)
    a, b = _mat(rng, 3, 4), _mat(rng, 5, 6)
    ws = zw.WeightSet(ctx, zw.preload_block([("w", a), ("w", b)]))
    assert len(ws) == 1
    buf, m, n, root = ws.get("w")
    assert (m, n) == (5, 6) and np.array_equal(buf.download(), b.reshape(-1)) and root == O.commit_weights_fast(b.reshape(-1))
    ws.close()


def test_preload_refuses_what_the_reference_refuses(ctx):
    rng = np.random.default_rng(5)
    good = zw.preload_block([("a", _mat(rng, 4, 4)), ("b", _mat(rng, 2, 8))])
    cases = {
        "truncated payload": good[:-3],
        "truncated header": good[:6],
        "count over the cap": struct.pack("<I", (1 << 16) + 1) + good[4:],
        "name_len over the cap": struct.pack("<II", 1, (1 << 12) + 1) + b"x" * 8,
        "dimension over the cap": struct.pack("<II", 1, 1) + b"w" + struct.pack("<II", (1 << 24) + 1, 1),
        "element count over the cap": struct.pack("<II", 1, 1) + b"w" + struct.pack("<II", 1 << 16, 1 << 15),
        "name not UTF-8": struct.pack("<II", 1, 2) + b"\xff\xfe" + struct.pack("<II", 1, 1) + struct.pack("<I", 7),
        "overlong UTF-8": struct.pack("<II", 1, 2) + b"\xc0\xaf" + struct.pack("<II", 1, 1) + struct.pack("<I", 7),
    }
    for what, block in cases.items():
        with pytest.raises(zk.ZkbError) as e:
            zw.WeightSet(ctx, block)
        assert e.value.code == 2, what
    # and the context is fine afterwards
    ws = zw.WeightSet(ctx, good)
    assert len(ws) == 2
    ws.close()
