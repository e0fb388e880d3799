"""Batch Basefold (basefold.rs:769-1590): the CPU restatement against the reference's own three tests
(basefold.rs:1849-1960: same-size batch round trip, tampered fold root rejected, multi-height round trip) plus
a few more tamperings, both node hashes, and the structure of the bincode image."""
import struct

import numpy as np
import pytest

from oracle import pyoracle as po

P = (1 << 31) - 1


def same_size_polys(k, n, mul, add):
    """basefold.rs:1853-1857 / :1892-1896"""
    return [np.array([((i + seed * 100) * mul + add) % P for i in range(n)], dtype=np.uint32) for seed in range(k)]


def multi_height_polys():
    """basefold.rs:1926-1934"""
    return ([np.array([(i * 17 + 3) % P for i in range(256)], np.uint32), np.array([(i * 31 + 7) % P for i in range(64)], np.uint32),
             np.array([(i * 43 + 11) % P for i in range(16)], np.uint32)], [8, 6, 4])


@pytest.mark.parametrize("kind", [0, 1])
def test_same_size_batch_round_trip_and_tampering(kind):
    polys = same_size_polys(4, 256, 17, 3)
    assert po.basefold_batch_roundtrip(polys, [8] * 4, True, kind) == 1
    polys = same_size_polys(3, 128, 13, 1)
    assert po.basefold_batch_roundtrip(polys, [7] * 3, True, kind) == 1
    for tamper in (1, 2, 3, 5):
        assert po.basefold_batch_roundtrip(polys, [7] * 3, True, kind, tamper) == 0, tamper


@pytest.mark.parametrize("kind", [0, 1])
def test_multi_height_round_trip_and_tampering(kind):
    polys, log_ns = multi_height_polys()
    assert po.basefold_batch_roundtrip(polys, log_ns, False, kind) == 1
    for tamper in (1, 2, 3, 4):
        assert po.basefold_batch_roundtrip(polys, log_ns, False, kind, tamper) == 0, tamper
    # order of the input does not matter for acceptance; two groups of several polynomials each, one size skipped
    rng = np.random.default_rng(2)
    polys = [rng.integers(0, P, n).astype(np.uint32) for n in (16, 200, 64, 256, 50, 9)]
    assert po.basefold_batch_roundtrip(polys, [4, 8, 6, 8, 6, 4], False, kind) == 1


def test_bincode_structure():
    polys, log_ns = multi_height_polys()
    b = po.basefold_batch_prove(po.Transcript(b"multi-height-test"), polys, log_ns)
    k, = struct.unpack_from("<Q", b, 0)
    assert k == 3
    at = 8
    for n, ln in zip((256, 64, 16), log_ns):                   # commitments in input order: root, num_coeffs, log_n
        assert struct.unpack_from("<QQ", b, at + 16) == (n, ln)
        at += 32
    num_polys, n_logs = struct.unpack_from("<QQ", b, at)
    assert (num_polys, n_logs) == (3, 3) and struct.unpack_from("<QQQ", b, at + 16) == (8, 6, 4)
    at += 16 + 24
    assert struct.unpack_from("<Q", b, at)[0] == 3             # roots
    at += 8 + 48 + 16                                          # roots, batched root
    assert struct.unpack_from("<Q", b, at)[0] == 8             # one fold root per variable of the largest polynomial
    # sorted by size whatever the input order: the same three polynomials shuffled give the same proof, permuted commitments
    b2 = po.basefold_batch_prove(po.Transcript(b"multi-height-test"), [polys[2], polys[0], polys[1]], [4, 8, 6])
    assert b2[8 + 96:] == b[8 + 96:]
    assert b2[8:8 + 32] == b[8 + 64:8 + 96] and b2[8 + 32:8 + 64] == b[8:8 + 32]


def test_verify_from_bytes():
    polys, log_ns = multi_height_polys()
    b = po.basefold_batch_prove(po.Transcript(b"v"), polys, log_ns)
    assert po.basefold_batch_verify_bytes(po.Transcript(b"v"), b)[0] == 1
    assert po.basefold_batch_verify_bytes(po.Transcript(b"other"), b)[0] == 0
    assert po.basefold_batch_verify_bytes(po.Transcript(b"v"), b[:-3])[0] == -1
    rejected = 0
    for at in range(8, len(b), 97):
        bad = bytearray(b); bad[at] ^= 1
        rejected += po.basefold_batch_verify_bytes(po.Transcript(b"v"), bytes(bad))[0] != 1
    # what the reference's verifier does not read may change unnoticed: the commitments (only the proof's own roots are absorbed),
    # the final value, values repeated for duplicate positions
    assert rejected > 0.85 * len(range(8, len(b), 97))
