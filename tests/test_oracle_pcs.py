"""CPU checks of the oracle's Merkle tree and Basefold restatements.  The reference holds no
literal vectors for them; its tests are round trips and tamper rejections
(rust/zk_ml_prover/src/proving/pcs.rs:459-530, basefold.rs:1615-1955), repeated here, plus pins
of the primitives against independent libraries (AES through `cryptography`, blake3 through the
`blake3` wheel) and of the table derivation against a direct numpy restatement."""
import numpy as np
import pytest

from oracle import pyoracle as O
from tests.util import P

KINDS = [O.NODE_BLAKE3, O.NODE_AES_MMO]


def test_aes_primitives_match_library():
    from cryptography.hazmat.primitives.ciphers import Cipher, algorithms, modes
    rng = np.random.default_rng(1)
    for _ in range(8):
        key, blk = rng.bytes(16), rng.bytes(16)
        enc = Cipher(algorithms.AES(key), modes.ECB()).encryptor()
        assert O.aes128_encrypt(key, blk) == enc.update(blk) + enc.finalize()
    # FIPS-197 appendix C.1
    key = bytes(range(16))
    blk = bytes.fromhex("00112233445566778899aabbccddeeff")
    assert O.aes128_encrypt(key, blk).hex() == "69c4e0d86a7b0430d8cdb78070b4c55a"


def test_blake3_node_matches_wheel():
    import blake3
    rng = np.random.default_rng(2)
    for _ in range(4):
        l, r = rng.bytes(16), rng.bytes(16)
        assert O.hash_node(l, r, O.NODE_BLAKE3) == blake3.blake3(l + r).digest()[:16]


def test_aes_node_structure():
    # ten rounds keyed L, R, L, ... then feed-forward: not symmetric, and sensitive to both children
    l, r = bytes(range(16)), bytes(range(16, 32))
    a = O.hash_node(l, r, O.NODE_AES_MMO)
    assert a != O.hash_node(r, l, O.NODE_AES_MMO)
    assert a != O.hash_node(l, bytes(16), O.NODE_AES_MMO)
    assert len(a) == 16


@pytest.mark.parametrize("kind", KINDS)
def test_merkle_root_recomputed_by_hand(kind):
    v = np.array([5, 7, 11, 13, 17], np.uint32)        # pads to 8 leaves with zeros (pcs.rs:514-530)
    leaf = lambda x: int(x).to_bytes(4, "little") + bytes(12)
    lv = [leaf(x) for x in list(v) + [0, 0, 0]]
    while len(lv) > 1:
        lv = [O.hash_node(lv[2 * i], lv[2 * i + 1], kind) for i in range(len(lv) // 2)]
    assert O.merkle_root(v, kind) == lv[0]
    # a single value still makes a two-leaf tree
    assert O.merkle_root(np.array([9], np.uint32), kind) == O.hash_node(leaf(9), leaf(0), kind)


@pytest.mark.parametrize("kind", KINDS)
def test_merkle_batch_open_roundtrip_and_tamper(kind):
    rng = np.random.default_rng(3)
    v = rng.integers(0, P, 1000, dtype=np.uint32)
    idx = [3, 3, 2, 999, 1023, 512, 0, 1]                # duplicates, siblings, padding region
    assert O.merkle_batch_roundtrip(v, kind, idx) == 3
    assert O.merkle_batch_roundtrip(v, kind, idx, tamper=1) & 1 == 0
    assert O.merkle_batch_roundtrip(v, kind, idx, tamper=2) & 1 == 0
    blob = O.merkle_batch_open(v, kind, idx)
    n = int.from_bytes(blob[:8], "little")
    assert n == len(idx)
    assert [int.from_bytes(blob[8 + 4 * i: 12 + 4 * i], "little") for i in range(n)] == idx   # caller order kept


def test_basefold_tables_match_numpy_restatement():
    import blake3
    log_n = 6
    seed = blake3.blake3(b"basefold-foldable-code" + log_n.to_bytes(8, "little")).digest()
    total = (1 << log_n) - 1
    raw = np.frombuffer(blake3.blake3(seed).digest(length=4 * total), dtype="<u4").astype(np.int64)
    t_ref = 1 + raw % (P - 1)
    t, w = O.basefold_tables(log_n)
    assert t.tolist() == t_ref.tolist()
    assert all((2 * int(a) * int(b)) % P == 1 for a, b in zip(t, w))


def test_basefold_encode_is_linear_and_folds_to_smaller_code():
    log_n = 5
    rng = np.random.default_rng(4)
    a = rng.integers(0, P, 1 << log_n, dtype=np.uint32)
    b = rng.integers(0, P, 1 << log_n, dtype=np.uint32)
    ea, eb = O.basefold_encode(a, log_n).astype(object), O.basefold_encode(b, log_n).astype(object)
    s = ((a.astype(object) + b.astype(object)) % P).astype(np.uint32)
    assert O.basefold_encode(s, log_n).tolist() == ((ea + eb) % P).tolist()
    # the two halves of the codeword are equal (chunks never cross the middle)
    assert ea[: 1 << log_n].tolist() == ea[1 << log_n:].tolist()


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("n", [1, 2, 5, 64, 300])
def test_basefold_roundtrip(kind, n):
    rng = np.random.default_rng(10 + n)
    c = rng.integers(0, P, n, dtype=np.uint32)
    log_n = 1 if n <= 1 else (n - 1).bit_length()
    pt = rng.integers(0, P, log_n, dtype=np.uint32)
    assert O.basefold_roundtrip(c, pt, kind) == 1
    for tamper in (1, 2, 3, 4):
        assert O.basefold_roundtrip(c, pt, kind, tamper) == 0


def test_basefold_proof_is_deterministic_and_short_point_squeezes():
    rng = np.random.default_rng(5)
    c = rng.integers(0, P, 128, dtype=np.uint32)
    pt = rng.integers(0, P, 7, dtype=np.uint32)
    a = O.basefold_commit_and_prove(O.Transcript(b"x"), c, pt, O.NODE_BLAKE3)
    b = O.basefold_commit_and_prove(O.Transcript(b"x"), c, pt, O.NODE_BLAKE3)
    assert a == b and len(a) > 2000
    assert a != O.basefold_commit_and_prove(O.Transcript(b"x"), c, pt, O.NODE_AES_MMO)
    # root (16) + num_coeffs + log_n, then fold_roots length
    assert int.from_bytes(a[16:24], "little") == 128 and int.from_bytes(a[24:32], "little") == 7
    assert int.from_bytes(a[32:40], "little") == 7
    # a point shorter than log_n: remaining challenges are squeezed (basefold.rs:508-513)
    assert O.basefold_roundtrip(c, pt[:3], O.NODE_BLAKE3) in (-1, 0, 1)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("mode", [O.BIND_BLAKE3, O.BIND_PCS, O.BIND_PCS_FULL])
@pytest.mark.parametrize("m,n", [(4, 4), (5, 7), (16, 12)])
def test_matmul_binding_modes_roundtrip(mode, m, n, kind):
    rng = np.random.default_rng(m * 100 + n)
    w = rng.integers(0, P, m * n, dtype=np.uint32)
    x = rng.integers(0, P, n, dtype=np.uint32)
    y = O.matmul_forward(w, x, m, n)
    plain = O.prove_matmul_succinct(O.Transcript(b"t"), w, x, y, m, n, ef=True)
    with O.features(mode, kind):
        assert O.matmul_succinct_roundtrip(w, x, y, m, n, True)
        assert not O.matmul_succinct_roundtrip(w, x, y, m, n, True, tamper=True)
        a = O.prove_matmul_succinct(O.Transcript(b"t"), w, x, y, m, n, ef=True)
    # the default mode ends with basefold_proof = None; the PCS modes append Some(proof)
    if mode == O.BIND_BLAKE3:
        assert a == plain and a[-1] == 0
    else:
        assert len(a) > len(plain) + 500


@pytest.mark.parametrize("mode", [O.BIND_PCS, O.BIND_PCS_FULL])
def test_qwen_layer_with_basefold_binding_verifies(mode):
    import hashlib
    from tests.util import rand_layer, small_table
    cfg, weights, x = rand_layer(3, 16, 32, 2, 1, 8)
    tin, silu = small_table(65536, 1)
    _, sig = small_table(65536, 2)
    ih = hashlib.sha256(b"in").digest()
    y0, plain, ok0 = O.qwen_layer_prove(cfg, weights, x, silu, sig, 0, ih, verify=True)
    with O.features(mode, O.NODE_BLAKE3):
        y, proof, ok = O.qwen_layer_prove(cfg, weights, x, silu, sig, 0, ih, verify=True)
    assert ok0 and ok and y.tolist() == y0.tolist()
    assert len(proof) > len(plain) + 8 * 500
