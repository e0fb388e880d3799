"""The C ABI used from compiled code: tests/cabi/caller.c is plain C11 and includes include/zkb200.h as a
foreign-function user would.  Without a GPU: the header compiles as strict C, the program links against
the library and fails loudly when no device exists.  With a GPU: its proofs equal the oracle's."""
import os
import subprocess

import numpy as np
import pytest

from zklm_compile_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = (1 << 31) - 1


@pytest.fixture(scope="module")
def caller(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cabi") / "caller")
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cabi", "caller.c"), "-L", libdir, "-lzkb200", f"-Wl,-rpath,{libdir}", "-o", out], check=True)
    return out


def test_header_is_valid_c_and_the_program_fails_loudly_without_a_gpu(caller):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    r = subprocess.run([caller, "4", "3", "8"], capture_output=True, text=True)
    assert r.returncode == 3 and "no CUDA device" in r.stderr and r.stdout == ""


class Lcg:
    def __init__(self):
        self.s = 12345

    def next(self):
        self.s = (self.s * 1664525 + 1013904223) & 0xFFFFFFFF
        return (self.s >> 1) % P

    def vec(self, n):
        return np.array([self.next() for _ in range(n)], dtype=np.uint32)


@pytest.mark.gpu
@pytest.mark.parametrize("nv,m,n", [(10, 7, 40), (15, 100, 260)])
def test_c_caller_proofs_equal_the_oracle(caller, nv, m, n):
    from oracle import pyoracle as O
    r = subprocess.run([caller, str(nv), str(m), str(n)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = dict(line.split(" ", 1) for line in r.stdout.strip().split("\n"))
    g = Lcg()
    f, gg = g.vec(1 << nv), g.vec(1 << nv)
    tr = O.Transcript(b"c-caller")
    polys, chal, fin = O.prove("product_ef", tr, [f, gg], nv)
    assert got["polys"] == np.asarray(polys, dtype="<u4").tobytes().hex()
    assert got["chal"] == np.asarray(chal, dtype="<u4").tobytes().hex()
    assert got["finals"] == np.concatenate([np.asarray(fin[0]), np.asarray(fin[1])]).astype("<u4").tobytes().hex()
    W, x = g.vec(m * n), g.vec(n)
    y = O.matmul_forward(W, x, m, n)
    assert got["y"] == y.astype("<u4").tobytes().hex()
    assert got["matmul"] == O.prove_matmul_succinct(tr, W, x, y, m, n, ef=True).hex()
    point = g.vec(nv)
    assert got["basefold"] == O.basefold_commit_and_prove(tr, f, point, O.NODE_BLAKE3).hex()
    assert got["verify_other_transcript"] == "0" and got["verify_same_transcript"] == "1"
    assert got["batch"] == O.basefold_batch_prove(O.Transcript(b"c-batch"), [f, gg[:(1 << (nv - 2)) - 3]], [nv, nv - 2]).hex()
    assert got["batch_verify"] == "1"
    table = ((np.arange(256, dtype=np.uint64) * 7 + 1) % 1000 + 1).astype(np.uint32)
    q, k, v = np.zeros(32, np.uint32), np.zeros(32, np.uint32), np.zeros(32, np.uint32)
    for i in range(32):
        q[i] = g.next() % 3; k[i] = g.next() % 3; v[i] = g.next()
    proof, st = O.prove_row_attention(O.Transcript(b"c-attn"), q, k, v, 2, 4, 4, table)
    assert st == 0 and got["attention"] == proof.hex()
    assert got["attention_out"] == O.row_attention_forward(q, k, v, 2, 4, 4, table)[0].astype("<u4").tobytes().hex()
    assert got["attention_verify"] == "1"
