#!/usr/bin/env python
"""Independent pins for what the reference holds no literal vector for: the M31^4 tower and
the byte stream of a product sumcheck with EF challenges.

Everything here is written from the definitions alone, in exact Python integers, and shares no
code with the C++ oracle or the CUDA kernels:

* EF = F_p[i]/(i^2 + 1) [Y]/(Y^2 - (2 + i)), p = 2^31 - 1, coordinates in the reference's wire
  order [re(c0), im(c0), re(c1), im(c1)] (rust/zk_ml_prover/src/proving/sumcheck.rs:19-21, 67-96).
  Products and inverses are computed as polynomial arithmetic modulo the two defining relations;
  the inverse is additionally checked by multiplying back to one.
* The transcript follows rust/zk_ml_prover/src/proving/sumcheck.rs:110-206 with `hashlib.sha256`,
  and `prove_product_ef` follows :1204-1258 literally (widen, per round s0 / s1 / s2, absorb all
  three, squeeze an EF challenge, fold with (1 - r) a + r b).

Output: tests/golden/ef_pins.json.  Run from the repository root: python tests/golden/make_golden_ef.py
"""
import hashlib
import json
import os
import random

P = (1 << 31) - 1


# ---- Complex<M31>: pairs (re, im) with i^2 = -1 ---------------------------------------------
def c_add(a, b):
    return ((a[0] + b[0]) % P, (a[1] + b[1]) % P)


def c_sub(a, b):
    return ((a[0] - b[0]) % P, (a[1] - b[1]) % P)


def c_mul(a, b):
    return ((a[0] * b[0] - a[1] * b[1]) % P, (a[0] * b[1] + a[1] * b[0]) % P)


def c_inv(a):
    n = pow((a[0] * a[0] + a[1] * a[1]) % P, P - 2, P)
    return (a[0] * n % P, (-a[1]) * n % P)


W = (2, 1)  # the non-residue 2 + i: Y^2 = W


# ---- EF: pairs (c0, c1) of complex numbers, element c0 + c1 Y ---------------------------------
def ef(w):
    return ((w[0] % P, w[1] % P), (w[2] % P, w[3] % P))


def words(a):
    return [a[0][0], a[0][1], a[1][0], a[1][1]]


def ef_add(a, b):
    return (c_add(a[0], b[0]), c_add(a[1], b[1]))


def ef_sub(a, b):
    return (c_sub(a[0], b[0]), c_sub(a[1], b[1]))


def ef_mul(a, b):
    # (a0 + a1 Y)(b0 + b1 Y) = a0 b0 + a1 b1 W + (a0 b1 + a1 b0) Y
    return (c_add(c_mul(a[0], b[0]), c_mul(c_mul(a[1], b[1]), W)), c_add(c_mul(a[0], b[1]), c_mul(a[1], b[0])))


def ef_inv(a):
    # 1 / (a0 + a1 Y) = (a0 - a1 Y) / (a0^2 - W a1^2)
    d = c_inv(c_sub(c_mul(a[0], a[0]), c_mul(W, c_mul(a[1], a[1]))))
    return (c_mul(a[0], d), c_mul(c_sub((0, 0), a[1]), d))


ONE, ZERO = ef([1, 0, 0, 0]), ef([0, 0, 0, 0])


# ---- Transcript (sumcheck.rs:110-206) -----------------------------------------------------------
class Transcript:
    def __init__(self, label: bytes):
        self.h = hashlib.sha256(label)

    def absorb(self, v: int):
        self.h.update(int(v).to_bytes(4, "little"))

    def absorb_ef(self, a):
        for w in words(a):
            self.absorb(w)

    def squeeze(self) -> int:
        while True:
            d = self.h.digest()
            self.h = hashlib.sha256(d)
            for c in range(4):
                raw = int.from_bytes(d[8 * c:8 * c + 8], "little")
                if raw < (1 << 64) - 4:
                    return raw % P

    def squeeze_ef(self):
        c = [self.squeeze() for _ in range(4)]
        return ef(c)


# ---- prove_product_ef (sumcheck.rs:1204-1258) -----------------------------------------------------
def prove_product_ef(f, g, num_vars, tr):
    fe = [ef([v, 0, 0, 0]) for v in f]
    ge = [ef([v, 0, 0, 0]) for v in g]
    size, polys, chal = len(fe), [], []
    for _ in range(num_vars):
        half = size // 2
        s0 = s1 = s2 = ZERO
        for j in range(half):
            f0, f1, g0, g1 = fe[j], fe[j + half], ge[j], ge[j + half]
            s0 = ef_add(s0, ef_mul(f0, g0))
            s1 = ef_add(s1, ef_mul(f1, g1))
            f2, g2 = ef_sub(ef_add(f1, f1), f0), ef_sub(ef_add(g1, g1), g0)
            s2 = ef_add(s2, ef_mul(f2, g2))
        tr.absorb_ef(s0); tr.absorb_ef(s1); tr.absorb_ef(s2)
        r = tr.squeeze_ef()
        omr = ef_sub(ONE, r)
        for j in range(half):
            fe[j] = ef_add(ef_mul(omr, fe[j]), ef_mul(r, fe[j + half]))
            ge[j] = ef_add(ef_mul(omr, ge[j]), ef_mul(r, ge[j + half]))
        polys.append([words(s0), words(s2)])
        chal.append(words(r))
        size = half
    return polys, chal, words(fe[0]), words(ge[0])


def main():
    rnd = random.Random(20251125)
    ef_cases = []
    specials = [[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1], [P - 1, P - 1, P - 1, P - 1], [2, 1, 0, 0], [0, 0, P - 1, 1]]
    operands = specials + [[rnd.randrange(P) for _ in range(4)] for _ in range(24)]
    for i, a in enumerate(operands):
        b = operands[(i * 7 + 3) % len(operands)]
        A, B = ef(a), ef(b)
        inv = ef_inv(A)
        assert ef_mul(A, inv) == ONE
        ef_cases.append({"a": a, "b": b, "mul": words(ef_mul(A, B)), "inv_a": words(inv)})
    # Y^2 = 2 + i and i^2 = -1, stated as products of basis elements
    assert words(ef_mul(ef([0, 0, 1, 0]), ef([0, 0, 1, 0]))) == [2, 1, 0, 0]
    assert words(ef_mul(ef([0, 1, 0, 0]), ef([0, 1, 0, 0]))) == [P - 1, 0, 0, 0]

    transcripts = []
    for label, ops in [(b"", [("squeeze", 3)]), (b"pin", [("absorb", [1, 2, P - 1]), ("squeeze", 2), ("absorb", [7]), ("squeeze", 5)]),
                       (b"x" * 70, [("absorb", list(range(40))), ("squeeze", 4)])]:
        t, out = Transcript(label), []
        for op, arg in ops:
            if op == "absorb":
                for v in arg:
                    t.absorb(v)
            else:
                out.append([t.squeeze() for _ in range(arg)])
        transcripts.append({"label": label.decode(), "ops": [[op, arg] for op, arg in ops], "squeezed": out})

    sumchecks = []
    # the reference's own tiny case first: f = [3, 5], g = [2, 4], claimed sum 26 (sumcheck.rs:1649-1661)
    cases = [(1, [3, 5], [2, 4])]
    for nv in (1, 2, 3, 5):
        cases.append((nv, [rnd.randrange(P) for _ in range(1 << nv)], [rnd.randrange(P) for _ in range(1 << nv)]))
    cases.append((2, [P - 1] * 4, [P - 1, 0, 1, P - 2]))
    for nv, f, g in cases:
        polys, chal, fs, gs = prove_product_ef(f, g, nv, Transcript(b"ef-pin"))
        sumchecks.append({"num_vars": nv, "f": f, "g": g, "label": "ef-pin", "round_polys": polys, "challenges": chal, "f_at_s": fs,
                          "g_at_s": gs})
    assert (sumchecks[0]["round_polys"][0][0][0] + (5 * 4)) % P == 26 % P          # s0 + s1 = 26

    out = {"p": P, "ef_cases": ef_cases, "transcripts": transcripts, "product_ef": sumchecks}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ef_pins.json")
    with open(path, "w") as fh:
        json.dump(out, fh, separators=(",", ":"))
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
