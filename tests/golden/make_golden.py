"""Regenerates tests/golden/m31_mle.json from the reference's own numpy restatement.

Run in a checkout that has the reference mounted:
    python tests/golden/make_golden.py /path/to/reference
It imports tests/reference/{m31,mle}.py from the reference tree (its cross-language
reference for the Rust field / MLE helpers) and records seeded input/output vectors.
The fixtures, not the reference, travel with this repository.
"""
import json
import os
import sys

import numpy as np


def main(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "tests", "reference"))
    import m31  # type: ignore
    import mle  # type: ignore

    rng = np.random.default_rng(20251125)
    P = m31.M31
    out = {}
    a = rng.integers(0, P, size=64, dtype=np.int64)
    b = rng.integers(0, P, size=64, dtype=np.int64)
    a[:4] = [0, 1, P - 1, P - 2]
    b[:4] = [P - 1, P - 1, P - 1, 2]
    out["a"] = a.tolist()
    out["b"] = b.tolist()
    out["mul"] = m31.mul(a, b).tolist()
    out["add"] = m31.add(a, b).tolist()
    out["sub"] = m31.sub(a, b).tolist()
    nz = np.where(a == 0, 1, a)
    out["inv_in"] = nz.tolist()
    out["inv"] = m31.inv(nz).tolist()
    out["is_qr"] = [bool(x) for x in m31.is_qr(a)]
    sq = m31.mul(a, a)
    out["sqrt_in"] = sq.tolist()
    out["sqrt"] = m31.mod_sqrt(sq).tolist()
    signed = rng.integers(-(1 << 40), 1 << 40, size=32, dtype=np.int64)
    out["signed"] = signed.tolist()
    out["from_signed"] = m31.from_signed(signed).tolist()
    out["to_signed"] = m31.to_signed(m31.from_signed(signed)).tolist()
    cases = []
    for k in range(0, 9):
        tab = rng.integers(0, P, size=1 << k, dtype=np.int64)
        pt = rng.integers(0, P, size=k, dtype=np.int64)
        cases.append({
            "k": k,
            "table": tab.tolist(),
            "point": pt.tolist(),
            "mle": int(mle.mle_evaluate(tab, pt)) if k > 0 else int(tab[0]),
            "eq": mle.eq_evals(pt).tolist(),
        })
    out["mle_cases"] = cases
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "m31_mle.json"), "w") as f:
        json.dump(out, f)
    print("wrote", len(cases), "mle cases")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: %s <path to a checkout of the reference repository>" % sys.argv[0])
    main(sys.argv[1])
