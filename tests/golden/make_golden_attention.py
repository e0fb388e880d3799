"""Regenerates tests/golden/attention_forward.json from the reference's own numpy restatement of row attention.

Run in a checkout that has the reference mounted:
    python tests/golden/make_golden_attention.py /path/to/reference
It imports tests/reference/{attention,reference}.py from the reference tree (`attention_full`, the cross-language reference for
`prove_row_attention`'s forward computation at seq_len >= 2, and `exp_table`) and records seeded inputs with their outputs.
The fixtures, not the reference, travel with this repository.
"""
import hashlib
import json
import os
import sys

import numpy as np


def main(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "tests", "reference"))
    import attention  # type: ignore
    import reference  # type: ignore

    P = (1 << 31) - 1
    rng = np.random.default_rng(20251126)
    out = {"cases": [], "exp_tables": {}}
    for scale in (100, 1000):
        t = np.asarray(reference.exp_table(scale))
        # the table is 65536 rows of (input, output); the output column in table order and a digest of the whole table
        out["exp_tables"][str(scale)] = {"rows": int(t.shape[0]), "sha256_outputs_le_u32": hashlib.sha256(t[:, 1].astype("<u4").tobytes()).hexdigest(),
                                         "sha256_inputs_le_u32": hashlib.sha256(t[:, 0].astype("<u4").tobytes()).hexdigest(),
                                         "first_outputs": [int(x) for x in t[:8, 1]], "last_outputs": [int(x) for x in t[-8:, 1]]}
    for (nh, s, d, lo, hi, scale) in [(2, 4, 4, -3, 4, 100), (1, 8, 3, -4, 5, 100), (3, 5, 2, -9, 10, 100), (2, 16, 8, -2, 3, 1000), (1, 2, 1, -10, 11, 100)]:
        n = nh * s * d
        q = np.mod(rng.integers(lo, hi, n), P).astype(np.uint32)
        k = np.mod(rng.integers(lo, hi, n), P).astype(np.uint32)
        v = rng.integers(0, P, n).astype(np.uint32)
        o = attention.attention_full(q, k, v, nh, s, d, scale)
        out["cases"].append({"num_heads": nh, "seq_len": s, "d_head": d, "exp_scale": scale, "q": q.tolist(), "k": k.tolist(), "v": v.tolist(),
                             "out": np.asarray(o, dtype=np.uint32).tolist()})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_forward.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
