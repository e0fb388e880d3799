"""Regenerates tests/golden/qwen_forward.json from the reference's numpy restatement of the
Qwen layer forward pass (tests/reference/transformer.py::qwen_layer_forward), for two small
seeded configurations (a GatedDeltaNet-shape layer with asymmetric V and a GQA layer).

    python tests/golden/make_golden_qwen.py /path/to/reference

The lookup-table output columns the reference builds are stored too, so the consumer needs no
floating-point code to replay the trace.
"""
import base64
import json
import os
import sys
import zlib

import numpy as np


def main(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "tests", "reference"))
    import reference  # type: ignore
    import transformer  # type: ignore

    P = (1 << 31) - 1
    out = {"cases": []}
    scale = 1000
    silu = reference.silu_table(scale)[:, 1].astype(np.int64)
    sigm = reference.sigmoid_table(scale)[:, 1].astype(np.int64)
    out["silu_scale"] = out["sigmoid_scale"] = scale
    # output columns as zlib-compressed little-endian int16 (signed representatives), base64
    def pack(col):
        signed = np.where(col > P // 2, col - P, col).astype(np.int16)
        return base64.b64encode(zlib.compress(signed.astype("<i2").tobytes(), 9)).decode()
    out["silu_table_out_i16_zlib_b64"] = pack(silu)
    out["sigmoid_table_out_i16_zlib_b64"] = pack(sigm)
    configs = [
        dict(d_model=16, d_ff=24, num_q_heads=2, num_kv_heads=2, d_head=4, v_num_heads=4, v_d_head=4),
        dict(d_model=16, d_ff=20, num_q_heads=4, num_kv_heads=2, d_head=4, v_num_heads=0, v_d_head=0),
        dict(d_model=12, d_ff=40, num_q_heads=2, num_kv_heads=2, d_head=8, v_num_heads=0, v_d_head=0),
    ]
    for ci, cfg in enumerate(configs):
        rng = np.random.default_rng(900 + ci)
        dm, dff = cfg["d_model"], cfg["d_ff"]
        q_dim = cfg["num_q_heads"] * cfg["d_head"]
        k_dim = cfg["num_kv_heads"] * cfg["d_head"]
        v_dim = (cfg["v_num_heads"] or cfg["num_kv_heads"]) * (cfg["v_d_head"] or cfg["d_head"])
        aod = q_dim if cfg["num_q_heads"] != cfg["num_kv_heads"] else v_dim

        def w(n):
            return np.mod(rng.integers(-127, 128, n), P).astype(np.uint32)

        weights = dict(norm1_gamma=w(dm), w_q=w(q_dim * dm), w_k=w(k_dim * dm), w_v=w(v_dim * dm), w_o=w(dm * aod),
                       w_g_proj=w(aod * dm), norm2_gamma=w(dm), w_gate=w(dff * dm), w_up=w(dff * dm), w_down=w(dm * dff))
        x = w(dm)
        full = dict(cfg, silu_scale=scale, sigmoid_scale=scale)
        tr = transformer.qwen_layer_forward(x, weights, full)
        case = {"config": cfg, "x": x.tolist(), "weights": {k: v.tolist() for k, v in weights.items()}, "trace": {}}
        for k, v in tr.items():
            case["trace"][k] = np.asarray(v).astype(np.int64).tolist() if isinstance(v, np.ndarray) else int(v)
        out["cases"].append(case)
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "qwen_forward.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("wrote", len(out["cases"]), "cases; keys:", sorted(out["cases"][0]["trace"]))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: %s <path to a checkout of the reference repository>" % sys.argv[0])
    main(sys.argv[1])
