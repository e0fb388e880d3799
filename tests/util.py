"""Shared helpers for the tests: fixture loading and seeded synthetic layers."""
import base64
import json
import os
import zlib

import numpy as np

P = (1 << 31) - 1
HERE = os.path.dirname(os.path.abspath(__file__))


def _unpack_col(b64: str) -> np.ndarray:
    signed = np.frombuffer(zlib.decompress(base64.b64decode(b64)), dtype="<i2").astype(np.int64)
    return np.mod(signed, P).astype(np.uint32)


def load_qwen_golden():
    with open(os.path.join(HERE, "golden", "qwen_forward.json")) as f:
        g = json.load(f)
    g["silu"] = _unpack_col(g["silu_table_out_i16_zlib_b64"])
    g["sigmoid"] = _unpack_col(g["sigmoid_table_out_i16_zlib_b64"])
    return g


def small_table(n_table: int, seed: int = 0):
    """A synthetic table: inputs in table order, outputs a seeded int16-range function."""
    if n_table == 65536:
        signed_in = np.arange(65536, dtype=np.uint16).astype(np.int16).astype(np.int64)
    else:
        signed_in = np.arange(n_table, dtype=np.uint8).astype(np.int8).astype(np.int64)
    out = (signed_in * (3 + seed) // 7 + 11 * seed) % 30000 - 15000
    return np.mod(signed_in, P).astype(np.uint32), np.mod(out, P).astype(np.uint32)


def rand_layer(seed, d_model, d_ff, heads, kv, d_head, v_heads=0, v_d_head=0):
    """Seeded int8-range weights embedded in M31 (negatives as p - |w|) for one Qwen-style layer."""
    rng = np.random.default_rng(seed)
    cfg = dict(d_model=d_model, d_ff=d_ff, num_q_heads=heads, num_kv_heads=kv, d_head=d_head,
               v_num_heads=v_heads, v_d_head=v_d_head)
    q_dim, k_dim = heads * d_head, kv * d_head
    v_dim = (v_heads or kv) * (v_d_head or d_head)
    aod = q_dim if heads != kv else v_dim

    def w(n):
        return np.mod(rng.integers(-127, 128, n), P).astype(np.uint32)

    weights = dict(norm1_gamma=w(d_model), w_q=w(q_dim * d_model), w_k=w(k_dim * d_model), w_v=w(v_dim * d_model),
                   w_o=w(d_model * aod), w_g_proj=w(aod * d_model), norm2_gamma=w(d_model), w_gate=w(d_ff * d_model),
                   w_up=w(d_ff * d_model), w_down=w(d_model * d_ff))
    return cfg, weights, w(d_model)
