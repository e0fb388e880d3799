"""Host-side lookup-table builders (f64 math stays on the host, as in the reference).

Follows rust/zk_ml_prover/src/proving/lookup.rs:122-253 and
rust/zk_ml_prover/src/field/common.rs:57-72: entry `raw` (0..65535) has input
`raw as i16` and output `quantize_i16(f(input / scale), scale)` with Rust's `f64::round`
(half away from zero) and saturation; both are embedded in M31 (negatives as p - |v|).
Only the output column is returned: the input column is a fixed function of the index.
"""
from __future__ import annotations

import numpy as np

P = (1 << 31) - 1


def _inputs_i16() -> np.ndarray:
    return np.arange(65536, dtype=np.uint16).astype(np.int16).astype(np.float64)


def quantize_i16(values: np.ndarray, scale: float) -> np.ndarray:
    v = values * scale
    r = np.sign(v) * np.floor(np.abs(v) + 0.5)          # f64::round
    r = np.where(np.isnan(r), 0.0, r)
    return np.clip(r, -32768.0, 32767.0).astype(np.int64)


def i16_to_field(v: np.ndarray) -> np.ndarray:
    return np.mod(np.asarray(v, dtype=np.int64), P).astype(np.uint32)


def table_inputs(n_table: int = 65536) -> np.ndarray:
    """Input column in table order (i16_to_field(raw as i16), or i8 for 256-entry tables)."""
    if n_table == 65536:
        return i16_to_field(np.arange(65536, dtype=np.uint16).astype(np.int16))
    return i16_to_field(np.arange(n_table, dtype=np.uint8).astype(np.int8))


def build_sigmoid_table(scale: int) -> np.ndarray:
    x = _inputs_i16() / float(scale)
    with np.errstate(over="ignore"):
        y = 1.0 / (1.0 + np.exp(-x))
    return i16_to_field(quantize_i16(y, float(scale)))


def build_silu_table(scale: int) -> np.ndarray:
    x = _inputs_i16() / float(scale)
    with np.errstate(over="ignore"):
        y = x * (1.0 / (1.0 + np.exp(-x)))
    return i16_to_field(quantize_i16(y, float(scale)))


def build_exp_table(scale: int) -> np.ndarray:
    x = _inputs_i16() / float(scale)
    with np.errstate(over="ignore"):
        y = np.exp(x)
    return i16_to_field(quantize_i16(y, float(scale)))


def build_gelu_table(scale: int) -> np.ndarray:
    """rust/zk_ml_prover/src/proving/gelu.rs:23-27: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))."""
    x = _inputs_i16() / float(scale)
    y = 0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3)))
    return i16_to_field(quantize_i16(y, float(scale)))


def requantize_to_i16_field(values) -> np.ndarray:
    """rust/zk_ml_prover/src/transformer/mod.rs:293-324: centre the field values, scale so that the
    largest magnitude maps to 32767 (integer division rounding half away from zero, truncating
    like Rust's `/`), clamp to i16, embed in M31.  The reference's Python drivers supply these
    requantised pairs to the prover (forward.rs:161-201), so this is host-side statement logic."""
    P = (1 << 31) - 1
    u = np.ascontiguousarray(values, dtype=np.uint32).astype(np.int64)
    s = np.where(u > P // 2, u - P, u)
    max_abs = max(int(np.max(np.abs(s))) if s.size else 1, 1)
    if max_abs <= 32767:
        scaled = s
    else:
        half = max_abs // 2
        num = np.where(s >= 0, s * 32767 + half, s * 32767 - half)
        scaled = np.sign(num) * (np.abs(num) // max_abs)          # truncation toward zero
    scaled = np.clip(scaled, -32768, 32767)
    return np.mod(scaled, P).astype(np.uint32)
