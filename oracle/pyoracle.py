"""ctypes loader for the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only the tests, the smoke check and the CPU-baseline leg of the benchmark import this.
The shipped package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

u32p = C.POINTER(C.c_uint32)
u8p = C.POINTER(C.c_uint8)


def build() -> str:
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    return os.path.join(_HERE, "libzkoracle.so")


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libzkoracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _LIB.zko_tr_new.restype = C.c_void_p
        _LIB.zko_tr_squeeze.restype = C.c_uint32
        _LIB.zko_mle_evaluate.restype = C.c_uint32
        _LIB.zko_from_field.restype = C.c_int64
        _LIB.zko_mod_sqrt.restype = C.c_uint32
    return _LIB


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(u32p)


def _u8(b: bytes):
    arr = (C.c_uint8 * max(len(b), 1)).from_buffer_copy(b if len(b) else b"\0")
    return arr


def sha256(b: bytes) -> bytes:
    out = (C.c_uint8 * 32)()
    lib().zko_sha256(_u8(b), C.c_size_t(len(b)), out)
    return bytes(out)


def blake3(b: bytes, n: int = 32) -> bytes:
    out = (C.c_uint8 * n)()
    lib().zko_blake3(_u8(b), C.c_size_t(len(b)), out, C.c_size_t(n))
    return bytes(out)


def hash_values(v) -> bytes:
    a, p = _u32(v)
    out = (C.c_uint8 * 32)()
    lib().zko_hash_values(p, C.c_size_t(a.size), out)
    return bytes(out)


def f_mul(a, b):
    o = C.c_uint32()
    lib().zko_f_mul(C.c_uint32(a), C.c_uint32(b), C.byref(o))
    return o.value


def f_inv(a):
    o = C.c_uint32()
    lib().zko_f_inv(C.c_uint32(a), C.byref(o))
    return o.value


def ef_mul(a, b):
    a_, pa = _u32(a)
    b_, pb = _u32(b)
    o = np.zeros(4, np.uint32)
    lib().zko_ef_mul(pa, pb, o.ctypes.data_as(u32p))
    return o


def ef_inv(a):
    a_, pa = _u32(a)
    o = np.zeros(4, np.uint32)
    lib().zko_ef_inv(pa, o.ctypes.data_as(u32p))
    return o


def to_field(x: int) -> int:
    o = C.c_uint32()
    lib().zko_to_field(C.c_int64(x), C.byref(o))
    return o.value


def from_field(x: int) -> int:
    return lib().zko_from_field(C.c_uint32(x))


class Transcript:
    """Mirror of the reference `Transcript` (rust/zk_ml_prover/src/proving/sumcheck.rs:110-206)."""

    def __init__(self, label: bytes):
        self.h = C.c_void_p(lib().zko_tr_new(_u8(label), C.c_size_t(len(label))))

    def __del__(self):
        if getattr(self, "h", None):
            lib().zko_tr_free(self.h)
            self.h = None

    def absorb(self, v: int):
        lib().zko_tr_absorb_u32(self.h, C.c_uint32(v))

    def absorb_many(self, vs):
        a, p = _u32(vs)
        lib().zko_tr_absorb_many(self.h, p, C.c_size_t(a.size))

    def absorb_bytes(self, b: bytes):
        lib().zko_tr_absorb_bytes(self.h, _u8(b), C.c_size_t(len(b)))

    def squeeze(self) -> int:
        return lib().zko_tr_squeeze(self.h)

    def squeeze_ef(self):
        o = np.zeros(4, np.uint32)
        lib().zko_tr_squeeze_ef(self.h, o.ctypes.data_as(u32p))
        return o


def eq_evals(r):
    a, p = _u32(r)
    out = np.zeros(1 << a.size, np.uint32)
    lib().zko_eq_evals(p, C.c_size_t(a.size), out.ctypes.data_as(u32p))
    return out


def eq_evals_ef(r):
    a, p = _u32(r)
    k = a.size // 4
    out = np.zeros((1 << k, 4), np.uint32)
    lib().zko_eq_evals_ef(p, C.c_size_t(k), out.ctypes.data_as(u32p))
    return out


def mle_evaluate(ev, pt) -> int:
    a, pa = _u32(ev)
    b, pb = _u32(pt)
    return lib().zko_mle_evaluate(pa, C.c_size_t(a.size), pb, C.c_size_t(b.size))


def mle_evaluate_ef(ev, pt):
    a, pa = _u32(ev)
    b, pb = _u32(pt)
    o = np.zeros(4, np.uint32)
    lib().zko_mle_evaluate_ef(pa, C.c_size_t(a.size), pb, C.c_size_t(b.size // 4), o.ctypes.data_as(u32p))
    return o


def mle_evaluate_efef(ev, pt):
    a, pa = _u32(ev)
    b, pb = _u32(pt)
    o = np.zeros(4, np.uint32)
    lib().zko_mle_evaluate_efef(pa, C.c_size_t(a.size // 4), pb, C.c_size_t(b.size // 4), o.ctypes.data_as(u32p))
    return o


# name -> (number of input tables, input widths (1 = base, 4 = EF), stored evals per round, output width)
SUMCHECKS = {
    "product": ("zko_prove_product", (1, 1), 3, 1),
    "triple": ("zko_prove_triple", (1, 1, 1), 4, 1),
    "product_ones": ("zko_prove_product_ones", (1,), 2, 1),
    "product_ef": ("zko_prove_product_ef", (1, 1), 2, 4),
    "product_ef_full": ("zko_prove_product_ef_full", (4, 4), 3, 4),
    "product_ef_mixed": ("zko_prove_product_ef_mixed", (4, 1), 3, 4),
    "triple_ef_full": ("zko_prove_triple_ef_full", (4, 4, 4), 3, 4),
    "product_ones_ef_full": ("zko_prove_product_ones_ef_full", (4,), 2, 4),
}


def prove(kind: str, tr: Transcript, tables, num_vars: int):
    """Run one sumcheck prover; returns (round_polys[nv, epr*w], challenges[nv, w], finals[k, w])."""
    fn, widths, epr, w = SUMCHECKS[kind]
    ptrs = []
    keep = []
    for t in tables:
        a, p = _u32(t)
        keep.append(a)
        ptrs.append(p)
    nfin = max(2, len(widths))
    polys = np.zeros((num_vars, epr * w), np.uint32)
    chal = np.zeros((num_vars, w), np.uint32)
    fin = np.zeros((nfin, w), np.uint32)
    getattr(lib(), fn)(tr.h, *ptrs, C.c_size_t(num_vars), polys.ctypes.data_as(u32p),
                       chal.ctypes.data_as(u32p), fin.ctypes.data_as(u32p))
    return polys, chal, fin


def verify(kind: str, tr: Transcript, claimed, polys, chal, fin) -> bool:
    """Verifier restatement for the matching prover kind (challenges may be an empty array)."""
    _, widths, epr, w = SUMCHECKS[kind]
    polys, pp = _u32(polys)
    chal, pc = _u32(chal)
    fin, pf = _u32(fin)
    nv = polys.shape[0]
    nchal = chal.size // w
    triple = kind.startswith("triple")
    if w == 1:
        fn = lib().zko_verify_triple if triple else lib().zko_verify_product
        return bool(fn(tr.h, C.c_uint32(int(claimed)), pp, C.c_size_t(nv), C.c_size_t(epr), pc, C.c_size_t(nchal), pf))
    cl, pcl = _u32(claimed)
    fn = lib().zko_verify_triple_ef if triple else lib().zko_verify_product_ef
    return bool(fn(tr.h, pcl, pp, C.c_size_t(nv), C.c_size_t(epr), pc, C.c_size_t(nchal), pf))


# ------------------------------------------------------------------------------------------
# protocol-level entry points (proofs come back as bincode bytes)
# ------------------------------------------------------------------------------------------
def _bytes_call(fn, *args, cap=1 << 22):
    buf = (C.c_uint8 * cap)()
    fn.restype = C.c_size_t
    n = fn(*args, buf, C.c_size_t(cap))
    if n > cap:
        return _bytes_call(fn, *args, cap=n)
    return bytes(buf[:n])


def commit_weights_fast(w) -> bytes:
    a, p = _u32(w)
    out = (C.c_uint8 * 32)()
    lib().zko_commit_weights_fast(p, C.c_size_t(a.size), out)
    return bytes(out)


def matmul_forward(w, x, m, n):
    W, pw = _u32(w)
    X, px = _u32(x)
    y = np.zeros(m, np.uint32)
    lib().zko_matmul_forward(pw, px, C.c_size_t(m), C.c_size_t(n), y.ctypes.data_as(u32p))
    return y


def _log2_ceil(n):
    return 1 if n <= 1 else (n - 1).bit_length()


def fold_eq_matvec(w, m, n, r):
    W, pw = _u32(w)
    R, pr = _u32(r)
    out = np.zeros(1 << _log2_ceil(n), np.uint32)
    lib().zko_fold_eq_matvec(pw, C.c_size_t(m), C.c_size_t(n), pr, C.c_size_t(R.size), out.ctypes.data_as(u32p))
    return out


def fold_eq_matvec_ef(w, m, n, r):
    W, pw = _u32(w)
    R, pr = _u32(r)
    out = np.zeros((1 << _log2_ceil(n), 4), np.uint32)
    lib().zko_fold_eq_matvec_ef(pw, C.c_size_t(m), C.c_size_t(n), pr, C.c_size_t(R.size // 4), out.ctypes.data_as(u32p))
    return out


def prove_matmul_succinct(tr, w, x, y, m, n, ef=False) -> bytes:
    W, pw = _u32(w); X, px = _u32(x); Y, py = _u32(y)
    fn = lib().zko_prove_matmul_succinct_ef if ef else lib().zko_prove_matmul_succinct
    return _bytes_call(fn, tr.h, pw, px, py, C.c_size_t(m), C.c_size_t(n))


def matmul_succinct_roundtrip(w, x, y, m, n, ef, tamper=False) -> bool:
    W, pw = _u32(w); X, px = _u32(x); Y, py = _u32(y)
    return bool(lib().zko_matmul_succinct_roundtrip(pw, px, py, C.c_size_t(m), C.c_size_t(n), C.c_int(int(ef)), C.c_int(int(tamper))))


def prove_mle_eval_bound(tr, w, point, label: bytes, ef=True):
    W, pw = _u32(w); Pt, pp = _u32(point)
    k = Pt.size // 4 if ef else Pt.size
    claimed = np.zeros(4, np.uint32)
    fn = lib().zko_prove_mle_eval_ef_base_bound if ef else lib().zko_prove_mle_eval_bound
    fn.restype = C.c_size_t
    cap = 1 << 20
    buf = (C.c_uint8 * cap)()
    n = fn(tr.h, pw, C.c_size_t(W.size), pp, C.c_size_t(k), _u8(label), C.c_size_t(len(label)), buf, C.c_size_t(cap),
           claimed.ctypes.data_as(u32p))
    return bytes(buf[:n]), (claimed if ef else int(claimed[0]))


def prove_elementwise_ef(tr, a, b, c, point, add: bool) -> bytes:
    A, pa = _u32(a); B, pb = _u32(b); Cc, pc = _u32(c); Pt, pp = _u32(point)
    fn = lib().zko_prove_add_ef if add else lib().zko_prove_hadamard_ef
    return _bytes_call(fn, tr.h, pa, pb, pc, C.c_size_t(A.size), pp, C.c_size_t(Pt.size // 4))


def elementwise_roundtrip(a, b, c, add: bool, tamper=False) -> bool:
    A, pa = _u32(a); B, pb = _u32(b); Cc, pc = _u32(c)
    return bool(lib().zko_elementwise_roundtrip(pa, pb, pc, C.c_size_t(A.size), C.c_int(int(add)), C.c_int(int(tamper))))


def rmsnorm_forward(x, gamma):
    X, px = _u32(x); G, pg = _u32(gamma)
    out = np.zeros(X.size, np.uint32); xu = np.zeros(X.size, np.uint32)
    lib().zko_rmsnorm_forward.restype = C.c_int32
    d = lib().zko_rmsnorm_forward(px, pg, C.c_size_t(X.size), out.ctypes.data_as(u32p), xu.ctypes.data_as(u32p))
    return out, xu, d


def requantize(v):
    V, pv = _u32(v)
    out = np.zeros(V.size, np.uint32)
    lib().zko_requantize(pv, C.c_size_t(V.size), out.ctypes.data_as(u32p))
    return out


def prove_rmsnorm_ef(tr, x, gamma, y, delta) -> bytes:
    X, px = _u32(x); G, pg = _u32(gamma); Y, py = _u32(y)
    return _bytes_call(lib().zko_prove_rmsnorm_ef, tr.h, px, pg, py, C.c_size_t(X.size), C.c_int32(delta))


def rmsnorm_roundtrip(x, gamma, y, delta, tamper=False) -> bool:
    X, px = _u32(x); G, pg = _u32(gamma); Y, py = _u32(y)
    return bool(lib().zko_rmsnorm_roundtrip(px, pg, py, C.c_size_t(X.size), C.c_int32(delta), C.c_int(int(tamper))))


def prove_lookup_ef(tr, table_out, inputs, outputs):
    """Returns (proof bytes, status): status 3 = LogUp identity failed, 4 = alpha collision."""
    T, pt = _u32(table_out); I, pi = _u32(inputs); O, po = _u32(outputs)
    st = C.c_int()
    cap = 1 << 22
    buf = (C.c_uint8 * cap)()
    lib().zko_prove_lookup_ef.restype = C.c_size_t
    n = lib().zko_prove_lookup_ef(tr.h, pt, C.c_size_t(T.size), pi, po, C.c_size_t(I.size), buf, C.c_size_t(cap), C.byref(st))
    return bytes(buf[:n]), st.value


def lookup_roundtrip(table_out, inputs, outputs, tamper=False) -> bool:
    T, pt = _u32(table_out); I, pi = _u32(inputs); O, po = _u32(outputs)
    return bool(lib().zko_lookup_roundtrip(pt, C.c_size_t(T.size), pi, po, C.c_size_t(I.size), C.c_int(int(tamper))))


WEIGHT_NAMES = ["norm1_gamma", "w_q", "w_k", "w_v", "w_o", "w_g_proj", "norm2_gamma", "w_gate", "w_up", "w_down"]
DIM_NAMES = ["d_model", "d_ff", "num_q_heads", "num_kv_heads", "d_head", "v_num_heads", "v_d_head"]


def qwen_layer_prove(config: dict, weights: dict, x, silu_out, sigmoid_out, layer_idx: int, input_hash: bytes, verify=False):
    """Forward + prove one layer; returns (y, proof bytes, accepted or None)."""
    dims = (C.c_uint64 * 7)(*[int(config.get(k, 0)) for k in DIM_NAMES])
    keep = [np.ascontiguousarray(weights[k], dtype=np.uint32) for k in WEIGHT_NAMES]
    wp = (u32p * 10)(*[a.ctypes.data_as(u32p) for a in keep])
    X, px = _u32(x); S, ps = _u32(silu_out); G, pg = _u32(sigmoid_out)
    y = np.zeros(int(config["d_model"]), np.uint32)
    acc = C.c_int(-1)
    cap = 1 << 24
    buf = (C.c_uint8 * cap)()
    lib().zko_qwen_layer_prove.restype = C.c_size_t
    n = lib().zko_qwen_layer_prove(dims, wp, px, ps, pg, C.c_size_t(S.size), C.c_uint32(layer_idx), _u8(input_hash),
                                   y.ctypes.data_as(u32p), buf, C.c_size_t(cap), C.c_int(int(verify)), C.byref(acc))
    return y, bytes(buf[:n]), (bool(acc.value) if verify else None)


class QwenLayer:
    """A layer whose weights are converted and committed once (what the reference's server does at
    load time); `prove` then costs forward + prove only, which is what the reference's
    prove_time_ms covers (pipeline/mod.rs:224-229)."""

    def __init__(self, config: dict, weights: dict, silu_out, sigmoid_out):
        dims = (C.c_uint64 * 7)(*[int(config.get(k, 0)) for k in DIM_NAMES])
        keep = [np.ascontiguousarray(weights[k], dtype=np.uint32) for k in WEIGHT_NAMES]
        wp = (u32p * 10)(*[a.ctypes.data_as(u32p) for a in keep])
        S, ps = _u32(silu_out); G, pg = _u32(sigmoid_out)
        lib().zko_qwen_layer_new.restype = C.c_void_p
        self.h = C.c_void_p(lib().zko_qwen_layer_new(dims, wp, ps, pg, C.c_size_t(S.size)))
        self.d_model = int(config["d_model"])

    def __del__(self):
        if getattr(self, "h", None):
            lib().zko_qwen_layer_free(self.h)
            self.h = None

    def verify_bytes(self, x, layer_idx, input_hash, y_expected, proof: bytes) -> int:
        """The restated verify_qwen_layer_ef_indexed on proof bytes: 1 accept, 0 reject, -1 undecodable."""
        X, px = _u32(x); Y, py = _u32(y_expected)
        return int(lib().zko_qwen_layer_verify_bytes_h(self.h, px, C.c_uint32(layer_idx), _u8(input_hash), py, _u8(proof), C.c_size_t(len(proof))))

    def prove(self, x, layer_idx: int, input_hash: bytes, verify=False):
        """Forward + prove; returns (y, proof bytes, accepted or None)."""
        X, px = _u32(x)
        y = np.zeros(self.d_model, np.uint32)
        acc = C.c_int(-1)
        cap = 1 << 24
        buf = (C.c_uint8 * cap)()
        lib().zko_qwen_layer_prove_h.restype = C.c_size_t
        n = lib().zko_qwen_layer_prove_h(self.h, px, C.c_uint32(layer_idx), _u8(input_hash), y.ctypes.data_as(u32p), buf, C.c_size_t(cap),
                                         C.c_int(int(verify)), C.byref(acc))
        return y, bytes(buf[:n]), (bool(acc.value) if verify else None)


def _layer_forward(self, x):
    """qwen_forward_indexed alone (keeps the trace for prove_trace); returns the layer output."""
    X, px = _u32(x)
    y = np.zeros(self.d_model, np.uint32)
    lib().zko_qwen_layer_forward_h(self.h, px, y.ctypes.data_as(u32p))
    return y


def _layer_prove_trace(self, layer_idx: int, input_hash: bytes) -> bytes:
    """prove_qwen_layer_precommitted_ef on the trace of the last forward."""
    return _bytes_call(lib().zko_qwen_layer_prove_trace_h, self.h, C.c_uint32(layer_idx), _u8(input_hash), cap=1 << 22)


QwenLayer.forward = _layer_forward
QwenLayer.prove_trace = _layer_prove_trace


class OpList:
    """The reference's op-list mode (pipeline/forward.rs + pipeline/prove.rs:191-648, oracle/oplist.hpp):
    ops are added in forward order; `prove(x)` runs the forward pass and returns
    bincode(Vec<SerializedLayerProof>) with the proofs in the reference's (reverse) push order."""

    def __init__(self):
        lib().zko_oplist_new.restype = C.c_void_p
        self.h = C.c_void_p(lib().zko_oplist_new())
        self.n_ops = 0

    def __del__(self):
        if getattr(self, "h", None):
            lib().zko_oplist_free(self.h)
            self.h = None

    def linear(self, name, w, b, m, n):
        W, pw = _u32(w)
        if b is None:
            lib().zko_oplist_linear(self.h, name.encode(), pw, None, C.c_size_t(m), C.c_size_t(n))
        else:
            B, pb = _u32(b)
            lib().zko_oplist_linear(self.h, name.encode(), pw, pb, C.c_size_t(m), C.c_size_t(n))
        self.n_ops += 1

    def simple(self, kind, name, aux=""):
        """relu, attention (seq_len 1), passthrough, save (aux = save_name), add_saved (aux = add_name)."""
        lib().zko_oplist_simple(self.h, kind.encode(), name.encode(), aux.encode())
        self.n_ops += 1

    def layernorm(self, name, gamma, beta):
        G, pg = _u32(gamma); B, pb = _u32(beta)
        lib().zko_oplist_layernorm(self.h, name.encode(), pg, pb, C.c_size_t(G.size))
        self.n_ops += 1

    def gelu(self, name, inputs, outputs, table_out):
        I, pi = _u32(inputs); Oo, po = _u32(outputs); T, pt = _u32(table_out)
        lib().zko_oplist_gelu(self.h, name.encode(), pi, po, C.c_size_t(I.size), pt, C.c_size_t(T.size))
        self.n_ops += 1

    def attention(self, name, num_heads, seq_len, d_head, table_out, k_values=None, v_values=None, num_kv_heads=0):
        """"attention" at seq_len >= 2: the activation is Q | K | V, or Q alone with K and V given here."""
        T, pt = _u32(table_out)
        pk = pv = None
        if k_values is not None:
            K, pk = _u32(k_values); V, pv = _u32(v_values)
        lib().zko_oplist_attention(self.h, name.encode(), C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len), C.c_size_t(d_head), pt,
                                   C.c_size_t(T.size), pk, pv)
        self.n_ops += 1

    def set_input(self, name, values):
        V, pv = _u32(values)
        lib().zko_oplist_set_input(self.h, name.encode(), pv, C.c_size_t(V.size))
        self.n_ops += 1

    def forward(self, x, upto=None):
        """Activation after op `upto` (default: the last one)."""
        X, px = _u32(x)
        upto = self.n_ops - 1 if upto is None else upto
        cap = 1 << 20
        out = np.zeros(cap, np.uint32)
        lib().zko_oplist_forward.restype = C.c_size_t
        n = lib().zko_oplist_forward(self.h, px, C.c_size_t(X.size), C.c_size_t(upto), out.ctypes.data_as(u32p), C.c_size_t(cap))
        return out[:n].copy()

    def prove(self, x) -> bytes:
        X, px = _u32(x)
        return _bytes_call(lib().zko_oplist_prove, self.h, px, C.c_size_t(X.size), cap=1 << 27)


def layernorm_sqr_roundtrip(x, gamma, beta, tamper=0) -> bool:
    X, px = _u32(x); G, pg = _u32(gamma); B, pb = _u32(beta)
    return bool(lib().zko_layernorm_sqr_roundtrip(px, pg, pb, C.c_size_t(X.size), C.c_int(tamper)))


def set_threads(n: int):
    """Worker threads of the row-parallel matrix loops (the reference uses rayon there); 1 = serial."""
    lib().zko_set_threads(C.c_int(int(n)))


# ---- Merkle tree and Basefold (oracle/pcs.hpp, oracle/basefold.hpp) ------------------------------
NODE_BLAKE3, NODE_AES_MMO = 0, 1


def aes128_encrypt(key: bytes, block: bytes) -> bytes:
    out = (C.c_uint8 * 16)()
    lib().zko_aes128_encrypt(_u8(key), _u8(block), out)
    return bytes(out)


def hash_node(left: bytes, right: bytes, kind: int) -> bytes:
    out = (C.c_uint8 * 16)()
    lib().zko_hash_node(_u8(left), _u8(right), C.c_int(kind), out)
    return bytes(out)


def merkle_root(values, kind: int) -> bytes:
    V, pv = _u32(values)
    out = (C.c_uint8 * 16)()
    lib().zko_merkle_root(pv, C.c_size_t(V.size), C.c_int(kind), out)
    return bytes(out)


def merkle_layers(values, kind: int) -> bytes:
    V, pv = _u32(values)
    return _bytes_call(lib().zko_merkle_layers, pv, C.c_size_t(V.size), C.c_int(kind), cap=max(1 << 16, 40 * V.size))


def _u64arr(idx):
    a = np.ascontiguousarray(idx, dtype=np.uint64)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint64))


def merkle_batch_open(values, kind: int, indices) -> bytes:
    V, pv = _u32(values); I, pi = _u64arr(indices)
    return _bytes_call(lib().zko_merkle_batch_open, pv, C.c_size_t(V.size), C.c_int(kind), pi, C.c_size_t(I.size))


def merkle_batch_roundtrip(values, kind: int, indices, tamper=0) -> int:
    """bit 0: batch proof verifies; bit 1: every single-path opening verifies."""
    V, pv = _u32(values); I, pi = _u64arr(indices)
    return int(lib().zko_merkle_batch_roundtrip(pv, C.c_size_t(V.size), C.c_int(kind), pi, C.c_size_t(I.size), C.c_int(tamper)))


def basefold_tables(log_n: int):
    total = (1 << log_n) - 1
    t = np.zeros(total, np.uint32); w = np.zeros(total, np.uint32)
    lib().zko_basefold_tables(C.c_size_t(log_n), t.ctypes.data_as(u32p), w.ctypes.data_as(u32p))
    return t, w


def basefold_encode(coeffs, log_n: int):
    Cf, pc = _u32(coeffs)
    assert Cf.size == 1 << log_n
    cw = np.zeros(2 << log_n, np.uint32)
    lib().zko_basefold_encode(pc, C.c_size_t(log_n), cw.ctypes.data_as(u32p))
    return cw


def basefold_commit_and_prove(tr, coeffs, point, kind: int) -> bytes:
    """bincode(BasefoldCommitment) || bincode(BasefoldOpeningProof)."""
    Cf, pc = _u32(coeffs); Pt, pp = _u32(point)
    return _bytes_call(lib().zko_basefold_commit_and_prove, tr.h, pc, C.c_size_t(Cf.size), pp, C.c_size_t(Pt.size), C.c_int(kind),
                       cap=1 << 22)


def basefold_verify_bytes(tr, blob: bytes, point, claimed: int, kind: int) -> int:
    """verify_opening on bincode(BasefoldCommitment) || bincode(BasefoldOpeningProof); the caller has absorbed the
    commitment root.  1 accept, 0 reject, -1 undecodable."""
    Pt, pp = _u32(point)
    return int(lib().zko_basefold_verify_bytes(tr.h, _u8(blob), C.c_size_t(len(blob)), pp, C.c_size_t(Pt.size), C.c_uint32(int(claimed)), C.c_int(kind)))


def basefold_roundtrip(coeffs, point, kind: int, tamper=0) -> int:
    Cf, pc = _u32(coeffs); Pt, pp = _u32(point)
    return int(lib().zko_basefold_roundtrip(pc, C.c_size_t(Cf.size), pp, C.c_size_t(Pt.size), C.c_int(kind), C.c_int(tamper)))


BIND_BLAKE3, BIND_PCS, BIND_PCS_FULL = 0, 1, 2


class features:
    """`with features(bind_mode, node_kind):` runs the oracle as the reference built with the
    matching cargo feature (default / pcs / pcs-full) for a target with that Merkle node hash."""

    def __init__(self, bind_mode: int = BIND_BLAKE3, node_kind: int = NODE_BLAKE3):
        self.v = (bind_mode, node_kind)

    def __enter__(self):
        lib().zko_set_features(C.c_int(self.v[0]), C.c_int(self.v[1]))
        return self

    def __exit__(self, *a):
        lib().zko_set_features(C.c_int(0), C.c_int(0))
        return False


def prove_elementwise(tr, a, b, c, point, add: bool) -> bytes:
    """Base-field prove_hadamard / prove_add as bincode bytes."""
    A, pa = _u32(a); B, pb = _u32(b); Cc, pc = _u32(c); Pt, pp = _u32(point)
    return _bytes_call(lib().zko_prove_elementwise, tr.h, C.c_int(int(add)), pa, pb, pc, C.c_size_t(A.size), pp, C.c_size_t(Pt.size))


def elementwise_base_roundtrip(a, b, c, point, add: bool, tamper=False) -> bool:
    A, pa = _u32(a); B, pb = _u32(b); Cc, pc = _u32(c); Pt, pp = _u32(point)
    return bool(lib().zko_elementwise_base_roundtrip(C.c_int(int(add)), pa, pb, pc, C.c_size_t(A.size), pp, C.c_size_t(Pt.size),
                                                C.c_int(int(tamper))))


def prove_lookup(tr, table_out, inputs, outputs):
    """Base-field prove_lookup (lookup.rs:432-604) -> (bincode bytes, status)."""
    T, pt = _u32(table_out); I, pi = _u32(inputs); Oo, po = _u32(outputs)
    st = C.c_int(0)
    cap = 1 << 22
    buf = (C.c_uint8 * cap)()
    lib().zko_prove_lookup.restype = C.c_size_t
    n = lib().zko_prove_lookup(tr.h, pt, C.c_size_t(T.size), pi, po, C.c_size_t(I.size), buf, C.c_size_t(cap), C.byref(st))
    return bytes(buf[:n]), st.value


def _batch_args(polys, log_ns):
    flat = np.concatenate([np.ascontiguousarray(p, dtype=np.uint32).reshape(-1) for p in polys]) if polys else np.zeros(0, np.uint32)
    n = np.array([np.asarray(p).size for p in polys], dtype=np.uint64)
    ln = np.array(log_ns, dtype=np.uint64)
    return flat, n, ln


def basefold_batch_prove(tr, polys, log_ns, individual_openings=False, kind=0) -> bytes:
    """batch_precommit_multi_height + batch_prove_with_precommit (basefold.rs:1183-1378; with individual_openings and equal sizes:
    batch_commit_and_prove, :801-956) -> bincode(Vec<BasefoldCommitment>) || bincode(BasefoldBatchProof)."""
    flat, n, ln = _batch_args(polys, log_ns)
    return _bytes_call(lib().zko_basefold_batch_prove, tr.h, flat.ctypes.data_as(u32p), n.ctypes.data_as(C.POINTER(C.c_uint64)),
                       ln.ctypes.data_as(C.POINTER(C.c_uint64)), C.c_size_t(len(polys)), C.c_int(int(individual_openings)), C.c_int(kind), cap=1 << 24)


def basefold_batch_verify_bytes(tr, blob: bytes, kind=0):
    """batch_verify_opening (basefold.rs:959-1137) on bincode(Vec<BasefoldCommitment>) || bincode(BasefoldBatchProof)
    -> (1 accept / 0 reject / -1 undecodable, the proof's final value)."""
    buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
    fv = C.c_uint32(0)
    rc = lib().zko_basefold_batch_verify_bytes(tr.h, buf, C.c_size_t(len(blob)), C.c_int(kind), C.byref(fv))
    return int(rc), fv.value


def basefold_batch_roundtrip(polys, log_ns, individual_openings=False, kind=0, tamper=0) -> int:
    flat, n, ln = _batch_args(polys, log_ns)
    return int(lib().zko_basefold_batch_roundtrip(flat.ctypes.data_as(u32p), n.ctypes.data_as(C.POINTER(C.c_uint64)), ln.ctypes.data_as(C.POINTER(C.c_uint64)),
                                                  C.c_size_t(len(polys)), C.c_int(int(individual_openings)), C.c_int(kind), C.c_int(tamper)))


def prove_row_attention(tr, q, k, v, num_heads: int, seq_len: int, d_head: int, table_out, num_kv_heads: int = 0):
    """prove_row_attention (attention.rs:116-276), or prove_row_attention_gqa (:386-500) when num_kv_heads != 0
    -> (bincode bytes of RowAttentionProof, status)."""
    Q, pq = _u32(q); K, pk = _u32(k); V, pv = _u32(v); T, pt = _u32(table_out)
    st = C.c_int(0)
    cap = (1 << 16) + num_heads * seq_len * (4 * (5 * seq_len + d_head) + 8192)
    buf = (C.c_uint8 * cap)()
    lib().zko_prove_row_attention.restype = C.c_size_t
    n = lib().zko_prove_row_attention(tr.h, pq, pk, pv, C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len), C.c_size_t(d_head), pt, C.c_size_t(T.size),
                                      buf, C.c_size_t(cap), C.byref(st))
    return bytes(buf[:n]), st.value


def row_attention_verify_bytes(tr, blob: bytes, k, v, num_heads: int, seq_len: int, d_head: int, num_kv_heads: int = 0) -> int:
    """verify_row_attention (attention.rs:279-385, GQA :503-590) on bincode(RowAttentionProof): 1 accept, 0 reject, -1 undecodable."""
    K, pk = _u32(k); V, pv = _u32(v)
    buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
    return int(lib().zko_row_attention_verify_bytes(tr.h, buf, C.c_size_t(len(blob)), pk, pv, C.c_size_t(num_heads), C.c_size_t(num_kv_heads),
                                                    C.c_size_t(seq_len), C.c_size_t(d_head)))


def row_attention_forward(q, k, v, num_heads: int, seq_len: int, d_head: int, table_out, num_kv_heads: int = 0):
    """The attention op's forward pass at seq_len >= 2 (pipeline/forward.rs:233-276) -> (values, status)."""
    Q, pq = _u32(q); K, pk = _u32(k); V, pv = _u32(v); T, pt = _u32(table_out)
    out = np.zeros(Q.size, dtype=np.uint32)
    st = lib().zko_row_attention_forward(pq, pk, pv, C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len), C.c_size_t(d_head), pt, C.c_size_t(T.size),
                                         out.ctypes.data_as(C.POINTER(C.c_uint32)))
    return out, st


def row_attention_roundtrip(q, k, v, num_heads: int, seq_len: int, d_head: int, table_out, tamper=0, num_kv_heads: int = 0) -> int:
    Q, pq = _u32(q); K, pk = _u32(k); V, pv = _u32(v); T, pt = _u32(table_out)
    return int(lib().zko_row_attention_roundtrip(pq, pk, pv, C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len), C.c_size_t(d_head), pt, C.c_size_t(T.size),
                                                 C.c_int(tamper)))


def lookup_base_roundtrip(table_out, inputs, outputs, tamper=0) -> bool:
    T, pt = _u32(table_out); I, pi = _u32(inputs); Oo, po = _u32(outputs)
    return bool(lib().zko_lookup_base_roundtrip(pt, C.c_size_t(T.size), pi, po, C.c_size_t(I.size), C.c_int(tamper)))


def prove_rmsnorm(tr, x, gamma, y, delta: int) -> bytes:
    """Base-field prove_rmsnorm (rmsnorm.rs:96-246) as bincode bytes."""
    X, px = _u32(x); G, pg = _u32(gamma); Y, py = _u32(y)
    return _bytes_call(lib().zko_prove_rmsnorm, tr.h, px, pg, py, C.c_size_t(X.size), C.c_int32(delta))


def rmsnorm_base_roundtrip(x, gamma, y, delta: int, tamper=0) -> bool:
    X, px = _u32(x); G, pg = _u32(gamma); Y, py = _u32(y)
    return bool(lib().zko_rmsnorm_base_roundtrip(px, pg, py, C.c_size_t(X.size), C.c_int32(delta), C.c_int(tamper)))
