"""Host-side mirror of the reference's op-list mode over the C ABI: MLP / GPT-2 shaped models as a
list of ops proved in reverse order on one transcript (rust/zk_ml_prover/src/pipeline/forward.rs,
pipeline/prove.rs:191-648).  Ops are added in forward order; weights stay resident on the GPU."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, u32p
from .protocols import _a
from .sumcheck import Context, DeviceBuffer

OP_RELU, OP_ATTENTION_SEQ1, OP_PASSTHROUGH, OP_SAVE, OP_ADD_SAVED, OP_SET_INPUT_REQUANT = 1, 2, 3, 4, 5, 6


class OpList:
    def __init__(self, ctx: Context, input_len: int):
        self.ctx = ctx
        self.h = C.c_void_p()
        self.n_ops = 0
        self._keep = []
        check(ctx.h, _lib.lib().zkb_oplist_create(ctx.h, C.c_uint32(input_len), C.byref(self.h)))

    def close(self):
        if self.h.value and self.ctx.h.value:
            _lib.lib().zkb_oplist_destroy.restype = None
            _lib.lib().zkb_oplist_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def linear(self, name: str, w, bias, m: int, n: int):
        W, pw = _a(w)
        if bias is None:
            check(self.ctx.h, _lib.lib().zkb_oplist_add_linear(self.h, name.encode(), pw, None, C.c_size_t(m), C.c_size_t(n)))
        else:
            B, pb = _a(bias)
            check(self.ctx.h, _lib.lib().zkb_oplist_add_linear(self.h, name.encode(), pw, pb, C.c_size_t(m), C.c_size_t(n)))
        self.n_ops += 1

    def _simple(self, kind, name, aux=""):
        check(self.ctx.h, _lib.lib().zkb_oplist_add_simple(self.h, C.c_int32(kind), name.encode(), aux.encode()))
        self.n_ops += 1

    def relu(self, name): self._simple(OP_RELU, name)
    def attention_seq1(self, name): self._simple(OP_ATTENTION_SEQ1, name)
    def passthrough(self, name): self._simple(OP_PASSTHROUGH, name)
    def save(self, name, save_name): self._simple(OP_SAVE, name, save_name)
    def add_saved(self, name, add_name): self._simple(OP_ADD_SAVED, name, add_name)
    def set_input_requant(self, name): self._simple(OP_SET_INPUT_REQUANT, name)

    def layernorm(self, name: str, gamma, beta):
        G, pg = _a(gamma)
        B, pb = _a(beta)
        check(self.ctx.h, _lib.lib().zkb_oplist_add_layernorm(self.h, name.encode(), pg, pb, C.c_size_t(G.size)))
        self.n_ops += 1

    def gelu(self, name: str, table_out: DeviceBuffer):
        """Requantise the current activation to int16 range and look it up in the table (device-resident output column)."""
        self._keep.append(table_out)
        check(self.ctx.h, _lib.lib().zkb_oplist_add_gelu(self.h, name.encode(), table_out.ptr, C.c_uint32(table_out.n)))
        self.n_ops += 1

    def attention(self, name: str, num_heads: int, seq_len: int, d_head: int, exp_table: DeviceBuffer, k_values=None, v_values=None,
                  num_kv_heads: int = 0):
        """"attention" at seq_len >= 2 (pipeline/forward.rs:202-306): the activation is Q | K | V, or Q alone with K and V given here;
        with num_kv_heads the "gqa_attention" op (forward.rs:555-660)."""
        self._keep.append(exp_table)
        pk = pv = None
        if k_values is not None:
            K, pk = _a(k_values); V, pv = _a(v_values)
        check(self.ctx.h, _lib.lib().zkb_oplist_add_attention(self.h, name.encode(), C.c_size_t(num_heads), C.c_size_t(num_kv_heads), C.c_size_t(seq_len),
                                                             C.c_size_t(d_head), exp_table.ptr, C.c_uint32(exp_table.n), pk, pv))
        self.n_ops += 1

    def set_attention_kv(self, op_index: int, k_values, v_values):
        """New K / V for the attention op at position `op_index` that was added with its own."""
        K, pk = _a(k_values); V, pv = _a(v_values)
        check(self.ctx.h, _lib.lib().zkb_oplist_set_attention_kv(self.h, C.c_uint32(op_index), pk, pv))

    def set_input(self, name: str, values):
        V, pv = _a(values)
        check(self.ctx.h, _lib.lib().zkb_oplist_add_set_input(self.h, name.encode(), pv, C.c_size_t(V.size)))
        self.n_ops += 1

    def forward(self, x):
        X, px = _a(x)
        check(self.ctx.h, _lib.lib().zkb_oplist_forward(self.h, px))

    def activation(self, op_index: int = None) -> np.ndarray:
        """Activation after op `op_index` (default: the last op) of the most recent forward pass."""
        if op_index is None:
            op_index = self.n_ops - 1
        n = C.c_size_t()
        cap = 1 << 17
        out = np.zeros(cap, np.uint32)
        check(self.ctx.h, _lib.lib().zkb_oplist_activation(self.h, C.c_uint32(op_index), out.ctypes.data_as(u32p), C.c_size_t(cap), C.byref(n)))
        return out[:n.value].copy()

    def prove(self, x, cap: int = 1 << 24) -> bytes:
        """Forward pass + all proofs: bincode(Vec<SerializedLayerProof>) in the reference's push order."""
        X, px = _a(x)
        buf = getattr(self, "_buf", None)
        if buf is None or len(buf) < cap:
            buf = self._buf = (C.c_uint8 * cap)()
        n = C.c_size_t()
        check(self.ctx.h, _lib.lib().zkb_oplist_prove(self.h, px, buf, C.c_size_t(len(buf)), C.byref(n)))
        return C.string_at(buf, n.value)
