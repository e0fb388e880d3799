"""A dense chain (linear, lookup activation, linear, ...) proved on one transcript: the shape of
the reference's Dense-4M benchmark (python/benchmark_dense4m.py) built from the sub-protocol
provers.  `ef=True` uses the extension-field provers (prove_matmul_succinct_ef + prove_lookup_ef,
rust/zk_ml_prover/src/proving/matmul.rs:963-997, lookup.rs:643-762), `ef=False` their base-field
twins (matmul.rs:482-511, lookup.rs:432-604).  Weights stay resident on the GPU."""
from __future__ import annotations

import numpy as np

from . import protocols as zp
from .sumcheck import Context, Transcript


class DenseChain:
    def __init__(self, ctx: Context, weights, dims, table_out):
        """weights[l]: (dims[l+1] x dims[l]) row-major u32; table_out: output column of a 65536-entry table."""
        self.ctx = ctx
        self.dims = list(dims)
        self.w = [ctx.upload(np.ascontiguousarray(w, dtype=np.uint32).reshape(-1)) for w in weights]
        self.table_out = np.ascontiguousarray(table_out, dtype=np.uint32)
        self._table_dev = ctx.upload(self.table_out)

    def forward(self, x):
        """Returns the trace [(x_l, y_l, q_l, a_l)]: y = W x, q = requantised y, a = table[q]."""
        trace, cur = [], np.ascontiguousarray(x, dtype=np.uint32)
        for l, w in enumerate(self.w):
            m, n = self.dims[l + 1], self.dims[l]
            y = zp.matmul_forward(self.ctx, w, cur, m, n)
            if l + 1 < len(self.w):
                q, a = zp.requantize_lookup(self.ctx, y, self._table_dev)      # on the device (requantize_to_i16_field + table lookup)
                trace.append((cur, y, q, a))
                cur = a
            else:
                trace.append((cur, y, None, None))
        return trace

    def prove(self, trace, transcript: Transcript, ef: bool = True):
        """One proof per op, in forward order, all bound to `transcript`."""
        mm = zp.prove_matmul_succinct_ef if ef else zp.prove_matmul_succinct
        lk = zp.prove_lookup_ef if ef else zp.prove_lookup
        proofs = []
        for l, (x, y, q, a) in enumerate(trace):
            proofs.append(mm(self.w[l], x, y, self.dims[l + 1], self.dims[l], transcript))
            if q is not None:
                proofs.append(lk(self.table_out, q, a, transcript))
        return proofs

    def close(self):
        for w in self.w:
            w.free()
        self.w = []
        self._table_dev.free()
