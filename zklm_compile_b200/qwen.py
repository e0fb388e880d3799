"""Resident Qwen3.5-style layers and the multi-layer prove loop.

Mirrors, for seq_len = 1:
  QwenLayerWeights / commit_qwen_layer   rust/zk_ml_prover/src/transformer/qwen.rs:62-73, 148-161
  qwen_forward_indexed                   rust/zk_ml_prover/src/transformer/qwen.rs:211-325
  prove_qwen_layer_precommitted_ef       rust/zk_ml_prover/src/transformer/qwen.rs:795-912
  the per-layer fan-out                  rust/zk_ml_prover/src/pipeline/prove.rs:158-189
"""
from __future__ import annotations

import ctypes as C
import hashlib
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import _lib
from ._lib import check, u32p
from .sumcheck import Context, DeviceBuffer

WEIGHT_NAMES = ["norm1_gamma", "w_q", "w_k", "w_v", "w_o", "w_g_proj", "norm2_gamma", "w_gate", "w_up", "w_down"]
DIM_NAMES = ["d_model", "d_ff", "num_q_heads", "num_kv_heads", "d_head", "v_num_heads", "v_d_head"]


def hash_values(values) -> bytes:
    """rust/zk_ml_prover/src/field/common.rs:78-85: SHA-256(len u32 LE || values u32 LE)."""
    a = np.ascontiguousarray(values, dtype="<u4")
    return hashlib.sha256(len(a).to_bytes(4, "little") + a.tobytes()).digest()


class QwenLayer:
    """One layer with its weights resident in HBM and its eight weight commitments computed at
    load time (the reference excludes `commit_qwen_layer` from prove time,
    rust/zk_ml_prover/src/pipeline/mod.rs:224-229)."""

    def __init__(self, ctx: Context, config: dict, weights: dict, silu_table: DeviceBuffer, sigmoid_table: DeviceBuffer):
        self.ctx = ctx
        self.config = dict(config)
        self.h = C.c_void_p()
        dims = (C.c_uint64 * 7)(*[int(config.get(k, 0)) for k in DIM_NAMES])
        keep = [np.ascontiguousarray(weights[k], dtype=np.uint32) for k in WEIGHT_NAMES]
        wp = (u32p * 10)(*[a.ctypes.data_as(u32p) for a in keep])
        self._tables = (silu_table, sigmoid_table)
        check(ctx.h, _lib.lib().zkb_qwen_layer_create(ctx.h, dims, wp, silu_table.ptr, sigmoid_table.ptr, C.c_uint32(silu_table.n),
                                                       C.byref(self.h)))
        self.d_model = int(config["d_model"])

    def close(self):
        if self.h.value and self.ctx.h.value:
            _lib.lib().zkb_qwen_layer_destroy.restype = None
            _lib.lib().zkb_qwen_layer_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def commitments(self):
        buf = (C.c_uint8 * 256)()
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_commitments(self.h, buf))
        b = bytes(buf)
        return [b[32 * i:32 * i + 32] for i in range(8)]

    def forward(self, x) -> np.ndarray:
        a = np.ascontiguousarray(x, dtype=np.uint32)
        y = np.zeros(self.d_model, np.uint32)
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_forward(self.h, a.ctypes.data_as(u32p), C.c_int32(0), y.ctypes.data_as(u32p), C.c_int32(0)))
        return y

    def forward_dev(self, x: DeviceBuffer):
        """Forward with a device-resident input vector."""
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_forward(self.h, x.ptr, C.c_int32(1), None, C.c_int32(0)))

    def forward_from(self, prev: "QwenLayer"):
        """Forward with the previous layer's device-resident output as input (no host copy)."""
        _lib.lib().zkb_qwen_layer_output_dev.restype = u32p
        src = _lib.lib().zkb_qwen_layer_output_dev(prev.h)
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_forward(self.h, src, C.c_int32(1), None, C.c_int32(0)))

    def forward_async(self, prev: "QwenLayer" = None, x=None):
        """Enqueue the forward pass without waiting: input is `prev`'s device-resident output, or
        `x` (host array or DeviceBuffer).  `prev.forward_async` must already have been called."""
        if prev is not None:
            check(self.ctx.h, _lib.lib().zkb_qwen_layer_forward_async(self.h, prev.h, None, C.c_int32(0)))
        elif isinstance(x, DeviceBuffer):
            check(self.ctx.h, _lib.lib().zkb_qwen_layer_forward_async(self.h, None, x.ptr, C.c_int32(1)))
        else:
            self._x_keep = np.ascontiguousarray(x, dtype=np.uint32)
            check(self.ctx.h, _lib.lib().zkb_qwen_layer_forward_async(self.h, None, self._x_keep.ctypes.data_as(u32p), C.c_int32(0)))

    def use_graph(self, on: bool):
        """Replay of the captured launch sequence (default on) or launch-by-launch enqueueing."""
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_use_graph(self.h, C.c_int32(1 if on else 0)))

    def graph_state(self) -> int:
        """0: the next proof is enqueued launch by launch, 1: it will be captured into a graph, 2: replayed."""
        return int(_lib.lib().zkb_qwen_layer_graph_state(self.h))

    def set_binding(self, bind_mode: int, node_hash: int = 0):
        """Weight binding of the matmul proofs: 0 default build, 1 feature pcs, 2 feature pcs-full
        (bind_weights_ef, rust/zk_ml_prover/src/proving/matmul.rs:360-453)."""
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_set_binding(self.h, C.c_int32(bind_mode), C.c_int32(node_hash)))
        self._bind_mode = bind_mode

    def read_output_after_forward(self) -> np.ndarray:
        """Output of an asynchronous forward, without waiting for a proof queued behind it."""
        y = np.zeros(self.d_model, np.uint32)
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_read_output(self.h, y.ctypes.data_as(u32p)))
        return y

    def wait_forward(self):
        """Host-side wait for this layer's asynchronous forward pass (not for its proof)."""
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_wait_forward(self.h))

    def output_address(self) -> int:
        """Device address of the layer output (d_model u32 words)."""
        fn = _lib.lib().zkb_qwen_layer_output_dev
        fn.restype = C.c_void_p
        return int(fn(self.h))

    def output(self) -> np.ndarray:
        _lib.lib().zkb_qwen_layer_output_dev.restype = u32p
        src = _lib.lib().zkb_qwen_layer_output_dev(self.h)
        y = np.zeros(self.d_model, np.uint32)
        check(self.ctx.h, _lib.lib().zkb_buf_download_u32(self.ctx.h, src, C.c_size_t(self.d_model), y.ctypes.data_as(u32p)))
        return y

    def prove_begin(self, layer_idx: int, input_hash: bytes):
        ih = (C.c_uint8 * 32).from_buffer_copy(input_hash)
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_prove_begin(self.h, C.c_uint32(layer_idx), ih))

    def prove_end(self, cap: int = None) -> bytes:
        if cap is None:      # eight Basefold openings make a layer proof of a few MB
            cap = (1 << 20) if getattr(self, "_bind_mode", 0) == 0 else (1 << 24)
        buf = getattr(self, "_proof_buf", None)
        if buf is None or len(buf) < cap:
            buf = self._proof_buf = (C.c_uint8 * cap)()
        n = C.c_size_t()
        st = _lib.lib().zkb_qwen_layer_prove_end(self.h, buf, C.c_size_t(len(buf)), C.byref(n))
        if st == 7 and n.value > len(buf):
            raise _lib.ZkbError(7, f"layer proof needs {n.value} bytes; call prove_end(cap=...) with a larger buffer")
        check(self.ctx.h, st)
        return C.string_at(buf, n.value)

    def verify(self, layer_idx: int, input_hash: bytes, proof: bytes, y_expected=None) -> bool:
        """verify_qwen_layer_ef_indexed (qwen.rs:932-1097) against the trace of the last forward pass."""
        buf = (C.c_uint8 * len(proof)).from_buffer_copy(proof)
        ok = C.c_int32(0)
        ye = None
        if y_expected is not None:
            y = np.ascontiguousarray(y_expected, dtype=np.uint32)
            ye = y.ctypes.data_as(u32p)
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_verify(self.h, C.c_uint32(layer_idx), (C.c_uint8 * 32).from_buffer_copy(input_hash), buf, C.c_size_t(len(proof)), ye, C.byref(ok)))
        return bool(ok.value)

    def verify_begin(self, layer_idx: int, input_hash: bytes, proof: bytes, y_expected=None):
        buf = (C.c_uint8 * len(proof)).from_buffer_copy(proof)
        ye = None
        if y_expected is not None:
            y = np.ascontiguousarray(y_expected, dtype=np.uint32)
            ye = y.ctypes.data_as(u32p)
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_verify_begin(self.h, C.c_uint32(layer_idx), (C.c_uint8 * 32).from_buffer_copy(input_hash), buf,
                                                                 C.c_size_t(len(proof)), ye))

    def verify_end(self) -> bool:
        ok = C.c_int32(0)
        check(self.ctx.h, _lib.lib().zkb_qwen_layer_verify_end(self.h, C.byref(ok)))
        return bool(ok.value)

    def prove(self, layer_idx: int, input_hash: bytes) -> bytes:
        """QwenLayerProofEF as bincode bytes; `forward` must have run."""
        self.prove_begin(layer_idx, input_hash)
        return self.prove_end()


class QwenModel:
    """A stack of layers on one GPU, one context (stream) per layer so that the independent
    per-layer proofs overlap on the device.  `weights` is a list of weight dicts or a callable
    i -> dict (so that only one layer's host copy is alive at a time); `first_layer` is the
    global index of this stack's first layer when a model is sharded over several GPUs."""

    def __init__(self, device: int, configs, weights, silu_out, sigmoid_out, first_layer: int = 0, shared_shapes: bool = False,
                 n_contexts: int = None):
        """`n_contexts` < number of layers makes the layers share that many contexts (layer i uses
        context i mod n_contexts) and proves them in waves of n_contexts, which bounds the scratch
        memory alive at once - what the reference's chunked fan-out does for pcs-full
        (rust/zk_ml_prover/src/pipeline/prove.rs:112-151)."""
        self.device = device
        self.first_layer = first_layer
        configs = list(configs)
        self.n_contexts = min(n_contexts or len(configs), max(1, len(configs)))
        pool_ctxs = [Context(device) for _ in range(self.n_contexts)]
        self.ctxs = [pool_ctxs[i % self.n_contexts] for i in range(len(configs))]
        self._own_ctxs = pool_ctxs
        if shared_shapes:                # measured slower on B200 for the 32-layer 4B shape (34.9 vs 32.7 ms): off by default
            for c in pool_ctxs:
                c.set_shared(True)
        self.tables = (self.ctxs[0].upload(silu_out), self.ctxs[0].upload(sigmoid_out))
        self.layers = []
        for i, (c, cfg) in enumerate(zip(self.ctxs, configs)):
            w = weights(i) if callable(weights) else weights[i]
            self.layers.append(QwenLayer(c, cfg, w, *self.tables))
            del w
        self.pool = ThreadPoolExecutor(max_workers=min(8, max(1, len(self.layers))))
        self.input_hash = bytes(32)
        # one high-priority stream for the forward passes of all layers (used by forward_and_prove)
        self._fwd_stream = C.c_void_p()
        if self.layers:
            check(self.ctxs[0].h, _lib.lib().zkb_stream_create(self.ctxs[0].h, C.c_int32(1), C.byref(self._fwd_stream)))
            for l in self.layers:
                check(l.ctx.h, _lib.lib().zkb_qwen_layer_set_forward_stream(l.h, self._fwd_stream))

    def forward(self, x, input_hash: bytes = None):
        """Sequential forward through the resident layers.  x: host vector or DeviceBuffer.
        `input_hash` is the hash of the *model* input (defaults to hash_values(x))."""
        if isinstance(x, DeviceBuffer):
            if input_hash is None:
                raise ValueError("input_hash is required with a device-resident input")
            self.input_hash = input_hash
            self.layers[0].forward_dev(x)
        else:
            self.input_hash = input_hash if input_hash is not None else hash_values(x)
            self.layers[0].forward(x)
        for prev, cur in zip(self.layers, self.layers[1:]):
            cur.forward_from(prev)

    def output(self) -> np.ndarray:
        return self.layers[-1].output()

    def prove(self):
        """Proofs of this stack's layers, in reverse layer order as the reference collects them
        (pipeline/prove.rs:183-188).  Enqueued from a few host threads, then collected."""
        n = len(self.layers)
        begin = lambda i: self.layers[i].prove_begin(self.first_layer + i, self.input_hash)
        if self.n_contexts < n:                                 # shared contexts: one wave of layers at a time
            proofs = []
            for w0 in range(0, n, self.n_contexts):
                wave = range(w0, min(n, w0 + self.n_contexts))
                for i in wave:
                    begin(i)
                proofs += [self.layers[i].prove_end() for i in wave]
            return proofs[::-1]
        if any(l.graph_state() == 1 for l in self.layers):      # one-off graph captures: one at a time
            for i in range(n):
                begin(i)
        else:
            list(self.pool.map(begin, range(n)))
        proofs = [l.prove_end() for l in self.layers]
        return proofs[::-1]

    @property
    def forward_stream(self) -> int:
        """The cudaStream_t (as an integer) that all forward passes of this model run on, for callers that order their
        own work with it on the device (e.g. a send of the last layer's output to the next GPU)."""
        return int(self._fwd_stream.value or 0)

    def forward_and_prove(self, x, input_hash: bytes = None, on_forward_done=None, on_forward_finished=None, on_forward_enqueued=None):
        """Forward pass and all layer proofs with the two overlapped: every layer's proof is
        enqueued right behind its own forward, the forward of the next layer only waits (on the
        GPU) for the previous layer's forward.  Returns the proofs in reverse layer order.
        `on_forward_done(output)` is called with the host copy of the output as soon as the last
        layer's forward has finished, while the proofs are still running; `on_forward_finished()` is
        called at the same moment without any copy (the output then sits at
        `layers[-1].output_address()` on the device: used to hand the activation to the next GPU);
        `on_forward_enqueued()` is called even earlier, as soon as the last layer's forward has been
        *enqueued* on `forward_stream` - work the caller then puts on that stream runs right behind it on the
        device, with no host wait in between."""
        import threading
        if isinstance(x, DeviceBuffer):
            if input_hash is None:
                raise ValueError("input_hash is required with a device-resident input")
            self.input_hash = input_hash
        else:
            self.input_hash = input_hash if input_hash is not None else hash_values(x)
        n = len(self.layers)
        if self.n_contexts < n:          # shared contexts: the whole forward pass first, then the proofs in waves
            self.forward(x, input_hash)
            if on_forward_enqueued is not None:
                on_forward_enqueued()
            if on_forward_finished is not None:
                self.layers[-1].ctx.sync()
                on_forward_finished()
            if on_forward_done is not None:
                on_forward_done(self.output())
            return self.prove()
        issued = [threading.Event() for _ in range(n)]
        failed = []

        def task(i):
            try:
                if i:
                    issued[i - 1].wait()
                    if failed:
                        raise RuntimeError("an earlier layer failed")
                    self.layers[i].forward_async(prev=self.layers[i - 1])
                else:
                    self.layers[0].forward_async(x=x)
            except Exception as e:       # never leave the next layer waiting
                failed.append(e)
                issued[i].set()
                raise
            issued[i].set()
            self.layers[i].prove_begin(self.first_layer + i, self.input_hash)

        if any(l.graph_state() == 1 for l in self.layers):
            # one-off graph captures: keep them on this thread, one at a time
            for i in range(n):
                task(i)
            futures = []
        else:
            futures = [self.pool.submit(task, i) for i in range(n)]
        if on_forward_done is not None or on_forward_finished is not None or on_forward_enqueued is not None:
            issued[n - 1].wait()
            if not failed and on_forward_enqueued is not None:
                on_forward_enqueued()
            if not failed and on_forward_finished is not None:
                self.layers[-1].wait_forward()
                on_forward_finished()
            if not failed and on_forward_done is not None:
                on_forward_done(self.layers[-1].read_output_after_forward())
        for f in futures:
            f.result()
        proofs = [l.prove_end() for l in self.layers]
        return proofs[::-1]

    def forward_and_verify(self, x, proofs, input_hash: bytes = None, y_expected=None) -> bool:
        """verify_qwen_layer_ef_indexed for every layer (qwen.rs:932-1097): the forward pass is run again, each
        layer's proof (`proofs` in the order forward_and_prove returns them: last layer first) is checked against
        that pass's trace, all layers side by side on their own contexts.  `y_expected` is the claimed model output."""
        if self.n_contexts < len(self.layers):
            raise ValueError("forward_and_verify needs one context per layer")
        if len(proofs) != len(self.layers):
            return False
        if isinstance(x, DeviceBuffer):
            if input_hash is None:
                raise ValueError("input_hash is required with a device-resident input")
            self.input_hash = input_hash
        else:
            self.input_hash = input_hash if input_hash is not None else hash_values(x)
        by_layer = proofs[::-1]
        n = len(self.layers)
        self.layers[0].forward_async(x=x)
        for i in range(1, n):
            self.layers[i].forward_async(prev=self.layers[i - 1])

        def task(i):
            self.layers[i].verify_begin(self.first_layer + i, self.input_hash, by_layer[i], y_expected if i == n - 1 else None)

        for f in [self.pool.submit(task, i) for i in range(n)]:
            f.result()
        verdicts = [l.verify_end() for l in self.layers]
        return all(verdicts)

    def close(self):
        self.pool.shutdown()
        for l in self.layers:
            l.close()
        if self._fwd_stream.value:
            _lib.lib().zkb_stream_destroy.restype = None
            _lib.lib().zkb_stream_destroy(self._fwd_stream)
            self._fwd_stream = C.c_void_p()
        for t in self.tables:
            t.free()
        for c in self._own_ctxs:
            c.close()
