"""The allocation-free weight fold against the regular one.

Some users of the library cannot allocate GPU memory once they are up and running: their
memory plan is fixed at start-up, or their host process forbids cudaMalloc afterwards.  For
them `zkb_fold_eq_matvec_ef_noalloc` keeps its accumulators in a fixed device array inside the
library.  This file checks, through the C ABI, that it returns exactly what the regular entry
point returns (integer field arithmetic, so bit for bit), on calls made one after the other
with different shapes so that leftovers of an earlier call in the shared array would show, and
that it refuses matrices wider than its fixed capacity.  The file name makes pytest collect
it last.
"""
import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import protocols as zp
from oracle import pyoracle as O

pytestmark = pytest.mark.gpu
P = (1 << 31) - 1


def _run_case(ctx, m, n, seed, oracle=False):
    rng = np.random.default_rng(seed)
    w = rng.integers(0, P, m * n, dtype=np.int64).astype(np.uint32)
    log_m = zp.log2_ceil(m)
    r = rng.integers(0, P, 4 * log_m, dtype=np.int64).astype(np.uint32)
    expected = zp.fold_eq_matvec(ctx, w, m, n, r, ef=True)             # the existing entry point
    eq = zp.eq_evals_ef(ctx, r.reshape(log_m, 4))
    n_pad = 1 << zp.log2_ceil(n)
    w_dev, eq_dev = ctx.upload(w), ctx.upload(eq)
    out_dev = ctx.upload(np.full(n_pad * 4, 0xDEADBEEF, np.uint32))    # every word must be overwritten
    # enqueue on the context's stream so the download below is ordered after it
    zp.fold_eq_matvec_ef_noalloc(w_dev, m, n, eq_dev, out_dev, stream=ctx.stream)
    got = out_dev.download().reshape(n_pad, 4)
    assert got.tolist() == expected.tolist(), f"allocation-free fold differs from the regular fold for {m} x {n}"
    if oracle:                             # and directly against the CPU restatement of fold_eq_matvec_ef (matmul.rs:743-835)
        assert got.tolist() == O.fold_eq_matvec_ef(w, m, n, r).tolist(), f"allocation-free fold differs from the oracle for {m} x {n}"


def test_noalloc_fold_matches_regular_fold_on_consecutive_calls():
    ctx = zk.Context(0)
    try:
        _run_case(ctx, 300, 2100, 1, oracle=True)   # first call on the device: also resolves the scratch address
        _run_case(ctx, 64, 40, 2)         # much narrower: stale accumulators beyond 64 columns must not matter
        _run_case(ctx, 77, 1023, 4, oracle=True)    # column count not a multiple of 4: the scalar row loads
        _run_case(ctx, 129, 16384, 3)     # exactly the capacity
        _run_case(ctx, 300, 2100, 1)      # and the first shape again
    finally:
        ctx.close()


def test_noalloc_fold_rejects_sizes_beyond_its_scratch():
    ctx = zk.Context(0)
    try:
        d = ctx.upload(np.zeros(16, np.uint32))
        with pytest.raises(zk.ZkbError) as e:
            zp.fold_eq_matvec_ef_noalloc(d, 1, 16385, d, d, stream=ctx.stream)
        assert e.value.code == 7 and "16384" in str(e.value)
    finally:
        ctx.close()
