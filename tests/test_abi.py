"""CPU-side checks of the drop-in boundary: the shared library loads and exports every symbol
the header declares.  No compute calls (there is no GPU where this runs)."""
import ctypes
import os
import re

import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import _lib


@pytest.fixture(scope="module")
def so():
    if not os.path.exists(_lib.LIB_PATH):
        zk.build()
    return ctypes.CDLL(_lib.LIB_PATH)


def declared_symbols():
    src = open(_lib.HEADER_PATH).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(zkb_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "zkb_ctx_create" in syms and "zkb_sumcheck_prove" in syms and len(syms) >= 20


def test_library_exports_every_declared_symbol(so):
    missing = [s for s in declared_symbols() if not hasattr(so, s)]
    assert not missing, f"declared in include/zkb200.h but not exported: {missing}"


def test_no_gpu_fails_loudly():
    """Without a CUDA device the context constructor must raise, never fall back."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(zk.ZkbError):
        zk.Context(0)
