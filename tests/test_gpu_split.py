"""GPU parity of the sumcheck that is split over several GPUs: the proof every rank obtains is
bit-identical to the oracle's single-machine proof.  With one GPU the exchange runs with a
world of one (every mailbox operation against the GPU's own memory); with two or more GPUs
the ranks run as child processes, one per GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest

import zklm_compile_b200 as zk
from zklm_compile_b200 import split as zs
from oracle import pyoracle as O
from tests.test_gpu_sumcheck import KIND_NAMES, rand_tables

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("kind", sorted(KIND_NAMES))
@pytest.mark.parametrize("nv", [1, 4, 13, 15])
def test_split_world_of_one_matches_oracle(kind, nv):
    ctx = zk.Context(0)
    xch = zs.Exchange(ctx, 1, 0)
    tables = rand_tables(kind, nv, 50 * kind + nv)
    for rep in range(2):                                    # sequence numbers keep advancing across proofs
        tr = zk.Transcript(ctx, b"w1")
        proof, *fin = zs.sumcheck_prove_split(kind, tables, nv, tr, xch)
        otr = O.Transcript(b"w1")
        polys, chal, ofin = O.prove(KIND_NAMES[kind], otr, tables, nv)
        assert proof.round_polys.reshape(nv, -1).tolist() == polys.tolist()
        assert proof.challenges.reshape(nv, -1).tolist() == chal.tolist()
        assert np.array([np.asarray(f, dtype=np.uint32).reshape(-1) for f in fin]).tolist() == ofin.tolist()
        assert tr.squeeze() == otr.squeeze()
    xch.close()
    ctx.close()


def test_silent_peer_times_out_and_context_stays_usable():
    # a bounded wait that runs out: the peer's flag is never set, the kernel gives up after the
    # limit, the host gets a status instead of a proof, and the GPU keeps working
    import time
    ctx = zk.Context(0)
    xch = zs.Exchange(ctx, 2, 0, timeout_ms=300, loopback=True)
    nv = 10
    tables = rand_tables(zk.SC_PRODUCT_EF, nv, 5)
    mine = [zs.slice_for_rank(t, 2, 0) for t in tables]
    t0 = time.time()
    with pytest.raises(zk.ZkbError) as e:
        zs.sumcheck_prove_split(zk.SC_PRODUCT_EF, mine, nv, zk.Transcript(ctx, b"to"), xch)
    assert e.value.code == 8                        # ZKB_E_TIMEOUT
    with pytest.raises(zk.ZkbError):                # sticky: the next call fails at once
        zs.sumcheck_prove_split(zk.SC_PRODUCT_EF, mine, nv, zk.Transcript(ctx, b"to"), xch)
    assert time.time() - t0 < 5.0
    xch.close()
    tr, otr = zk.Transcript(ctx, b"after"), O.Transcript(b"after")
    proof, *_ = zk.sumcheck_prove(zk.SC_PRODUCT_EF, tables, nv, tr)
    polys, _, _ = O.prove("product_ef", otr, tables, nv)
    assert proof.round_polys.reshape(nv, -1).tolist() == polys.tolist()
    ctx.close()


def _gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_split_over_several_gpus_matches_oracle(world):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29600 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "split_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(": OK") == world, r.stdout[-3000:]
