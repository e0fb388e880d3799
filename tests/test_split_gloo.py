"""CPU check (two gloo ranks) of the ownership and ordering rules behind the split sumcheck:
rank g owns the elements j with j mod world == g, rounds are local while at least `world`
elements remain, per-round partial sums are added across ranks, every rank runs the same
transcript, and the per-rank remainders, ordered by rank, finish the proof.  The local
arithmetic is restated here in Python for the base-field product sumcheck
(rust/zk_ml_prover/src/proving/sumcheck.rs:211-272) and the result is compared with the
oracle's proof of the whole tables."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = (1 << 31) - 1


def _round_sums(f, g):
    half = len(f) // 2
    f0, f1, g0, g1 = f[:half], f[half:], g[:half], g[half:]
    f2, g2 = (2 * f1 - f0) % P, (2 * g1 - g0) % P
    return [int(np.sum(f0 * g0 % P) % P), int(np.sum(f1 * g1 % P) % P), int(np.sum(f2 * g2 % P) % P)]


def _fold(t, r):
    half = len(t) // 2
    return (t[:half] + r * ((t[half:] - t[:half]) % P)) % P


def _worker(rank, world, port, nv, q):
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as O
    from zklm_compile_b200.split import slice_for_rank
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(nv)
    n = 1 << nv
    F = rng.integers(0, P, n, dtype=np.int64)
    G = rng.integers(0, P, n, dtype=np.int64)
    f = slice_for_rank(F, world, rank).astype(object)
    g = slice_for_rank(G, world, rank).astype(object)
    tr = O.Transcript(b"gloo-split")
    polys, chal = [], []
    log_w = world.bit_length() - 1
    for rnd in range(nv):
        if rnd == nv - log_w:                     # gather the per-rank remainders, ordered by rank
            mine = torch.tensor([int(f[0]), int(g[0])], dtype=torch.int64)
            allv = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(allv, mine)
            f = np.array([int(v[0]) for v in allv], dtype=object)
            g = np.array([int(v[1]) for v in allv], dtype=object)
        s = torch.tensor(_round_sums(f, g), dtype=torch.int64)
        if rnd < nv - log_w:
            dist.all_reduce(s)                    # sums of canonical values: no overflow for world <= 2^32
        s = [int(v) % P for v in s]
        for v in s:
            tr.absorb(v)
        r = tr.squeeze()
        polys.append(s); chal.append(r)
        f, g = _fold(f, r), _fold(g, r)
    otr = O.Transcript(b"gloo-split")
    op, oc, ofin = O.prove("product", otr, [F.astype(np.uint32), G.astype(np.uint32)], nv)
    ok = (op.tolist() == polys and [int(c) for c in oc.reshape(-1)] == chal and int(ofin[0][0]) == int(f[0]) and int(ofin[1][0]) == int(g[0]))
    q.put((rank, ok))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,nv", [(2, 5), (2, 2)])
def test_split_ownership_and_ordering_on_gloo(world, nv):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + nv
    procs = [ctx.Process(target=_worker, args=(r, world, port, nv, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert res == [(r, True) for r in range(world)]
