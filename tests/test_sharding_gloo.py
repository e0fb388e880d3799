"""The multi-rank host logic (layer ownership, the activation hop, gathering proofs in reverse
layer order) on CPU ranks: two processes, gloo backend, a stand-in for the per-layer work."""
import hashlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from zklm_compile_b200 import sharding


def test_layer_ranges_partition_everything():
    for L in (1, 5, 8, 32, 33):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                lo, hi = sharding.layer_range(r, world, L)
                seen += list(range(lo, hi))
                for i in range(lo, hi):
                    assert sharding.owner_of(i, world, L) == r
            assert seen == list(range(L))
    assert sharding.layer_range(7, 8, 32) == (28, 32)      # 4 layers per GPU at 8 GPUs


def test_merge_reverse():
    assert sharding.merge_reverse([[b"1", b"0"], [b"3", b"2"]]) == [b"3", b"2", b"1", b"0"]


def test_pack_unpack_proofs_roundtrip():
    buf = torch.empty(256, dtype=torch.uint8)
    for proofs in ([], [b""], [b"abc", b"", b"\x00" * 40]):
        sharding.pack_proofs(proofs, buf)
        assert sharding.unpack_proofs(buf) == proofs
    with pytest.raises(ValueError):
        sharding.pack_proofs([b"x" * 300], buf)


def _fake_layer(x, idx):
    """Stand-in for forward + prove of one layer: deterministic in (input, layer index)."""
    y = (x * 3 + idx + 1) % 2147483647
    proof = hashlib.sha256(x.tobytes() + idx.to_bytes(4, "little")).digest()
    return y, proof


def _worker(rank, world, port, L, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = sharding.layer_range(rank, world, L)
    act = torch.zeros(8, dtype=torch.int64)
    if rank == 0:
        act = torch.arange(8, dtype=torch.int64)
    else:
        sharding.recv_activation(dist, act, rank - 1)
    x = act.numpy().copy()
    proofs = []
    for i in range(lo, hi):
        x, p = _fake_layer(x, i)
        proofs.append(p)
    if rank + 1 < world:
        sharding.send_activation(dist, torch.from_numpy(x), rank + 1)
    gathered = sharding.ProofGather(dist, rank, world, 4096).gather(proofs[::-1])
    if rank == 0:
        out_q.put(sharding.merge_reverse(gathered))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,L", [(2, 5), (2, 8)])
def test_two_ranks_match_single_process(world, L):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, L, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = np.arange(8, dtype=np.int64)
    exp = []
    for i in range(L):
        x, pr = _fake_layer(x, i)
        exp.append(pr)
    assert got == exp[::-1]
