"""Child process of tests/test_gpu_split.py: one rank of a sumcheck split over several GPUs.
Launched by torch.distributed.run; rendezvous and the exchange of mailbox handles go over gloo."""
import os
import sys

import numpy as np
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import zklm_compile_b200 as zk  # noqa: E402
from zklm_compile_b200 import split as zs  # noqa: E402
from oracle import pyoracle as O  # noqa: E402

P = (1 << 31) - 1
NAMES = {zk.SC_PRODUCT: "product", zk.SC_TRIPLE: "triple", zk.SC_PRODUCT_ONES: "product_ones", zk.SC_PRODUCT_EF: "product_ef",
         zk.SC_PRODUCT_EF_FULL: "product_ef_full", zk.SC_PRODUCT_EF_MIXED: "product_ef_mixed",
         zk.SC_TRIPLE_EF_FULL: "triple_ef_full", zk.SC_PRODUCT_ONES_EF_FULL: "product_ones_ef_full"}


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = zk.Context(local)
    xch = zs.Exchange(ctx, world, rank)
    failures = []
    cases = [(k, nv) for k in sorted(NAMES) for nv in (3, 6, 13, 16)] + [(zk.SC_PRODUCT_EF, 20), (zk.SC_PRODUCT, 19)]
    for kind, nv in cases:
        if nv <= int(np.log2(world)):
            continue
        rng = np.random.default_rng(100 * kind + nv)            # same tables on every rank
        widths = O.SUMCHECKS[NAMES[kind]][1]
        n = 1 << nv
        tables = [rng.integers(0, P, (n, w) if w == 4 else n, dtype=np.int64).astype(np.uint32) for w in widths]
        label = b"split-%d-%d" % (kind, nv)
        tr = zk.Transcript(ctx, label)
        mine = [zs.slice_for_rank(t, world, rank, w) for t, w in zip(tables, widths)]
        proof, *fin = zs.sumcheck_prove_split(kind, mine, nv, tr, xch)
        otr = O.Transcript(label)
        polys, chal, ofin = O.prove(NAMES[kind], otr, tables, nv)
        got = np.array([np.asarray(f, dtype=np.uint32).reshape(-1) for f in fin])
        ok = (proof.round_polys.reshape(nv, -1).tolist() == polys.tolist() and proof.challenges.reshape(nv, -1).tolist() == chal.tolist()
              and got.tolist() == ofin.tolist() and tr.squeeze() == otr.squeeze())
        if not ok:
            failures.append((kind, nv))
    dist.barrier()
    xch.close()
    ctx.close()
    print(f"rank {rank}: {'OK' if not failures else 'FAIL ' + repr(failures)} ({len(cases)} cases)", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
