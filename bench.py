#!/usr/bin/env python
"""Benchmark of the sumcheck hot path (product sumcheck with M31^4 challenges over two
2^n-element M31 tables — the isolated microbench configuration).

One "step" = one complete n-round `prove_product_ef` (all folds, all round polynomials, the
SHA-256 transcript on the device, the final evaluations).  Prints ONE JSON line.

    python bench.py --gpus N --steps K --warmup W [--n 28] [--impl reference]

N > 1 (under torchrun): every rank proves its own independent sumcheck of the same size
(weak scaling, no data-path collective); time is the max over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

P = (1 << 31) - 1


def algorithmic_bytes(n):
    """Per fold launch and total: the launch that folds round k reads both tables of
    N_k = 2^(n-k) elements (4 B each for k = 0, 16 B after) and writes both half-size EF tables."""
    per = []
    for k in range(n):
        nk = 1 << (n - k)
        e = 4 if k == 0 else 16
        per.append(2 * nk * e + 2 * (nk // 2) * 16)
    return per, sum(per)


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for nm, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_reference_leg(n_cpu, steps, warmup):
    """The reference's own algorithm for this path on the host: `prove_product_ef` is a
    single-threaded loop in the reference (rust/zk_ml_prover/src/proving/sumcheck.rs:1204-1258),
    timed here through the C++ restatement (no Rust toolchain exists on this box)."""
    from oracle import pyoracle as O
    rng = np.random.default_rng(1234)
    f = rng.integers(0, P, 1 << n_cpu, dtype=np.int64).astype(np.uint32)
    g = rng.integers(0, P, 1 << n_cpu, dtype=np.int64).astype(np.uint32)
    for _ in range(warmup):
        O.prove("product_ef", O.Transcript(b"bench-product"), [f, g], n_cpu)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.prove("product_ef", O.Transcript(b"bench-product"), [f, g], n_cpu)
    dt = (time.perf_counter() - t0) / steps
    _, total = algorithmic_bytes(n_cpu)
    return total / dt / 1e9, dt * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--n", type=int, default=28, help="log2 of the table length")
    ap.add_argument("--n-cpu", type=int, default=24, help="log2 table length of the bounded CPU sample")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    metric = "sumcheck fold HBM GB/s (product sumcheck with M31^4 challenges, all rounds)"
    config = {"workload": f"isolated product-sumcheck microbench, two tables of 2^{args.n} M31 elements "
                          f"uniform in [0, 2^31-1), {args.n} rounds, seeded transcript 'bench-product'",
              "n": args.n, "l2_policy": "inputs (2 x %d MiB) are larger than L2" % ((4 << args.n) >> 20),
              "parallelism": f"{world} independent sumchecks, one per GPU" if world > 1 else "single GPU"}

    if args.impl == "reference":
        if rank != 0:
            return
        gbps, ms = cpu_reference_leg(args.n_cpu, max(1, min(args.steps, 3)), min(args.warmup, 1))
        line = {"impl": "reference", "metric": metric, "value": round(gbps, 4), "unit": "GB/s", "n_gpus": args.gpus,
                "steps": max(1, min(args.steps, 3)), "warmup": min(args.warmup, 1), "ms_per_step": round(ms, 3),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32 (M31 / M31^4)",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": round(gbps, 4), "unit": "GB/s", "cores": 1, "kind": "port",
                                 "sample": f"same workload at 2^{args.n_cpu} elements per table (bounded sample); "
                                           "prove_product_ef is single-threaded in the reference; Rust toolchain "
                                           "unavailable on this box, so the C++ restatement is timed"},
                "e2e": {"value": round(gbps, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import zklm_compile_b200 as zk

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ctx = zk.Context(local)
    n, N = args.n, 1 << args.n
    rng = np.random.default_rng(20251125 + rank)
    f_host = ctx.pinned_u32(N)
    g_host = ctx.pinned_u32(N)
    chunk = 1 << 24
    for off in range(0, N, chunk):
        m = min(chunk, N - off)
        f_host[off:off + m] = rng.integers(0, P, m, dtype=np.int64).astype(np.uint32)
        g_host[off:off + m] = rng.integers(0, P, m, dtype=np.int64).astype(np.uint32)
    f_dev, g_dev = ctx.upload(f_host), ctx.upload(g_host)
    per_launch_bytes, total_bytes = algorithmic_bytes(n)

    def step_dev():
        tr = zk.Transcript(ctx, b"bench-product")
        return zk.prove_product_ef(f_dev, g_dev, n, tr)

    def step_host():
        tr = zk.Transcript(ctx, b"bench-product")
        return zk.prove_product_ef(f_host, g_host, n, tr)

    # ---- kernel-side number: inputs resident in HBM ------------------------------------------
    for _ in range(args.warmup):
        ref = step_dev()
    ctx.profile(True)
    sampler = ClockSampler(local)
    sampler.start()
    ctx.sync(); barrier()
    launches0 = ctx.launches
    prof_acc = None
    ctx.timer_start()
    for _ in range(args.steps):
        out = step_dev()
        pr = np.array(ctx.profile_read())
        prof_acc = pr if prof_acc is None else prof_acc + pr
    ms_total = ctx.timer_stop_ms()
    ctx.sync(); barrier()
    launches = ctx.launches - launches0
    clocks = sampler.stop()
    ctx.profile(False)
    assert out[0].round_polys.tolist() == ref[0].round_polys.tolist()
    ms_step = max_over_ranks(ms_total / args.steps)
    value = world * total_bytes / (ms_step * 1e-3) / 1e9
    prof = (prof_acc / args.steps).tolist()

    # dominant kernel: the fold launches (index >= 1); launch i folds round i-1
    fold = [(per_launch_bytes[i - 1] / (prof[i] * 1e-3) / 1e9, prof[i], i) for i in range(1, len(prof) - 1)
            if prof[i] > 0]
    dom = max(fold, key=lambda x: x[1]) if fold else (0.0, 0.0, 0)
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peaks = json.load(fh)
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    roofline = {"bound": "hbm", "achieved": round(dom[0], 1), "peak": peak, "unit": "GB/s",
                "frac": round(dom[0] / peak, 4), "traffic": None,
                "peak_source": "MEASURED_PEAKS.json (of measured)" if peaks else "fallback 6650 GB/s (of fallback)",
                "kernel": f"sc_round_kernel fold launch {dom[2]} (folds round {dom[2] - 1}), "
                          f"{per_launch_bytes[dom[2] - 1] if dom[2] else 0} algorithmic bytes, {dom[1]:.4f} ms",
                "per_launch_gbps": [round(x[0], 1) for x in fold[:12]],
                "per_launch_ms": [round(x, 4) for x in prof[:14]]}

    # ---- end to end through the host-pointer ABI ---------------------------------------------
    e2e = None
    if not args.no_e2e:
        for _ in range(2):
            step_host()
        ctx.sync(); barrier()
        ctx.timer_start()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            out_h = step_host()
        ms_e2e = ctx.timer_stop_ms()
        wall = (time.perf_counter() - t0) * 1e3
        assert out_h[0].round_polys.tolist() == ref[0].round_polys.tolist()
        ms_e2e_step = max_over_ranks(ms_e2e / args.steps)
        proof_words = n * 2 * 4 + n * 4 + 8
        e2e = {"value": round(world * total_bytes / (ms_e2e_step * 1e-3) / 1e9, 2), "unit": "GB/s",
               "ms_per_step": round(ms_e2e_step, 3), "wall_ms_per_step": round(wall / args.steps, 3),
               "h2d_bytes_per_step": 2 * N * 4, "d2h_bytes_per_step": proof_words * 4}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        gbps, ms = cpu_reference_leg(args.n_cpu, 2, 1)
        cpu = {"value": round(gbps, 4), "unit": "GB/s", "cores": 1, "kind": "port", "ms_per_step": round(ms, 2),
               "sample": f"same workload at 2^{args.n_cpu} elements per table, 2 timed runs; single-threaded as in "
                         "the reference's prove_product_ef"}

    if rank == 0:
        line = {"metric": metric, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "u32 (M31 / M31^4)", "data": "synthetic",
                "config": config, "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": int(launches), "clocks": clocks,
                "algorithmic_bytes_per_step": total_bytes}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
