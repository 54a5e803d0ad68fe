#!/usr/bin/env python
"""Benchmark of the proving hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl zkh|reference]

Workload (BASELINE.json configs[1], the sumcheck microbench): a degree-2 sumcheck
(product of two multilinear polynomials) over 2^28 uniformly random Goldilocks
elements per column, inputs seeded by the LCG the reference's selftests use.  One step =
one complete sumcheck proof: 28 rounds of message + Fiat-Shamir challenge + fold.
At N > 1 the hypercube is split on its top log2(N) variables: every rank folds a 2^28
slice (weak scaling: the instance has 2^28 * N vertices) and the ranks exchange
(nt) field elements per round.

Metric: sumcheck fold GB/s = algorithmic bytes / time with
algorithmic bytes = 24 * nc * N per sumcheck (12 * nc * n per fused round of input length n,
summed over the rounds).  Printed as ONE JSON line by rank 0.
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

METRIC = "sumcheck fold GB/s (degree-2, 2^28 Goldilocks MLEs)"
UNIT = "GB/s"
SEED = 0xBEEF1234
DRAM_PER_ALG_BYTE = {"sc_fused_kernel": 0.953}


def alg_bytes(nc, logn):
    return 24 * nc * (1 << logn)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

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
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def lcg_cols(orc, n, count, seed):
    cols, s = [], seed
    for _ in range(count):
        a, s = orc.lcg(n, s)
        cols.append(a)
    return cols


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, no MEASURED_PEAKS.json)"


def cpu_baseline(logn_sample, nthreads, use_reference):
    """The same degree-2 sumcheck on the host cores, bounded sample."""
    from oracle import F_PROD2, Oracle, Reference
    orc = Oracle()
    cols = lcg_cols(orc, 1 << logn_sample, 2, SEED)
    st0 = orc.tr_init("bench-sc2")
    kind = "port"
    t0 = time.perf_counter()
    if use_reference and Reference.available():
        # the reference's host sumcheck loop (p3hwl::sc5_prove, OpenMP over all host threads)
        Reference().sc5_prove(st0, "sc", 0, cols)
        kind = "reference"
    else:
        orc.sumcheck(st0, "sc", F_PROD2, 3, cols, (), nthreads)
    dt = time.perf_counter() - t0
    return {"value": alg_bytes(2, logn_sample) / dt / 1e9, "unit": UNIT, "cores": nthreads, "kind": kind,
            "sample": "one degree-2 sumcheck over 2^%d elements per column (%.1f s)" % (logn_sample, dt)}


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the path, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    ncores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(ncores))
    logn = args.ref_logn
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        base = cpu_baseline(logn, ncores, True)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / max(len(times), 1)
    val = alg_bytes(2, logn) / (ms / 1e3) / 1e9
    base["value"] = val
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u64 (Goldilocks field)", "data": "synthetic",
        "config": {"workload": "degree-2 sumcheck, bounded sample 2^%d elements per column on the host "
                               "cores (full workload 2^28)" % logn, "nc": 2, "nt": 3},
        "cpu_baseline": base,
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="zkh", choices=["zkh", "reference"])
    ap.add_argument("--logn", type=int, default=28, help="log2 elements per column per GPU")
    ap.add_argument("--ref-logn", type=int, default=22, help="sample size of the CPU reference arm")
    ap.add_argument("--cpu-logn", type=int, default=24, help="sample size of the cpu_baseline leg")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import zkh_import
    zk = zkh_import.load()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run" % (args.gpus, world))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle import Oracle
    orc = Oracle()  # input generator (the LCG) and the cpu_baseline leg only

    logn, nc, nt = args.logn, 2, 3
    n = 1 << logn
    stream = torch.cuda.current_stream()
    prover = zk.Prover(local, stream.cuda_stream)

    # inputs: seeded, resident in HBM before the timed region (8 GB > L2, no flush needed)
    host_cols = lcg_cols(orc, n, nc, SEED + 1000 * rank)
    dcols = [zk.p3.to_device(c, "cuda:%d" % local) for c in host_cols]
    torch.cuda.synchronize()

    def step():
        tr = zk.Transcript("bench-sc2")
        if world == 1:
            return prover.sc_prove_gpu(tr, "sc", dcols, zk.F_PROD2, nt)
        return zk.p3.sc_prove_sharded(prover, tr, "sc", dcols, zk.F_PROD2, nt, dist)

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kern_ms = []
    ev0.record()
    for _ in range(args.steps):
        step()
        kern_ms.append(prover.profile_last())
    ev1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    total_logn = logn + (world.bit_length() - 1)
    value = alg_bytes(nc, logn) * world / (ms_step / 1e3) / 1e9

    # dominant kernel: the fused bind+message round on the full-size columns
    kname = kern_ms[0][0]
    k_ms = float(np.mean([k[1] for k in kern_ms]))
    k_bytes = kern_ms[0][2]
    peak, peak_src = measured_peak()
    achieved = k_bytes / (k_ms / 1e3) / 1e9
    # DRAM bytes per algorithmic byte from the ncu capture of a smaller launch of the same kernel
    # (profiles/sc_fused_kernel_deg2_sumcheck.md), scaled linearly to this launch
    traffic = DRAM_PER_ALG_BYTE.get(kname)
    traffic = traffic * k_bytes if traffic else None

    # end to end through the C ABI with host buffers (pinned): H2D of the columns, proof back
    e2e = None
    if world == 1 and args.e2e_steps > 0:
        pinned = [torch.from_numpy(c.view(np.int64)).pin_memory() for c in host_cols]
        pcols = [t.numpy().view(np.uint64) for t in pinned]
        prover.sc_prove_host(zk.Transcript("bench-sc2"), "sc", pcols, zk.F_PROD2, nt)  # warm-up
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            r, m, fin = prover.sc_prove_host(zk.Transcript("bench-sc2"), "sc", pcols, zk.F_PROD2, nt)
        e1.record()
        torch.cuda.synchronize()
        e_ms = e0.elapsed_time(e1) / args.e2e_steps
        e2e = {"value": alg_bytes(nc, logn) / (e_ms / 1e3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": nc * n * 8, "d2h_bytes_per_step": int(m.nbytes + r.nbytes + fin.nbytes + 32),
               "ms_per_step": e_ms, "call": "zkh_sumcheck_host (pinned host columns in, proof out)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        ncores = os.cpu_count() or 1
        cpu = cpu_baseline(args.cpu_logn, ncores, False)

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u64 (Goldilocks field)", "data": "synthetic",
            "config": {"workload": "degree-2 sumcheck (product of 2 MLEs), 2^%d elements per column per GPU, "
                                   "instance 2^%d" % (logn, total_logn),
                       "nc": nc, "nt": nt, "rounds": total_logn, "l2": "inputs (%.1f GB per GPU) exceed the 126 MB L2; "
                       "no flush between steps" % (nc * n * 8 / 1e9),
                       "parallelism": "hypercube split on the top %d variables" % (world.bit_length() - 1)},
            "roofline": {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "unit": UNIT,
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                         "launch_ms": k_ms, "alg_bytes_per_launch": k_bytes},
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(args.steps * ((1 + (logn - 12) + 1) if world == 1 else (2 * logn + 3))),
            "clocks": clocks,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
