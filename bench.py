#!/usr/bin/env python
"""Benchmark of the grouped n:m hot path:  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("sweep"): the density sweep on one layer -- weight 4096 x 4096 ~ N(0,1) (seed 0) sparsified to grouped
n:m for n:m in {1:4, 2:4, 1:8, 2:8, 1:16} with g = 16, activations 4096 tokens x 4096 ~ N(0,1) (seed 1), fp32.
One step is one pass of the hot path over that batch: y = x W^T for each of the five sparse weights.
metric = useful (non-zero) GFLOP/s = sum over the five of 2*M*K*tokens*n/m, divided by the step time.

With N > 1 ranks (torchrun) every rank runs the same sweep on its own 4096-token shard of the batch (token rows
are independent, so no collective is on the data path): weak scaling, value = N * per-rank work / max-over-ranks
time.

Printed JSON (one line, rank 0):
  value        device-resident throughput (inputs already in HBM), CUDA events around exactly K steps
  e2e          same metric through the public plugin API (F.linear on SparseParameterWrapper weights) with pinned
               HOST activations: the H2D copy of x and the D2H copy of every y are inside the timed region
  roofline     the dominant kernel (SIMT forward, 2:4) against the fp32 FMA peak measured on this GPU
  cpu_baseline the reference's CPU-SIMD kernels (oracle/_ref) or the oracle port on this host's cores
  sweep        per-pattern device times, fp32 and bf16, next to torch.mm (cuBLAS) on the densified weight
`--impl reference` times only the CPU implementation on a bounded token sample and prints the same line shape.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SWEEP = [(1, 4), (2, 4), (1, 8), (2, 8), (1, 16)]
G = 16
M = K = 4096
TOKENS = 4096
METRIC = "nmg_spmm_useful_gflops"
UNIT = "GFLOP/s"


def useful_flops(n, m, tokens=TOKENS):
    return 2.0 * M * K * tokens * n / m


def step_flops(tokens=TOKENS):
    return sum(useful_flops(n, m, tokens) for n, m in SWEEP)


def config_dict(n_gpus):
    return {"workload": "density sweep: W 4096x4096 N(0,1) seed 0, nmg {1:4,2:4,1:8,2:8,1:16} g=16, X 4096x4096 fp32 seed 1",
            "tokens_per_gpu": TOKENS, "group_size": G, "parallelism": f"token-sharded x{n_gpus}, no collective",
            "l2": "per-step working set ~0.5 GB (5 outputs of 64 MiB + activations + weights) exceeds the 126 MB L2"}


# ------------------------------------------------------------------------------------------------ CPU side
def cpu_spmm_fn(n, m):
    """(callable(val, idx, x) -> y, kind): the reference's micro-kernels when built for this problem, else the oracle port."""
    from oracle import build_ref, nmg_oracle
    if build_ref.load(n, m, G, K) is not None:
        return (lambda val, idx, x: build_ref.spmm(val, idx, x, M, K, n, m, G)), "reference"
    return (lambda val, idx, x: nmg_oracle.spmm(val, idx, x, M, K, n, m, G)), "port"


def cpu_problem(tokens):
    import numpy as np
    import torch
    from oracle import nmg_oracle
    w = torch.randn(M, K, generator=torch.Generator().manual_seed(0)).numpy()
    x = torch.randn(TOKENS, K, generator=torch.Generator().manual_seed(1)).numpy()[:tokens]
    packs = {}
    for n, m in SWEEP:
        packs[(n, m)] = nmg_oracle.sparsify(w, n, m, G)
    return packs, np.ascontiguousarray(x)


def time_cpu(steps, warmup, tokens):
    """Seconds per step (one pass over the five patterns on `tokens` tokens), kind, threads."""
    from oracle import nmg_oracle
    packs, x = cpu_problem(tokens)
    fns = {nm: cpu_spmm_fn(*nm) for nm in SWEEP}
    kind = "reference" if all(k == "reference" for _, k in fns.values()) else "port"

    def one_step():
        for nm in SWEEP:
            fns[nm][0](packs[nm][0], packs[nm][1], x)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / steps
    return dt, kind, nmg_oracle.num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    tokens = 1024  # bounded sample: a quarter of the batch, every pattern
    dt, kind, cores = time_cpu(args.steps, args.warmup, tokens)
    val = step_flops(tokens) / dt / 1e9
    sample = f"{tokens} of {TOKENS} tokens, all five patterns, fp32, {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))
    return 0


# ------------------------------------------------------------------------------------------------ GPU side
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except (ValueError, IndexError):
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_ours(args):
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    import sten_b200 as sten
    from sten_b200 import _native as nat, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sten.set_dispatch_failure("raise")

    # ---- data: same weight on every rank, a different token shard per rank
    w = torch.randn(M, K, generator=torch.Generator().manual_seed(0)).to(dev)
    x_host = torch.randn(TOKENS, K, generator=torch.Generator().manual_seed(1 + rank)).pin_memory()
    x = x_host.to(dev)
    packs = {nm: ops.sparsify(w.unsqueeze(0), nm[0], nm[1], G) for nm in SWEEP}
    outs = {nm: torch.empty(TOKENS, M, device=dev) for nm in SWEEP}

    def step():
        for (n, m) in SWEEP:
            val, idx = packs[(n, m)]
            ops.spmm(val, idx, M, K, n, m, G, x, out=outs[(n, m)])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = world * step_flops() / (ms_per_step * 1e-3) / 1e9
    launches = args.steps * len(SWEEP) * 2  # activation re-layout + matmul kernel per call

    # ---- end to end through the plugin API with host buffers (weights are model state and stay resident)
    sb = sten.SparsityBuilder()
    layers = torch.nn.ModuleList([torch.nn.Linear(K, M, bias=False, device=dev) for _ in SWEEP])
    for i, (n, m) in enumerate(SWEEP):
        layers[i].weight.data.copy_(w)
        sb.set_weight(f"{i}.weight", initial_sparsifier=sten.GroupedNMSparsifier(n, m, G), out_format=sten.GroupedNMTensor)
    sparse_layers = sb.sparsify_model_inplace(layers)
    y_host = [torch.empty(TOKENS, M).pin_memory() for _ in SWEEP]

    def e2e_step():
        xd = x_host.to(dev, non_blocking=True)
        with torch.no_grad():
            for layer, yh in zip(sparse_layers, y_host):
                yh.copy_(layer(xd), non_blocking=True)

    for _ in range(max(1, args.warmup // 2)):
        e2e_step()
    barrier()
    k_e2e = max(1, args.steps // 2)
    e0.record()
    for _ in range(k_e2e):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    e2e_value = world * step_flops() / (ms_e2e / k_e2e * 1e-3) / 1e9
    h2d = x_host.numel() * 4
    d2h = sum(y.numel() * 4 for y in y_host)

    result = None
    if rank == 0:
        # ---- roofline of the dominant kernel (2:4 SIMT forward), timed alone with events around its launch
        import ctypes
        L = nat.lib()
        peak = ctypes.c_double(0.0)
        nat.check(L.nmg_measure_fma_peak(ctypes.byref(peak), torch.cuda.current_stream().cuda_stream))
        n, m = 2, 4
        val, idx = packs[(n, m)]
        ks, ke = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ks.record()
        ke.record()  # torch creates the underlying CUDA events on first record
        torch.cuda.synchronize()
        kernel_ms = []
        for _ in range(8):
            nat.check(L.nmg_profile_next(ks.cuda_event, ke.cuda_event))
            ops.spmm(val, idx, M, K, n, m, G, x, out=outs[(n, m)])
            torch.cuda.synchronize()
            kernel_ms.append(ks.elapsed_time(ke))
        kms = sum(kernel_ms[2:]) / len(kernel_ms[2:])
        achieved = useful_flops(n, m) / (kms * 1e-3) / 1e12
        roofline = {"bound": "fma", "kernel": "spmm_fwd_simt_kernel<2,4> fp32", "achieved": achieved, "peak": peak.value,
                    "unit": "TFLOP/s", "frac": achieved / peak.value if peak.value else None,
                    "peak_source": "fp32 FFMA loop measured in this run (nmg_measure_fma_peak)",
                    "traffic": None, "ms_per_launch": kms,
                    "algorithmic_flops_per_launch": useful_flops(n, m)}

        # ---- per-pattern sweep, fp32 and bf16, next to cuBLAS on the densified weight
        sweep = []
        for dtype, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            xd = x.to(dtype)
            for (n, m) in SWEEP:
                v32, i32 = packs[(n, m)]
                vv = v32.to(dtype)
                dense = ops.densify(vv, i32, 1, M, K, n, m, G)[0]
                o = torch.empty(TOKENS, M, device=dev, dtype=dtype)

                def timed(fn, reps=5):
                    fn()
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(reps):
                        fn()
                    b.record()
                    torch.cuda.synchronize()
                    return a.elapsed_time(b) / reps

                t_nmg = timed(lambda: ops.spmm(vv, i32, M, K, n, m, G, xd, out=o))
                t_dense = timed(lambda: torch.mm(xd, dense.t()))
                sweep.append({"nm": f"{n}:{m}", "dtype": name, "ms": t_nmg, "useful_gflops": useful_flops(n, m) / t_nmg / 1e6,
                              "cublas_dense_ms": t_dense, "speedup_vs_cublas": t_dense / t_nmg})

        # ---- CPU baseline on this host (bounded sample)
        cpu_tokens = 1024
        dt, kind, cores = time_cpu(3, 1, cpu_tokens)
        cpu = {"value": step_flops(cpu_tokens) / dt / 1e9, "unit": UNIT, "cores": cores, "kind": kind,
               "sample": f"{cpu_tokens} of {TOKENS} tokens, all five patterns, fp32, 3 timed passes"}

        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config_dict(world),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu, "sweep": sweep,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if result is not None:
        print(json.dumps(result))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
