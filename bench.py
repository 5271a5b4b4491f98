#!/usr/bin/env python
"""Benchmark of the grouped n:m hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload sharded|sweep] [--impl reference]
    torchrun --nproc-per-node N ... bench.py --gpus N ...          (one rank per GPU, NCCL)

Workload "sharded" (default, every N): the large row-sharded matmul.  W 16384 x 16384 ~ N(0, 0.02) (seed 0), rounded
to bf16, grouped n:m 2:8 with g = 16, split by output rows over the N ranks; activations X 16384 tokens x 16384
~ N(0, 1) (seed 1) bf16, replicated.  One step computes C = W X^T: every rank multiplies by its row panels and the
output row slabs are combined with in-place NCCL all-gathers (one per row panel, overlapped with the next panel's
matmul; C = W X^T is kept as [M, tokens] so that slabs are contiguous); with N = 1 there is no collective.
Total work is fixed, so scaling is "strong".  metric = useful (non-zero) GFLOP/s = 2*M*K*tokens*n/m / step time.

Workload "encoder": BERT-large-shaped fp16 encoder with all encoder linears at nmg 2:4 through SparsityBuilder, batch
32 x seq 384 split over the ranks; tokens/s eager, as a CUDA graph, and for the dense fp16 model.

Workload "sweep": the 4096 x 4096 density sweep in fp32 (n:m in {1:4, 2:4, 1:8, 2:8, 1:16}, g = 16, 4096 tokens);
one step is the five matmuls; with N > 1 every rank runs it on its own token shard (weak scaling, no collective).

JSON line (rank 0):
  value        operands resident in HBM, CUDA events around exactly K steps, max over ranks
  e2e          same step through the public API with pinned HOST buffers: H2D of x and D2H of y inside the timed region
  roofline     the dominant kernel, timed alone with events recorded around its launch (nmg_profile_next)
  cpu_baseline the reference's CPU-SIMD kernels (oracle/_ref) on this host's cores, on a bounded sample
  sweep        (N = 1) per-pattern device times of the 4096^2 sweep in fp32 and bf16 next to cuBLAS on the densified weight
`--impl reference` times only the reference's CPU implementation on the bounded sample and prints the same line shape.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "nmg_spmm_useful_gflops"
UNIT = "GFLOP/s"
G = 16
SWEEP = [(1, 4), (2, 4), (1, 8), (2, 8), (1, 16)]
SW_M = SW_K = SW_TOK = 4096
SH_M = SH_K = SH_TOK = 16384
SH_N, SH_MM = 2, 8
# DRAM traffic of one full-size call of the default workload (expansion pass 0.683 GB + matmul kernel 9.416 GB), from one
# ncu capture on a B200; reported in roofline.traffic at N = 1
NCU_DRAM_BYTES_PER_CALL = 10.10e9
# bounded CPU sample of the sharded workload: one of eight row shards x 1024 tokens
CPU_ROWS, CPU_TOK = 2048, 1024


def useful_flops(M, K, tokens, n, m):
    return 2.0 * M * K * tokens * n / m


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "MEASURED_PEAKS.json"
    except (OSError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def config_dict(workload, n_gpus, exchange="peer", rounds=1):
    if workload == "sharded":
        how = ("no exchange" if n_gpus == 1 else
               "the matmul epilogue stores every output tile into all ranks' buffers over NVLink (multimem.st through the NVSwitch multicast address "
               "when the allocation has one, else one peer store per rank), one 4-byte all-reduce orders the ranks"
               if exchange == "peer" else f"{exchange}: {rounds} block-cyclic round(s), in-place NCCL all-gather of output slices overlapped with the next round")
        return {"workload": "row-sharded matmul: W 16384x16384 N(0,0.02) seed 0 bf16, nmg 2:8 g=16, X 16384x16384 N(0,1) seed 1 bf16",
                "group_size": G, "parallelism": f"weight rows split over {n_gpus} rank(s); {how}",
                "l2": "operands (0.5 GB activations + 0.5 GB output per step) exceed the 126 MB L2"}
    return {"workload": "density sweep: W 4096x4096 N(0,1) seed 0, nmg {1:4,2:4,1:8,2:8,1:16} g=16, X 4096x4096 fp32 seed 1",
            "tokens_per_gpu": SW_TOK, "group_size": G, "parallelism": f"token-sharded x{n_gpus}, no collective",
            "l2": "per-step working set ~0.5 GB exceeds the 126 MB L2"}


# ------------------------------------------------------------------------------------------------ CPU side
def cpu_spmm_fn(M, K, n, m):
    """(callable(val, idx, x) -> y, kind): the reference's micro-kernels when built for this K, else the oracle port."""
    from oracle import build_ref, nmg_oracle
    if build_ref.load(n, m, G, K) is not None:
        return (lambda val, idx, x: build_ref.spmm(val, idx, x, M, K, n, m, G)), "reference"
    return (lambda val, idx, x: nmg_oracle.spmm(val, idx, x, M, K, n, m, G)), "port"


def time_cpu(workload, steps, warmup):
    """Seconds per step of the bounded CPU sample, its useful flops, kind, threads, description."""
    import numpy as np
    import torch
    from oracle import build_ref, nmg_oracle
    # every host core this process may use, stated explicitly: launchers (torch.distributed.run) export OMP_NUM_THREADS=1
    # for their workers, which would otherwise make this a one-thread measurement
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    nmg_oracle.set_threads(cores)
    build_ref.set_threads(cores)
    torch.set_num_threads(cores)
    if workload == "sharded":
        w = (torch.randn(CPU_ROWS, SH_K, generator=torch.Generator().manual_seed(0)) * 0.02).bfloat16().float().numpy()
        x = torch.randn(CPU_TOK, SH_K, generator=torch.Generator().manual_seed(1)).bfloat16().float().numpy()
        jobs = [(CPU_ROWS, SH_K, SH_N, SH_MM, *nmg_oracle.sparsify(w, SH_N, SH_MM, G))]
        flops = useful_flops(CPU_ROWS, SH_K, CPU_TOK, SH_N, SH_MM)
        desc = f"rows 0..{CPU_ROWS - 1} of W (one of eight row shards) x {CPU_TOK} of {SH_TOK} tokens, fp32 arithmetic"
    else:
        w = torch.randn(SW_M, SW_K, generator=torch.Generator().manual_seed(0)).numpy()
        x = torch.randn(SW_TOK, SW_K, generator=torch.Generator().manual_seed(1)).numpy()[:CPU_TOK]
        jobs = [(SW_M, SW_K, n, m, *nmg_oracle.sparsify(w, n, m, G)) for n, m in SWEEP]
        flops = sum(useful_flops(SW_M, SW_K, CPU_TOK, n, m) for n, m in SWEEP)
        desc = f"{CPU_TOK} of {SW_TOK} tokens, all five patterns, fp32"
    x = np.ascontiguousarray(x)
    fns = [cpu_spmm_fn(M, K, n, m) for (M, K, n, m, _, _) in jobs]
    kind = "reference" if all(k == "reference" for _, k in fns) else "port"

    def one_step():
        for (fn, _), (M, K, n, m, val, idx) in zip(fns, jobs):
            fn(val, idx, x)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    return (time.perf_counter() - t0) / steps, flops, kind, cores, desc


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    dt, flops, kind, cores, desc = time_cpu(args.workload, args.steps, args.warmup)
    val = flops / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.workload == "sharded" else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(args.workload, args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))
    return 0


# ------------------------------------------------------------------------------------------------ GPU side
class ClockSampler:
    """SM clock and clock-event reasons of one GPU, polled through NVML every 5 ms while the timed region runs (read-only
    queries; falls back to `nvidia-smi -lms 100` when the NVML bindings are missing)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def _poll_nvml(self, nv, handle):
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                mask = int(get_reasons(handle))
                for name, bit in self.REASON_BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001 - a failed read is a missing sample
                pass
            self._stop.wait(0.005)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and visible.replace(",", "").isdigit() else self.index
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._poll_nvml, args=(nv, handle), daemon=True)
            self._thread.start()
            return
        except Exception:  # noqa: BLE001 - any NVML problem selects the nvidia-smi route
            self._thread = None
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
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            busy = sorted(self.samples)
            return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(self.reasons), "samples": len(busy), "source": "NVML, 5 ms period"}
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
        busy = sorted(sm[len(sm) // 4:]) if sm else []  # the first samples precede the load
        return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi -lms 100"}


def timed_loop(fn, steps, barrier, torch, dist, world, dev):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def kernel_time(call, torch, nat, reps=6):
    """Mean device time of the dominant kernel of `call`, events recorded right around its launch."""
    L = nat.lib()
    ks, ke = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ks.record()
    ke.record()  # torch creates the underlying CUDA events on first record
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        nat.check(L.nmg_profile_next(ks.cuda_event, ke.cuda_event))
        call()
        torch.cuda.synchronize()
        out.append(ks.elapsed_time(ke))
    out = out[2:] if len(out) > 3 else out
    return sum(out) / len(out)


CHECK_ROWS = 64
TOL = {"bf16": 1e-2, "f16": 1e-2, "f32": 1e-5}


def sampled_rows(torch, count, limit, seed, dev):
    rows = torch.randperm(limit, generator=torch.Generator().manual_seed(seed))[:count - 2]
    return torch.cat([rows, torch.tensor([0, limit - 1])]).sort().values.to(dev)


def rel_fro(got, want):
    got, want = got.double(), want.double()
    return float((got - want).norm() / want.norm())


def sweep_table(torch, ops, nat, dev, peaks, fma_peak):
    """4096^2 sweep, fp32 (SIMT) and bf16 (tensor cores), next to cuBLAS on the densified weight."""
    w = torch.randn(SW_M, SW_K, generator=torch.Generator().manual_seed(0)).to(dev)
    x = torch.randn(SW_TOK, SW_K, generator=torch.Generator().manual_seed(1)).to(dev)
    rows = []

    def timed(fn, reps=10):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    variants = ((torch.float32, "f32", nat.NMG_ALGO_SIMT, "simt fp32 FMA"),
                (torch.float32, "f32", nat.NMG_ALGO_TENSOR, "tensor cores, 6 bf16 split products"),
                (torch.bfloat16, "bf16", nat.NMG_ALGO_TENSOR, "tensor cores"))
    for dtype, name, algo, how in variants:
        xd = x.to(dtype)
        for (n, m) in SWEEP:
            val, idx = ops.sparsify(w.to(dtype).unsqueeze(0), n, m, G)
            dense = ops.densify(val, idx, 1, SW_M, SW_K, n, m, G)[0]
            packed = ops.pack(val, idx, SW_M, SW_K, n, m, G) if algo == nat.NMG_ALGO_TENSOR else None
            o = torch.empty(SW_TOK, SW_M, device=dev, dtype=dtype)
            t_nmg = timed(lambda: ops.spmm(val, idx, SW_M, SW_K, n, m, G, xd, out=o, packed=packed, algo=algo))
            t_dense = timed(lambda: torch.mm(xd, dense.t()))
            rows_chk = sampled_rows(torch, CHECK_ROWS, SW_M, 11, dev)
            err = rel_fro(o[:, rows_chk], xd.double() @ dense[rows_chk].double().t())
            useful = useful_flops(SW_M, SW_K, SW_TOK, n, m) / t_nmg / 1e9  # TFLOP/s
            tensor = algo == nat.NMG_ALGO_TENSOR
            peak = peaks["bf16_tflops"] if tensor else fma_peak
            executed = useful * m / n * (6 if (tensor and dtype == torch.float32) else 1) if tensor else useful
            row = {"nm": f"{n}:{m}", "dtype": name, "kernel": how, "ms": t_nmg, "useful_tflops": useful,
                   "bound": "tensor" if tensor else "fma", "frac_of_peak_useful": useful / peak,
                   "frac_of_peak_executed": executed / peak,
                   "cublas_dense_ms": t_dense, "speedup_vs_cublas": t_dense / t_nmg,
                   "rel_fro_vs_float64": err, "tolerance": TOL[name]}
            if dtype == torch.bfloat16:
                # opt-in: the expanded 16-bit weight kept across calls (no expansion pass, no memory saving): the matmul kernel alone
                kept = ops.expand(val, idx, SW_M, SW_K, n, m, G)
                t_kept = timed(lambda: ops.spmm_expanded(kept, SW_M, SW_K, xd, out=o))
                row["ms_kept_expanded_copy"] = t_kept
                row["speedup_vs_cublas_kept_expanded_copy"] = t_dense / t_kept
                row["rel_fro_kept_expanded_copy"] = rel_fro(o[:, rows_chk], xd.double() @ dense[rows_chk].double().t())
                del kept
            rows.append(row)
            del val, idx, dense, packed, o
    return rows


def transposed_table(torch, ops, nat, dev, peaks):
    """Transposed product dX = dY W (the backward pass) in bf16: structured-sparse tensor cores (tcgen05.mma.sp) with the
    compressed copy built per call and kept across calls, the dense-rate tensor-core kernels, and cuBLAS on the densified
    weight.  4096^2 at every pattern of the sweep, and the 16384^2 2:8 weight of the sharded workload."""
    rows = []

    def timed(fn, reps=10):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    cases = [(SW_M, SW_K, SW_TOK, n, m, 1.0, 10) for (n, m) in SWEEP] + [(SH_M, SH_K, SH_TOK, SH_N, SH_MM, 0.02, 4)]
    for (M, K, TOK, n, m, scale, reps) in cases:
        w = (torch.randn(M, K, generator=torch.Generator(device=dev).manual_seed(0), device=dev) * scale).bfloat16()
        dy = torch.randn(TOK, M, generator=torch.Generator(device=dev).manual_seed(2), device=dev).bfloat16()
        val, idx = ops.sparsify(w.unsqueeze(0), n, m, G)
        del w
        dense = ops.densify(val, idx, 1, M, K, n, m, G)[0]
        sp24 = ops.pack_sp24(val, idx, M, K, n, m, G)
        t_sp = timed(lambda: ops.spmm_t(val, idx, M, K, n, m, G, dy), reps)
        t_kept = timed(lambda: ops.spmm_t(val, idx, M, K, n, m, G, dy, sp24=sp24), reps)
        t_rate = timed(lambda: ops.spmm_t(val, idx, M, K, n, m, G, dy, algo=nat.NMG_ALGO_TENSOR_DENSE), reps)
        t_cublas = timed(lambda: torch.mm(dy, dense), reps)
        dx = ops.spmm_t(val, idx, M, K, n, m, G, dy, sp24=sp24)
        cols = sampled_rows(torch, CHECK_ROWS, K, 13, dev)
        err = rel_fro(dx[:, cols], dy.double() @ dense[:, cols].double())
        flops_dense = 2.0 * M * K * TOK
        rows.append({"shape": f"{M}x{K}x{TOK}", "nm": f"{n}:{m}", "dtype": "bf16",
                     "ms_sparse_mma": t_sp, "ms_sparse_mma_kept_copy": t_kept, "ms_dense_rate_kernels": t_rate, "cublas_dense_ms": t_cublas,
                     "speedup_vs_cublas": t_cublas / t_kept, "speedup_vs_dense_rate_kernels": t_rate / t_kept,
                     "dense_equivalent_tflops": flops_dense / t_kept / 1e9, "useful_tflops": flops_dense * n / m / t_kept / 1e9,
                     "frac_of_sparse_tensor_peak": flops_dense / t_kept / 1e9 / (2 * peaks["bf16_tflops"]),
                     "rel_fro_vs_float64": err, "tolerance": TOL["bf16"]})
        del val, idx, dense, sp24, dy, dx
        torch.cuda.empty_cache()
    return rows


def run_ours(args):
    import torch
    import torch.distributed as dist
    import sten_b200 as sten
    from sten_b200 import _native as nat, ops
    from sten_b200.sharded import RowShardedNMMatmul

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sten.set_dispatch_failure("raise")
    peaks, peaks_src = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.workload == "sharded":
        M, K, TOK, n, m = SH_M, SH_K, SH_TOK, SH_N, SH_MM
        gen = torch.Generator(device=dev).manual_seed(0)
        rounds = (args.rounds or (1 if args.exchange == "peer" else 4)) if world > 1 else 1
        rp = RowShardedNMMatmul.panel_rows(M, world, rounds, m)
        owned = {(p * world + rank): p for p in range(rounds)}  # global panel index -> local round
        # the same seeded stream on every rank; only this rank's row panels are kept (block-cyclic over ranks)
        panels_dense = [None] * rounds
        check_q = (rank + 1) % world  # global index of a panel ANOTHER rank computes (round 0): the output check below uses it
        check_dense = None
        for q in range(world * rounds):
            blk = (torch.randn(rp, K, generator=gen, device=dev) * 0.02).bfloat16()
            if q in owned:
                panels_dense[owned[q]] = blk
            if q == check_q:
                check_dense = blk
            del blk
        x = torch.randn(TOK, K, generator=torch.Generator(device=dev).manual_seed(1), device=dev).bfloat16()
        panels = [sten.GroupedNMTensor.from_dense(wd, n, m, sparse_dim=0, group_size=G, group_dim=1) for wd in panels_dense]
        del panels_dense
        layer = RowShardedNMMatmul(panels, M, exchange=args.exchange)
        layer.multicast = not args.no_multicast
        peer = args.exchange == "peer" and world > 1  # the layer then owns the (peer-mapped) output buffer
        y_dev = None if peer else torch.empty(M, TOK, dtype=torch.bfloat16, device=dev)
        total_flops = useful_flops(M, K, TOK, n, m)
        launches_per_step = 2 * rounds  # expansion pass + matmul kernel per panel

        def step():
            # peer exchange: the layer returns one of its two peer-mapped buffers (they alternate between calls)
            return layer(x, out=None if peer else y_dev)

        exchange_used = args.exchange if world > 1 else "none"
        if peer:
            # allocates and maps the output buffers once, outside the timed region; if any rank cannot map its peers'
            # buffers, every rank falls back to the NCCL all-gather exchange (and the result says so)
            try:
                y_dev = layer(x)
                ok = 1.0
            except Exception as exc:  # noqa: BLE001 - reported through exchange_used
                ok, peer_error = 0.0, f"{type(exc).__name__}: {exc}"[:160]
            flag = torch.tensor([ok], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if float(flag.item()) < 1.0:
                layer = RowShardedNMMatmul(panels, M, exchange="gather")
                peer = False
                y_dev = torch.empty(M, TOK, dtype=torch.bfloat16, device=dev)
                exchange_used = "gather (peer mapping failed" + (": " + peer_error if ok == 0.0 else " on another rank") + ")"

        x_host = torch.empty(TOK, K, dtype=torch.bfloat16).pin_memory()
        x_host.copy_(x)
        y_host = torch.empty(M, TOK, dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            # pinned host operands in, pinned host result out: chunked 3-stream pipeline on one GPU; on several, every
            # rank uploads 1/N of X (completed over NVLink) and downloads the rows it computed
            layer.forward_host(x_host, y_host)

        h2d, d2h = x_host.numel() * 2, y_host.numel() * 2  # summed over ranks: every byte of X goes up once, of C comes down once
        dtype_name, scaling = "bf16", "strong"

        def check_output(y_last):
            """Sampled parity check of the step's result, after the timed loop: CHECK_ROWS rows of C that ANOTHER rank
            produced (rank r checks the panel of rank r+1, read from its own copy of C, so the exchange is verified as
            well) against float64 dot products of the densified weight rows with X.  One rank: its own rows."""
            val_c, idx_c = ops.sparsify(check_dense.unsqueeze(0), n, m, G)
            rows = sampled_rows(torch, CHECK_ROWS, rp, 17 + rank, dev)
            w_rows = ops.densify(val_c, idx_c, 1, rp, K, n, m, G)[0][rows].double()
            want = w_rows @ x.double().t()
            return rel_fro(y_last[check_q * rp + rows], want), int(rows.numel())

        def check_e2e(y_last):
            """The end-to-end leg's host result against the device-resident one, on this rank's rows (the rows it downloads)."""
            errs = []
            for p_ in range(rounds):
                q = p_ * world + rank
                errs.append(rel_fro(y_host[q * rp:(q + 1) * rp].to(dev), y_last[q * rp:(q + 1) * rp]))
            return max(errs)
    else:
        M, K, TOK = SW_M, SW_K, SW_TOK
        w = torch.randn(M, K, generator=torch.Generator().manual_seed(0)).to(dev)
        x_host = torch.randn(TOK, K, generator=torch.Generator().manual_seed(1 + rank)).pin_memory()
        x = x_host.to(dev)
        packs = {nm: ops.sparsify(w.unsqueeze(0), nm[0], nm[1], G) for nm in SWEEP}
        outs = {nm: torch.empty(TOK, M, device=dev) for nm in SWEEP}
        total_flops = world * sum(useful_flops(M, K, TOK, n, m) for n, m in SWEEP)
        launches_per_step = 2 * len(SWEEP)  # activation re-layout + matmul kernel per call

        def step():
            for (n, m) in SWEEP:
                val, idx = packs[(n, m)]
                ops.spmm(val, idx, M, K, n, m, G, x, out=outs[(n, m)])

        sb = sten.SparsityBuilder()
        layers = torch.nn.ModuleList([torch.nn.Linear(K, M, bias=False, device=dev) for _ in SWEEP])
        for i, (n, m) in enumerate(SWEEP):
            layers[i].weight.data.copy_(w)
            sb.set_weight(f"{i}.weight", initial_sparsifier=sten.GroupedNMSparsifier(n, m, G), out_format=sten.GroupedNMTensor)
        sparse_layers = sb.sparsify_model_inplace(layers)
        y_hosts = [torch.empty(TOK, M).pin_memory() for _ in SWEEP]

        def e2e_step():
            xd = x_host.to(dev, non_blocking=True)
            with torch.no_grad():
                for lyr, yh in zip(sparse_layers, y_hosts):
                    yh.copy_(lyr(xd), non_blocking=True)

        h2d, d2h = x_host.numel() * 4, sum(y.numel() * 4 for y in y_hosts)
        dtype_name, scaling = "f32", "weak"

        def check_output(_):
            """Sampled parity check after the timed loop: CHECK_ROWS output features of every pattern against float64."""
            worst = 0.0
            for (n_, m_) in SWEEP:
                val_, idx_ = packs[(n_, m_)]
                rows = sampled_rows(torch, CHECK_ROWS, M, 17 + rank, dev)
                w_rows = ops.densify(val_, idx_, 1, M, K, n_, m_, G)[0][rows].double()
                worst = max(worst, rel_fro(outs[(n_, m_)][:, rows], x.double() @ w_rows.t()))
            return worst, CHECK_ROWS * len(SWEEP)

        def check_e2e(_):
            return max(rel_fro(yh.to(dev), outs[nm]) for yh, nm in zip(y_hosts, SWEEP))

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # sampled from the warm-up steps (same kernels, same load) to the end of the end-to-end leg
    for _ in range(args.warmup):
        step()
    ms_per_step = timed_loop(step, args.steps, barrier, torch, dist, world, dev)
    value = total_flops / (ms_per_step * 1e-3) / 1e9
    y_last = step()  # one more (untimed) step whose result is checked; the timed steps computed exactly this
    chk_err, chk_rows = check_output(y_last)

    for _ in range(2):
        e2e_step()
    k_e2e = max(2, args.steps // 2)
    ms_e2e = timed_loop(e2e_step, k_e2e, barrier, torch, dist, world, dev)
    clocks = sampler.stop() if rank == 0 else None
    e2e_value = total_flops / (ms_e2e * 1e-3) / 1e9
    torch.cuda.synchronize()
    e2e_err = check_e2e(y_last)
    tol = TOL[dtype_name]
    if world > 1:
        t = torch.tensor([chk_err, e2e_err], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        chk_err, e2e_err = float(t[0].item()), float(t[1].item())
    check = {"rel_fro": chk_err, "rows": chk_rows * world, "tokens": TOK, "tolerance": tol,
             "against": "float64 dot products of the densified weight rows; every rank checks rows of C that another rank produced, read from its own buffer"
                        if world > 1 else "float64 dot products of the densified weight rows",
             "e2e_rel_fro_vs_device_result": e2e_err, "max_over_ranks": True}
    failed = not (chk_err <= tol and e2e_err <= tol)

    # the metric's second half: sparse-encoder tokens/s at this N (every rank takes part; batch split over the ranks)
    encoder = None
    if args.workload == "sharded" and not args.no_encoder:
        try:
            encoder = encoder_numbers(torch, dist, world, rank, dev, max(5, args.steps // 2), 3, barrier)
        except ImportError as exc:  # transformers missing: the matmul result stands on its own
            encoder = {"unavailable": f"{type(exc).__name__}: {exc}"[:120]}
        torch.cuda.empty_cache()

    result = None
    if rank == 0:
        L = nat.lib()
        fma = ctypes.c_double(0.0)
        nat.check(L.nmg_measure_fma_peak(ctypes.byref(fma), torch.cuda.current_stream().cuda_stream))
        if args.workload == "sharded":
            from sten_b200.sharded import _default_matmul_rows
            kms = kernel_time(lambda: _default_matmul_rows(panels[0], x, y_dev[:rp]), torch, nat)
            alg = useful_flops(rp, K, TOK, n, m)
            achieved = alg / (kms * 1e-3) / 1e12
            peak = peaks["bf16_tflops"]
            roofline = {"bound": "tensor",
                        "kernel": "gemm_tc_kernel<bf16> (persistent TMA-fed tcgen05 matmul) + expand_dense_kernel<bf16> (weight expansion pass), timed together",
                        "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "peak_source": f"{peaks_src} bf16_tflops (burst: the call is timed alone), of measured",
                        "traffic": NCU_DRAM_BYTES_PER_CALL if world == 1 else None,
                        "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of both kernels of one full-size call "
                                          "(profiles/gemm_tc_two_pass_2-8_16384x16384_bf16_launches.txt); operands + result are 1.7 GB",
                        "ms_per_launch": kms, "algorithmic_flops_per_launch": alg,
                        "executed_tflops": achieved * m / n, "executed_frac": achieved * m / n / peak,
                        "ceiling_frac": n / m, "frac_of_ceiling": achieved * m / n / peak,
                        "note": "algorithmic = useful (non-zero) flops 2*M*K*tokens*n/m; the n:m blocks lie along the output-row axis, "
                                "so the tensor cores execute the dense product (m/n times as many flops) and frac cannot exceed n/m"}
        else:
            n, m = 2, 4
            val, idx = packs[(n, m)]
            kms = kernel_time(lambda: ops.spmm(val, idx, M, K, n, m, G, x, out=outs[(n, m)]), torch, nat)
            alg = useful_flops(M, K, TOK, n, m)
            achieved = alg / (kms * 1e-3) / 1e12
            roofline = {"bound": "fma", "kernel": "spmm_fwd_simt_kernel<2,4> fp32", "achieved": achieved, "peak": fma.value,
                        "unit": "TFLOP/s", "frac": achieved / fma.value if fma.value else None,
                        "peak_source": "fp32 FFMA loop measured in this run (nmg_measure_fma_peak)", "traffic": None,
                        "ms_per_launch": kms, "algorithmic_flops_per_launch": alg}
        # format conversion of the step's weight (N = 1: the whole 16384^2 bf16 matrix): sparsifier and densifier against the
        # HBM roofline on their algorithmic bytes (dense read + val / idx written, resp. val / idx read + dense written)
        convert = None
        if world == 1 and args.workload == "sharded":
            def timed_ms(fn, reps=5):
                fn()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(reps):
                    fn()
                b.record()
                torch.cuda.synchronize()
                return a.elapsed_time(b) / reps
            wd = check_dense.unsqueeze(0)
            val_c, idx_c = ops.sparsify(wd, n, m, G)
            nbytes = wd.numel() * 2 + val_c.numel() * 2 + idx_c.numel() * 2
            ms_s = timed_ms(lambda: ops.sparsify(wd, n, m, G))
            ms_d = timed_ms(lambda: ops.densify(val_c, idx_c, 1, rp, K, n, m, G))
            hbm = peaks["hbm_gbs"]
            convert = {"weight": f"{rp}x{K} bf16 {n}:{m} g={G}", "algorithmic_bytes": nbytes,
                       "sparsify": {"ms": ms_s, "gbs": nbytes / ms_s / 1e6, "frac": nbytes / ms_s / 1e6 / hbm},
                       "densify": {"ms": ms_d, "gbs": nbytes / ms_d / 1e6, "frac": nbytes / ms_d / 1e6 / hbm},
                       "peak_gbs": hbm, "peak_source": f"{peaks_src} hbm_gbs, of measured"}
            del val_c, idx_c, wd
        sweep = transposed = None
        if world == 1 and not args.no_sweep:
            if args.workload == "sharded":
                del layer, panels, x, y_dev, y_last
                torch.cuda.empty_cache()
            sweep = sweep_table(torch, ops, nat, dev, peaks, fma.value)
            transposed = transposed_table(torch, ops, nat, dev, peaks)
        cpu = None
        if world == 1:  # the CPU baseline is reported at N = 1 only; `bench.py --impl reference` times it at every N
            dt, flops, kind, cores, desc = time_cpu(args.workload, 3, 1)
            cpu = {"value": flops / dt / 1e9, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc + ", 3 timed passes"}
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": dtype_name, "data": "synthetic", "config": config_dict(args.workload, world, exchange_used if args.workload == "sharded" else "none", rounds if args.workload == "sharded" else 1),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": args.steps * launches_per_step, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "fp32_fma_peak_tflops": fma.value, "sweep": sweep, "transposed": transposed, "check": check, "encoder": encoder, "convert": convert,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if result is not None:
        print(json.dumps(result))
    if failed:
        print(f"output check failed: rel. Frobenius error {chk_err:.3e} (end to end {e2e_err:.3e}) above {tol}", file=sys.stderr)
        return 1
    return 0


def encoder_numbers(torch, dist, world, rank, dev, steps, warmup, barrier):
    """BERT-large-shaped encoder (24 layers, hidden 1024, FFN 4096, 16 heads, random init seed 0, fp16) with every encoder
    Linear weight at nmg 2:4 (g = 16) through SparsityBuilder, bias + GELU and bias + residual fused into the matmul
    epilogue (fuse_linear_epilogues); attention stays dense.  Inference on 32 x 384 random token ids (seed 1), the batch
    split evenly over the ranks (no collective).  tokens/s eager and as a replayed CUDA graph, next to the dense fp16 model,
    and the last hidden state checked against the same model with densified weights."""
    import copy
    import sten_b200 as sten
    from transformers import BertConfig, BertModel

    BATCH, SEQ = 32, 384
    cfg = BertConfig(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096,
                     vocab_size=30522, max_position_embeddings=512)
    torch.manual_seed(0)
    model = BertModel(cfg, add_pooling_layer=False).half().to(dev).eval()
    names = [n + ".weight" for n, mod in model.named_modules() if isinstance(mod, torch.nn.Linear) and "encoder.layer" in n]
    sb = sten.SparsityBuilder()
    for w in names:
        sb.set_weight(name=w, initial_sparsifier=sten.GroupedNMSparsifier(n=2, m=4, g=G), out_format=sten.GroupedNMTensor)
    dense_model = model
    sparse_model = sb.sparsify_model_inplace(copy.deepcopy(model))
    fused = sten.fuse_linear_epilogues(sparse_model)
    # the same network with the sparse weights written back densely: what the sparse model must reproduce
    densified = copy.deepcopy(model)
    sparse_params = dict(sparse_model.named_parameters())
    with torch.no_grad():
        for name, prm in densified.named_parameters():
            if name in names:
                prm.copy_(sparse_params[name].wrapped_tensor.to_dense())
    per_rank = BATCH // world
    ids_all = torch.randint(0, 30522, (BATCH, SEQ), generator=torch.Generator().manual_seed(1))
    ids = ids_all[rank * per_rank:(rank + 1) * per_rank].to(dev)

    def fwd(m, batch_ids=None):
        # embeddings + encoder stack called directly with no attention mask (the batch has no padding): the model's own
        # mask preparation keeps an all-ones mask while a CUDA graph is being captured, which pushes attention onto a
        # slow fp32 path in the captured graph only; without a mask eager and captured runs use the same fused attention
        with torch.no_grad():
            return m.encoder(m.embeddings(input_ids=ids if batch_ids is None else batch_ids), attention_mask=None).last_hidden_state

    for _ in range(max(warmup, 3)):
        out = fwd(sparse_model)
    ref = fwd(densified)
    err = rel_fro(out, ref)
    del densified, ref
    ms_eager = timed_loop(lambda: fwd(sparse_model), steps, barrier, torch, dist, world, dev)
    for _ in range(3):
        fwd(dense_model)
    ms_dense = timed_loop(lambda: fwd(dense_model), steps, barrier, torch, dist, world, dev)

    # CUDA graphs of both forwards: removes the host-side dispatch cost (144 sparse linears go through the plugin)
    def graphed(m, batch_ids=None):
        try:
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fwd(m, batch_ids)
            torch.cuda.current_stream().wait_stream(side)
            with torch.cuda.graph(g):
                static_out = fwd(m, batch_ids)  # noqa: F841 - keeps the graph's output alive
            return timed_loop(g.replay, steps, barrier, torch, dist, world, dev)
        except Exception:  # graph capture is an optimisation of the host path, not part of the result's validity
            return None

    ms_graph = graphed(sparse_model)
    ms_graph_dense = graphed(dense_model)
    # Several ranks: besides the split batch, the data-parallel serving case -- every replica takes a whole batch of 32
    # (no collective either; per-GPU work as at N = 1)
    replicas = None
    if world > 1:
        ids_full = ids_all.to(dev)
        for _ in range(3):
            fwd(sparse_model, ids_full)
            fwd(dense_model, ids_full)
        ms_full = graphed(sparse_model, ids_full) or timed_loop(lambda: fwd(sparse_model, ids_full), steps, barrier, torch, dist, world, dev)
        ms_full_dense = graphed(dense_model, ids_full) or timed_loop(lambda: fwd(dense_model, ids_full), steps, barrier, torch, dist, world, dev)
        replicas = {"tokens_per_s": world * BATCH * SEQ / (ms_full * 1e-3), "dense_tokens_per_s": world * BATCH * SEQ / (ms_full_dense * 1e-3),
                    "speedup_vs_dense_fp16": ms_full_dense / ms_full,
                    "workload": f"batch 32 x seq 384 on each of the {world} ranks (weak scaling), slowest rank's time"}
    # opt-in variant: every weight keeps its expanded 16-bit copy (set_spmm_opt(kernel="sm100-expanded")): no expansion pass
    # per call, no memory saving; reported beside the default, never as the headline
    for name, prm in sparse_model.named_parameters():
        if name in names:
            prm.wrapped_tensor.set_spmm_opt(kernel="sm100-expanded")
    for _ in range(3):
        out_exp = fwd(sparse_model)
    err_exp = rel_fro(out_exp, out)
    ms_exp_eager = timed_loop(lambda: fwd(sparse_model), steps, barrier, torch, dist, world, dev)
    ms_exp_graph = graphed(sparse_model)
    ms_exp = min(ms_exp_eager, ms_exp_graph) if ms_exp_graph else ms_exp_eager
    toks = BATCH * SEQ
    # headline: the captured graph when capture worked (steady-state serving replays a graph; every replay recomputes the
    # whole forward through the same plugin calls), else the eager loop
    ms_best = min(ms_eager, ms_graph) if ms_graph else ms_eager
    ms_dense_best = min(ms_dense, ms_graph_dense) if ms_graph_dense else ms_dense
    return {
        "tokens_per_s": toks / (ms_best * 1e-3), "ms_per_forward": ms_best,
        "execution": "cuda graph replay" if ms_graph and ms_graph <= ms_eager else "eager",
        "eager_tokens_per_s": toks / (ms_eager * 1e-3),
        "cuda_graph_tokens_per_s": (toks / (ms_graph * 1e-3)) if ms_graph else None,
        "dense_tokens_per_s": toks / (ms_dense_best * 1e-3),
        "dense_fp16_eager_tokens_per_s": toks / (ms_dense * 1e-3),
        "dense_fp16_cuda_graph_tokens_per_s": (toks / (ms_graph_dense * 1e-3)) if ms_graph_dense else None,
        "speedup_vs_dense_fp16": ms_dense_best / ms_best,
        "expanded_weights_opt_in": {"tokens_per_s": toks / (ms_exp * 1e-3), "speedup_vs_dense_fp16": ms_dense_best / ms_exp,
                                    "rel_fro_vs_default_path": err_exp,
                                    "note": "set_spmm_opt(kernel='sm100-expanded'): the expanded 16-bit weight is kept across calls"},
        "one_batch_per_rank": replicas,
        "sparse_linears_per_forward": len(names), "fused_epilogue_modules": fused,
        "rel_fro_vs_densified_model": err, "output_finite": bool(torch.isfinite(out.float()).all()),
        "config": {"workload": "BERT-large-shaped encoder, 24 layers, all encoder linears nmg 2:4 g=16 fp16, batch 32 x seq 384",
                   "parallelism": f"batch split over {world} rank(s), no collective"},
    }


def run_encoder(args):
    import torch
    import torch.distributed as dist
    import sten_b200 as sten

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sten.set_dispatch_failure("raise")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    enc = encoder_numbers(torch, dist, world, rank, dev, args.steps, args.warmup, barrier)
    if rank == 0:
        line = {"metric": "sparse_encoder_tokens_per_s", "value": enc["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": enc["ms_per_forward"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic"}
        line.update(enc)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="sharded", choices=["sharded", "sweep", "encoder"])
    ap.add_argument("--rounds", type=int, default=0, help="row panels per rank when N > 1 (default: 1 for --exchange peer, 4 for gather)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "gather"],
                    help="how row shards combine their output slices when N > 1: stores into every rank's buffer from the matmul epilogue, or NCCL all-gathers")
    ap.add_argument("--no-multicast", action="store_true", help="peer exchange with one store per destination instead of NVSwitch multicast stores")
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-pattern 4096^2 table")
    ap.add_argument("--no-encoder", action="store_true", help="skip the sparse-encoder tokens/s block of the default workload")
    args = ap.parse_args()
    if args.workload == "encoder":
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference cannot run this encoder on its CPU path in bounded time; "
                                  "its per-layer matmul is what the default workload's reference arm times"}))
            return 0
        return run_encoder(args)
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
