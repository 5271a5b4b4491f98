"""Run one kernel of the library a few times on a seeded problem, for use under a profiler.

    python profile_case.py --op fwd --nm 2:4 --g 16 --rows 4096 --cols 4096 --tokens 4096 --dtype f32 --reps 3

``--op`` is one of ``fwd`` (y = x W^T), ``fwd_rows`` (C = W x^T from token-major x), ``fwd_kmajor`` (C = W B), ``bwd`` (dX = dY W), ``sparsify``, ``densify``.
Prints the mean device time per call measured with CUDA events (meaningless under a profiler, useful without).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from sten_b200 import _native as nat  # noqa: E402
from sten_b200 import ops  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="fwd", choices=["fwd", "fwd_rows", "fwd_kmajor", "bwd", "sparsify", "densify"])
    ap.add_argument("--nm", default="2:4")
    ap.add_argument("--g", type=int, default=16)
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16", "bf16"])
    ap.add_argument("--algo", default="auto", choices=["auto", "simt", "tensor", "tensor_dense"])
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--no-packed", action="store_true", help="rebuild the column-ordered weight copy in every call")
    ap.add_argument("--bias", action="store_true", help="fwd: add a bias vector in the matmul's epilogue")
    ap.add_argument("--gelu", action="store_true", help="fwd: bias + GELU in the matmul's epilogue")
    ap.add_argument("--residual", action="store_true", help="fwd: add a residual tensor of the output's shape in the epilogue")
    ap.add_argument("--expanded", action="store_true", help="fwd: keep the expanded 16-bit weight across calls (no expansion pass per call)")
    ap.add_argument("--graph", action="store_true", help="time the repetitions as one replayed CUDA graph (no host launch cost between calls)")
    ap.add_argument("--sp24", action="store_true", help="bwd: keep the compressed transposed copy across calls (as the plugin's backward does)")
    a = ap.parse_args()
    n, m = map(int, a.nm.split(":"))
    dtype = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[a.dtype]
    algo = {"auto": nat.NMG_ALGO_AUTO, "simt": nat.NMG_ALGO_SIMT, "tensor": nat.NMG_ALGO_TENSOR, "tensor_dense": nat.NMG_ALGO_TENSOR_DENSE}[a.algo]
    dev = torch.device("cuda", 0)
    M, K, g = a.rows, a.cols, a.g
    w = torch.randn(M, K, generator=torch.Generator().manual_seed(0)).to(dev)
    val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    val = val.to(dtype)
    x = torch.randn(a.tokens, K, generator=torch.Generator().manual_seed(1)).to(dev).to(dtype)
    dy = torch.randn(a.tokens, M, generator=torch.Generator().manual_seed(2)).to(dev).to(dtype)
    xt = x.t().contiguous()
    wd = w.to(dtype).unsqueeze(0)
    packed = None if a.no_packed else ops.pack(val, idx, M, K, n, m, g)
    sp24 = ops.pack_sp24(val, idx, M, K, n, m, g) if a.sp24 else None
    bias = torch.randn(M, generator=torch.Generator().manual_seed(3)).to(dev).to(dtype) if (a.bias or a.gelu) else None
    residual = torch.randn(a.tokens, M, generator=torch.Generator().manual_seed(4)).to(dev).to(dtype) if a.residual else None
    activation = "gelu" if a.gelu else None
    expanded = ops.expand(val, idx, M, K, n, m, g) if a.expanded else None

    def call():
        if a.op == "fwd" and expanded is not None:
            return ops.spmm_expanded(expanded, M, K, x, bias=bias, activation=activation, residual=residual)
        if a.op == "fwd":
            return ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=algo, packed=packed, activation=activation, residual=residual)
        if a.op == "fwd_rows":
            return ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS, algo=algo, packed=packed)
        if a.op == "fwd_kmajor":
            return ops.spmm(val, idx, M, K, n, m, g, xt, layout=nat.NMG_ACT_K_MAJOR, algo=algo)
        if a.op == "bwd":
            return ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=algo, packed=packed, sp24=sp24)
        if a.op == "sparsify":
            return ops.sparsify(wd, n, m, g)
        return ops.densify(val, idx, 1, M, K, n, m, g)

    call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(a.reps):
                call()
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    else:
        e0.record()
        for _ in range(a.reps):
            call()
        e1.record()
    torch.cuda.synchronize()
    ops.read_status(dev)
    print(f"{a.op} {a.nm} g={g} {M}x{K} tokens={a.tokens} {a.dtype}: {e0.elapsed_time(e1) / a.reps:.4f} ms per call")


if __name__ == "__main__":
    main()
