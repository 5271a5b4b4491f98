"""ctypes front-end of the plain-C oracle (``nmg_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this module;
the shipped package must never do so.  Parity status: pinned (see the header of ``nmg_oracle.c``).

The shared object is compiled on first use for the CPU it runs on (``gcc -O3 -march=native -fopenmp``,
the flags the reference uses for its own generated CPU code: src/sten/grouped_nm/native_scripting.py:44-59)
and cached next to this file under ``_build/``, keyed by source hash and CPU flags, so a library built
on one machine is never executed on another with a different instruction set.
"""
import ctypes
import hashlib
import math
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def _cpu_key():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return hashlib.sha256(line.encode()).hexdigest()[:12]
    except OSError:
        pass
    return "generic"


def build(verbose=False):
    """Compile nmg_oracle.c for this CPU (if not cached) and return the path of the shared object."""
    src = os.path.join(_HERE, "nmg_oracle.c")
    with open(src, "rb") as f:
        key = hashlib.sha256(f.read()).hexdigest()[:12] + "_" + _cpu_key()
    for root in (os.path.join(_HERE, "_build"), os.path.join(tempfile.gettempdir(), "nmg_oracle_build")):
        out = os.path.join(root, key, "libnmg_oracle.so")
        if os.path.isfile(out):
            return out
        try:
            os.makedirs(os.path.dirname(out), exist_ok=True)
            tmp = out + f".{os.getpid()}.tmp"
            cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", "-o", tmp, src, "-lm"]
            if verbose:
                print(" ".join(cmd))
            subprocess.check_call(cmd)
            os.replace(tmp, out)
            return out
        except (OSError, subprocess.CalledProcessError):
            continue
    raise RuntimeError("could not build the CPU oracle (gcc missing or no writable directory)")


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        i64, ci, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.nmg_oracle_comb.restype = i64
        L.nmg_oracle_comb.argtypes = [ci, ci]
        L.nmg_oracle_order.restype = i64
        L.nmg_oracle_order.argtypes = [ci, ci, vp]
        L.nmg_oracle_sparsify_f32.restype = ci
        L.nmg_oracle_sparsify_f32.argtypes = [vp, i64, i64, i64, ci, ci, ci, vp, vp]
        L.nmg_oracle_densify_f32.restype = ci
        L.nmg_oracle_densify_f32.argtypes = [vp, vp, i64, i64, i64, ci, ci, ci, vp]
        L.nmg_oracle_spmm_f32.restype = ci
        L.nmg_oracle_spmm_f32.argtypes = [vp, vp, vp, i64, i64, i64, i64, ci, ci, ci, vp, i64]
        L.nmg_oracle_num_threads.restype = ci
        L.nmg_oracle_set_threads.restype = None
        L.nmg_oracle_set_threads.argtypes = [ci]
        _LIB = L
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def num_threads():
    return int(lib().nmg_oracle_num_threads())


def set_threads(n):
    """OpenMP team size of the following calls (explicit, so that an inherited OMP_NUM_THREADS=1 does not decide it)."""
    lib().nmg_oracle_set_threads(int(n))


def order(n, m):
    """Pattern order of the reference (make_n_m, grouped_nm_tensor.py:37-50) as an int8 array [C, n]."""
    C = math.comb(m, n)
    out = np.zeros((C, max(n, 1)), dtype=np.int8)[:, :n].copy()
    got = lib().nmg_oracle_order(n, m, _p(out))
    assert got == C
    return out


def geometry(M, K, n, m, g):
    C = math.comb(m, n)
    cc = C * g
    nb, nc = -(-M // m), -(-K // cc)
    return dict(C=C, cc=cc, nb=nb, nc=nc, Mp=nb * m, Kp=nc * cc)


def sparsify(dense, n, m, g):
    """dense float32 [..., M, K] -> (val [T, C, g, n] float32, idx [T, C, g, 1] int16), reference tile order."""
    dense = np.ascontiguousarray(dense, dtype=np.float32)
    M, K = dense.shape[-2:]
    B = int(np.prod(dense.shape[:-2], dtype=np.int64)) if dense.ndim > 2 else 1
    geo = geometry(M, K, n, m, g)
    T = B * geo["nc"] * geo["nb"]
    val = np.zeros((T, geo["C"], g, n), dtype=np.float32)
    idx = np.full((T, geo["C"], g, 1), -1, dtype=np.int16)
    rc = lib().nmg_oracle_sparsify_f32(_p(dense), B, M, K, n, m, g, _p(val), _p(idx))
    if rc != 0:
        raise ValueError(f"oracle sparsify failed ({rc})")
    return val, idx


def densify(val, idx, shape, n, m, g):
    """Inverse of :func:`sparsify` for a weight of the given dense shape [..., M, K]."""
    val = np.ascontiguousarray(val, dtype=np.float32)
    idx = np.ascontiguousarray(idx, dtype=np.int16)
    M, K = shape[-2:]
    B = int(np.prod(shape[:-2], dtype=np.int64)) if len(shape) > 2 else 1
    out = np.zeros(tuple(shape), dtype=np.float32)
    rc = lib().nmg_oracle_densify_f32(_p(val), _p(idx), B, M, K, n, m, g, _p(out))
    assert rc == 0
    return out


def spmm(val, idx, x, M, K, n, m, g):
    """y[tokens, Mp] = x[tokens, K] @ densify(val, idx)^T with the reference's accumulation structure."""
    val = np.ascontiguousarray(val, dtype=np.float32)
    idx = np.ascontiguousarray(idx, dtype=np.int16)
    x = np.ascontiguousarray(x, dtype=np.float32)
    ntok = x.shape[0]
    assert x.shape[1] == K
    geo = geometry(M, K, n, m, g)
    out = np.zeros((ntok, geo["Mp"]), dtype=np.float32)
    rc = lib().nmg_oracle_spmm_f32(_p(val), _p(idx), _p(x), ntok, K, M, K, n, m, g, _p(out), geo["Mp"])
    if rc != 0:
        raise ValueError(f"oracle spmm failed ({rc})")
    return out
