"""Build the reference's own CPU-SIMD nmg matmul into ``oracle/_ref/`` (TEST INFRASTRUCTURE ONLY).

The reference emits its AVX2 / AVX-512 micro-kernels as text at run time
(``generate_sparse_dense_microkernel_avx2`` / ``_avx512``, src/sten/grouped_nm/dace_gnm_mult.py:23-256) and hands
them to the DaCe compiler, which only schedules them (loop nest of dace_gnm_mult.py:724-805).  DaCe is a
third-party package that is not installed, so this script

  1. imports the reference package from its own tree (a stub stands in for the ``dace`` module, which is
     only touched inside ``nmg_mult``),
  2. asks the reference generators for the micro-kernel text of one (n, m, g, K) problem, using the stride
     arguments ``nmg_mult`` passes for ``local_b = local_c = True`` (dace_gnm_mult.py:615-646),
  3. wraps it in the small OpenMP driver below, which follows the reference loop nest (token-block panel
     copy with transpose, full k-chunks x row-blocks, k-remainder chunk, panel write-back), and
  4. compiles it with g++.  The rendered source lives in a temporary directory; only the shared objects are
     kept, in ``oracle/_ref/`` (git-ignored).  Nothing from the reference is copied into the repository.

The reference compiles with ``-march=native`` (native_scripting.py:50).  The objects built here must also run
on a different host, so the ISA is named explicitly (``-mavx2 -mfma`` or ``-mavx512f``) and picked at load
time from the CPU flags the same way the reference picks it (grouped_nm_tensor.py:893-897).

Usage:  python oracle/build_ref.py --reference /path/to/reference     (builds the default problem list; the path may
        also come from the environment variable NMG_REFERENCE_ROOT)
"""
import argparse
import ctypes
import math
import os
import subprocess
import sys
import tempfile
import types

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")

# (n, m, g, K): the problems of the benchmark configurations and of the golden fixtures.
DEFAULT_PROBLEMS = [
    (2, 4, 4, 1024), (2, 4, 16, 1024),                        # 1024 x 1024 plumbing case
    (1, 4, 16, 768), (1, 4, 16, 3072),                        # BERT-base FFN pair
    (1, 4, 16, 4096), (2, 4, 16, 4096), (1, 8, 16, 4096), (2, 8, 16, 4096), (1, 16, 16, 4096),  # density sweep
    (2, 4, 16, 16384), (2, 8, 16, 16384),                     # large sharded case
    (2, 4, 2, 100), (1, 4, 3, 50), (2, 8, 2, 120), (3, 6, 4, 96),  # small fixtures with k-remainders
]

DRIVER = r"""
#include <immintrin.h>
#include <omp.h>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#define FOR(i, n) for (int i = 0; i < n; ++i)
static const int V4 = %(v4)d;      // tokens per block = 4 vectors
static const int KK = %(K)d;       // reduction length baked into the micro-kernels
static const int CC = %(cc)d;      // columns per chunk
static const int MM = %(m)d;
static const int NN = %(n)d;

static inline void tile_full(const float* ptr_a_val, const int16_t* ptr_a_idx, float* ptr_b, float* ptr_c) {
%(code_full)s
}
static inline void tile_rem(const float* ptr_a_val, const int16_t* ptr_a_idx, float* ptr_b, float* ptr_c) {
%(code_rem)s
}

extern "C" int nmg_ref_tokens_per_block() { return V4; }
// OpenMP team size, stated by the caller instead of inherited from OMP_NUM_THREADS (launchers export 1 for their workers)
extern "C" void nmg_ref_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
extern "C" int nmg_ref_num_threads() { return omp_get_max_threads(); }

// out[tok][Mp] = X[tok][K] * densify(A)^T ; ntok must be a multiple of V4 (dace_gnm_mult.py:605-606)
extern "C" int nmg_ref_spmm(const int16_t* A_idx, const float* A_val, const float* X, float* out,
                            int64_t ntok, int64_t M) {
    if (ntok %% V4 != 0) return -1;
    const int64_t nb = (M + MM - 1) / MM, Mp = nb * MM;
    const int64_t nc = (KK + CC - 1) / CC;
    const bool has_rem = (KK %% CC) != 0;
    const int64_t nfull = has_rem ? nc - 1 : nc;
    #pragma omp parallel
    {
        float* Bl = (float*)aligned_alloc(64, sizeof(float) * (size_t)KK * V4);
        float* Cl = (float*)aligned_alloc(64, sizeof(float) * (size_t)Mp * V4);
        #pragma omp for schedule(dynamic, 1)
        for (int64_t bn = 0; bn < ntok / V4; ++bn) {
            for (int64_t t = 0; t < V4; ++t)
                for (int64_t k = 0; k < KK; ++k) Bl[k * V4 + t] = X[(bn * V4 + t) * KK + k];
            memset(Cl, 0, sizeof(float) * (size_t)Mp * V4);
            for (int64_t bk = 0; bk < nfull; ++bk)
                for (int64_t bm = 0; bm < nb; ++bm)
                    tile_full(A_val + (bk * nb + bm) * CC * NN, A_idx + (bk * nb + bm) * CC,
                              Bl + bk * CC * V4, Cl + bm * MM * V4);
            if (has_rem)
                for (int64_t bm = 0; bm < nb; ++bm)
                    tile_rem(A_val + (nfull * nb + bm) * CC * NN, A_idx + (nfull * nb + bm) * CC,
                             Bl + nfull * CC * V4, Cl + bm * MM * V4);
            for (int64_t t = 0; t < V4; ++t)
                for (int64_t r = 0; r < Mp; ++r) out[(bn * V4 + t) * Mp + r] = Cl[r * V4 + t];
        }
        free(Bl); free(Cl);
    }
    return 0;
}
"""


def import_reference(ref_root):
    stub = types.ModuleType("dace")
    stub.nodes = types.ModuleType("dace.nodes")
    stub.SDFG = object
    stub.SDFGState = object
    sys.modules.setdefault("dace", stub)
    sys.modules.setdefault("dace.nodes", stub.nodes)
    src = os.path.join(ref_root, "src")
    if src not in sys.path:
        sys.path.insert(0, src)
    cwd = os.getcwd()
    os.chdir(tempfile.gettempdir())  # the reference writes ./.compile_cache
    try:
        import sten  # noqa: F401
        from sten.grouped_nm import dace_gnm_mult
    finally:
        os.chdir(cwd)
    return dace_gnm_mult


def lib_name(n, m, g, K, isa):
    return f"libnmg_ref_{n}_{m}_{g}_K{K}_{isa}.so"


def build_one(gen_mod, n, m, g, K, isa, verbose=False):
    v = 8 if isa == "avx2" else 16
    gen = getattr(gen_mod, f"generate_sparse_dense_microkernel_{isa}")
    cc = math.comb(m, n) * g
    common = dict(ptr_a_val="ptr_a_val", ptr_a_idx="ptr_a_idx", ptr_b="ptr_b", ptr_c="ptr_c", M=m, Nblocks=1,
                  SAMS=1, SAKS=n, SAMI=1, SAKI=1, SBV=1, SBB=v, SBK=4 * v, SCM=4 * v, SCB=v, SCV=1,
                  n=n, m=m, g=g, num_vectors_b=4, v=v)
    code_full = gen(K=cc, **common)
    code_rem = gen(K=K % cc, **common) if K % cc else ";"
    src = DRIVER % dict(v4=4 * v, K=K, cc=cc, m=m, n=n, code_full=code_full, code_rem=code_rem)
    os.makedirs(OUT_DIR, exist_ok=True)
    out = os.path.join(OUT_DIR, lib_name(n, m, g, K, isa))
    isa_flags = ["-mavx2", "-mfma"] if isa == "avx2" else ["-mavx512f", "-mavx2", "-mfma"]
    with tempfile.TemporaryDirectory() as tmp:
        cpp = os.path.join(tmp, "ref_kernel.cpp")
        with open(cpp, "w") as f:
            f.write(src)
        cmd = ["g++", "-O3", *isa_flags, "-fopenmp", "-shared", "-fPIC", "-o", out, cpp]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return out


def reference_root(explicit=None):
    """Path of the reference tree: the argument, else $NMG_REFERENCE_ROOT; None when neither names a tree."""
    root = explicit or os.environ.get("NMG_REFERENCE_ROOT")
    return root if root and os.path.isdir(os.path.join(root, "src", "sten")) else None


def is_current():
    """Whether oracle/_ref holds every default problem, built from this version of the driver."""
    isa = host_isa()
    for (n, m, g, K) in DEFAULT_PROBLEMS:
        path = os.path.join(OUT_DIR, lib_name(n, m, g, K, isa))
        if not os.path.isfile(path):
            return False
        try:
            ctypes.CDLL(path).nmg_ref_set_threads
        except (OSError, AttributeError):
            return False
    return True


def build_all(ref_root, problems=None, verbose=False):
    gen_mod = import_reference(ref_root)
    built = []
    for (n, m, g, K) in problems or DEFAULT_PROBLEMS:
        for isa in ("avx2", "avx512"):
            built.append(build_one(gen_mod, n, m, g, K, isa, verbose))
    return built


# ---- loading (no reference tree needed) -------------------------------------------------------------------
def host_isa():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return "avx512" if " avx512f" in line else "avx2"
    except OSError:
        pass
    return "avx2"


def load(n, m, g, K, isa=None):
    """Return (callable, tokens_per_block) for a prebuilt problem, or None when it was not built."""
    isa = isa or host_isa()
    path = os.path.join(OUT_DIR, lib_name(n, m, g, K, isa))
    if not os.path.isfile(path):
        return None
    L = ctypes.CDLL(path)
    L.nmg_ref_spmm.restype = ctypes.c_int
    L.nmg_ref_spmm.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int64]
    L.nmg_ref_tokens_per_block.restype = ctypes.c_int
    L.nmg_ref_set_threads.argtypes = [ctypes.c_int]
    L.nmg_ref_set_threads.restype = None
    if _THREADS:
        L.nmg_ref_set_threads(_THREADS)
    return L.nmg_ref_spmm, int(L.nmg_ref_tokens_per_block())


_THREADS = 0


def set_threads(n):
    """OpenMP team size for every kernel loaded from now on (each shared object carries the same OpenMP runtime, so one
    call per load is enough)."""
    global _THREADS
    _THREADS = int(n)


def spmm(val, idx, x, M, K, n, m, g, isa=None):
    """numpy front-end: y[tokens, Mp] = x[tokens, K] @ densify(val, idx)^T with the reference micro-kernels."""
    import numpy as np
    got = load(n, m, g, K, isa)
    if got is None:
        raise FileNotFoundError("reference kernel for this problem was not built")
    fn, tb = got
    val = np.ascontiguousarray(val, dtype=np.float32)
    idx = np.ascontiguousarray(idx, dtype=np.int16)
    x = np.ascontiguousarray(x, dtype=np.float32)
    ntok = x.shape[0]
    pad = (-ntok) % tb
    if pad:
        x = np.concatenate([x, np.zeros((pad, K), np.float32)])
    Mp = -(-M // m) * m
    out = np.zeros((ntok + pad, Mp), dtype=np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    rc = fn(p(idx), p(val), p(x), p(out), ntok + pad, M)
    if rc != 0:
        raise ValueError("reference kernel rejected the problem")
    return out[:ntok]


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="root of the reference tree (or set NMG_REFERENCE_ROOT)")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    root = reference_root(a.reference)
    if root is None:
        ap.error("no reference tree: pass --reference or set NMG_REFERENCE_ROOT")
    for pth in build_all(root, verbose=a.verbose):
        print(pth)
