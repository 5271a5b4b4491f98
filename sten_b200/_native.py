"""ctypes binding of ``libnmg_b200.so`` (the C ABI declared in ``include/nmg_b200.h``).

The library is the only implementation of the arithmetic: if it cannot be loaded, or a tensor is not on a
CUDA device, the operations raise -- there is no CPU or eager-PyTorch fallback.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnmg_b200.so")

NMG_F32, NMG_F16, NMG_BF16 = 0, 1, 2
NMG_ACT_TOKEN_MAJOR, NMG_ACT_K_MAJOR, NMG_ACT_TOKEN_MAJOR_OUT_ROWS = 0, 1, 2
NMG_ALGO_AUTO, NMG_ALGO_SIMT, NMG_ALGO_TENSOR, NMG_ALGO_TENSOR_DENSE = 0, 1, 2, 3
NMG_NOALLOC_SCRATCH_BYTES = 32 << 20
NMG_EPI_NONE, NMG_EPI_GELU = 0, 1

# name -> (restype, argtypes); must list every function of include/nmg_b200.h (checked by the test-suite)
_i64, _int, _vp, _sz = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
SIGNATURES = {
    "nmg_version": (_int, []),
    "nmg_last_error": (ctypes.c_char_p, []),
    "nmg_num_patterns": (_i64, [_int, _int]),
    "nmg_pattern_order": (_int, [_int, _int, _vp]),
    "nmg_sparsify": (_int, [_vp, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _int, _vp, _vp, _vp]),
    "nmg_densify": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _int, _int, _int, _vp, _i64, _i64, _vp]),
    "nmg_gather": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _int, _vp, _vp]),
    "nmg_perfect_nm_select": (_int, [_vp, _i64, _i64, _i64, _int, _int, _int, _vp, _vp, _vp]),
    "nmg_perfect_nm_densify": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp, _vp]),
    "nmg_packed_bytes": (_sz, [_i64, _i64, _int, _int, _int, _int]),
    "nmg_pack": (_int, [_vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _sz, _vp]),
    "nmg_spmm_workspace_bytes": (_sz, [_i64, _i64, _i64, _int, _int, _int, _int, _int, _int, _int]),
    "nmg_spmm": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _i64, _i64, _vp, _vp, _i64, _int, _int,
                        _vp, _sz, _vp]),
    "nmg_spmm_fused": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _i64, _i64, _vp, _int, _vp, _i64, _vp, _i64, _int,
                              _int, _vp, _sz, _vp]),
    "nmg_spmm_t_workspace_bytes": (_sz, [_i64, _i64, _i64, _int, _int, _int, _int, _int, _int]),
    "nmg_spmm_t": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _i64, _i64, _vp, _i64, _int, _vp, _sz,
                          _vp]),
    "nmg_sp24_bytes": (_sz, [_i64, _i64, _int, _int, _int, _int]),
    "nmg_pack_sp24": (_int, [_vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _sz, _vp]),
    "nmg_spmm_t_sp24": (_int, [_vp, _i64, _i64, _int, _int, _int, _int, _vp, _i64, _i64, _vp, _i64, _vp]),
    "nmg_expanded_bytes": (_sz, [_i64, _i64, _int, _int, _int, _int]),
    "nmg_expand": (_int, [_vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _sz, _vp]),
    "nmg_spmm_expanded": (_int, [_vp, _i64, _i64, _int, _vp, _i64, _i64, _vp, _int, _vp, _i64, _vp, _i64, _int, _vp]),
    "nmg_spmm_uses_packed": (_int, [_i64, _i64, _i64, _int, _int, _int, _int, _int, _int, _int]),
    "nmg_spmm_replicated_workspace_bytes": (_sz, [_i64, _i64, _i64, _int, _int, _int, _int]),
    "nmg_spmm_replicated": (_int, [_vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _i64, _i64, _vp, _vp, _int, _vp, _i64, _vp, _sz, _vp]),
    "nmg_spmm_noalloc": (_int, [_vp, _vp, _i64, _i64, _int, _int, _int, _int, _vp, _i64, _i64, _vp, _vp, _i64, _int, _vp]),
    "nmg_profile_next": (_int, [_vp, _vp]),
    "nmg_measure_fma_peak": (_int, [ctypes.POINTER(ctypes.c_double), _vp]),
    "nmg_memcpy_2d_async": (_int, [_vp, _sz, _vp, _sz, _sz, _sz, _vp]),
    "nmg_read_status": (_int, [_vp, ctypes.POINTER(_int)]),
    "nmg_selftest_wait": (ctypes.c_int, [ctypes.c_uint64, _vp]),
}

_lib = None


class NmgError(RuntimeError):
    """A call into libnmg_b200.so returned a non-zero status."""

    def __init__(self, status, message):
        super().__init__(f"nmg_b200 status {status}: {message}")
        self.status = status


def lib():
    """Load the library once.  Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m sten_b200.build` (needs nvcc). "
                "sten_b200 has no CPU or PyTorch fallback for the grouped n:m kernels.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status):
    if status != 0:
        raise NmgError(status, lib().nmg_last_error().decode(errors="replace"))
