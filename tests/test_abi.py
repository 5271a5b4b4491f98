"""The C-ABI library: it loads, exports every symbol the public header declares, and its host-side
validation answers with status codes (no GPU needed for any call made here)."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT
from sten_b200 import _native as nat
from sten_b200.layout import make_n_m


def _declared():
    text = open(os.path.join(ROOT, "include", "nmg_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nmg_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = nat.lib()
    names = _declared()
    assert len(names) >= 15
    for name in names:
        assert hasattr(L, name), f"{name} is declared in include/nmg_b200.h but not exported"
        assert name in nat.SIGNATURES, f"{name} has no ctypes signature in sten_b200/_native.py"
    assert set(nat.SIGNATURES) == set(names)


def test_host_only_entry_points():
    L = nat.lib()
    assert L.nmg_version() >= 100
    for (n, m) in [(1, 4), (2, 4), (2, 8), (1, 16), (3, 6), (5, 12)]:
        want = make_n_m(n, m)
        assert L.nmg_num_patterns(n, m) == len(want)
        buf = np.zeros((len(want), n), dtype=np.int8)
        assert L.nmg_pattern_order(n, m, buf.ctypes.data_as(ctypes.c_void_p)) == 0
        assert [tuple(r) for r in buf.tolist()] == want


def test_invalid_arguments_return_status_not_abort():
    L = nat.lib()
    one = ctypes.c_void_p(16)  # never dereferenced: validation fails first
    # n > m
    assert L.nmg_sparsify(one, 1, 8, 8, 8, 64, 5, 4, 2, nat.NMG_F32, one, one, None) == 1
    assert b"n" in L.nmg_last_error()
    # comb(m, n) * g must fit int16
    assert L.nmg_densify(one, one, 1, 8, 8, 2, 8, 2000, nat.NMG_F32, one, 8, 64, None) == 1
    assert b"int16" in L.nmg_last_error()
    # unknown dtype
    assert L.nmg_sparsify(one, 1, 8, 8, 8, 64, 2, 4, 2, 7, one, one, None) == 1
    # NULL operands
    assert L.nmg_spmm(None, None, None, 8, 8, 2, 4, 2, nat.NMG_F32, None, 8, 4, None, None, 8, 0, 0, None, 0, None) == 1
    # leading dimension too small
    assert L.nmg_spmm(one, one, None, 8, 8, 2, 4, 2, nat.NMG_F32, one, 4, 4, None, one, 8, 0, 0, None, 0, None) == 1
    assert b"ld_act" in L.nmg_last_error()
    assert L.nmg_spmm_t(one, one, None, 8, 8, 2, 4, 2, nat.NMG_F32, one, 8, 4, one, 4, 0, None, 0, None) == 1
    with pytest.raises(nat.NmgError):
        nat.check(1)
    # workspace queries are pure arithmetic
    assert L.nmg_spmm_workspace_bytes(4096, 4096, 4096, 2, 4, 16, nat.NMG_F32, 0, 0, 0) >= 4096 * 4096 * 4
    assert L.nmg_spmm_t_workspace_bytes(64, 64, 8, 2, 4, 2, nat.NMG_F32, 0, 0) > 0
    assert L.nmg_packed_bytes(64, 64, 2, 4, 2, nat.NMG_F16) > 64 * 64 // 4 * 6


def test_cpu_tensors_are_rejected_loudly():
    import torch
    import sten_b200 as sten
    with pytest.raises(RuntimeError, match="CUDA"):
        sten.GroupedNMTensor.from_dense(torch.randn(8, 12), 2, 4, sparse_dim=0, group_size=2, group_dim=1)


def test_kernel_choice_queries_are_pure_host_arithmetic():
    """Which variant a call takes decides what it reads (packed copy or val / idx) and how much workspace it needs."""
    L = nat.lib()
    BF, F32 = nat.NMG_BF16, nat.NMG_F32
    TM, KM = nat.NMG_ACT_TOKEN_MAJOR, nat.NMG_ACT_K_MAJOR
    AUTO, SIMT, TENSOR = nat.NMG_ALGO_AUTO, nat.NMG_ALGO_SIMT, nat.NMG_ALGO_TENSOR
    # fused tensor-core kernel below 1280 tokens reads the packed copy; the two-pass variant above does not
    assert L.nmg_spmm_uses_packed(4096, 4096, 256, 2, 4, 16, BF, TM, AUTO, 0) == 1
    assert L.nmg_spmm_uses_packed(4096, 4096, 2048, 2, 4, 16, BF, TM, AUTO, 0) == 0
    # SIMT forward reads val / idx; SIMT transposed reads the packed copy
    assert L.nmg_spmm_uses_packed(4096, 4096, 256, 2, 4, 16, BF, TM, SIMT, 0) == 0
    # K-major activations (torch.mm) are transposed into the workspace and then take the same tensor-core kernels
    assert L.nmg_spmm_uses_packed(4096, 4096, 256, 2, 4, 16, BF, KM, AUTO, 0) == 1
    assert L.nmg_spmm_uses_packed(4096, 4096, 8, 2, 4, 16, BF, KM, AUTO, 0) == 0   # a handful of columns stays on the SIMT kernel
    assert L.nmg_spmm_workspace_bytes(4096, 4096, 4096, 2, 4, 16, BF, KM, TENSOR, 0) >= 2 * 4096 * 4096 * 2
    assert L.nmg_spmm_uses_packed(4096, 4096, 16, 2, 4, 16, F32, TM, AUTO, 1) == 1
    assert L.nmg_spmm_uses_packed(4096, 4096, 4096, 2, 4, 16, F32, TM, AUTO, 1) == 0
    # 3:6 has no fused kernel: the tensor-core path is always the two-pass variant
    assert L.nmg_spmm_uses_packed(600, 600, 512, 3, 6, 4, BF, TM, TENSOR, 0) == 0
    # the two-pass variant's workspace holds the expanded weight (M * K * 2 bytes; three planes + split activation in fp32)
    ws = L.nmg_spmm_workspace_bytes(4096, 4096, 4096, 2, 4, 16, BF, TM, TENSOR, 0)
    assert 4096 * 4096 * 2 <= ws <= 4096 * 4096 * 2 + 4096
    ws32 = L.nmg_spmm_workspace_bytes(4096, 4096, 4096, 2, 4, 16, F32, TM, TENSOR, 0)
    assert ws32 >= 6 * 4096 * 4096 * 2
    # transposed product, 16-bit, two-pass regime: the workspace holds W^T compressed 2:4 along the reduction (M * K bytes of
    # values + M * K / 8 bytes of metadata), or the dense W^T (2 * M * K bytes) when the dense-rate kernels are forced
    ws_sp = L.nmg_spmm_t_workspace_bytes(4096, 4096, 4096, 2, 4, 16, BF, TENSOR, 0)
    assert ws_sp >= 4096 * 4096 * 2
    assert L.nmg_spmm_t_workspace_bytes(4096, 4096, 4096, 2, 4, 16, BF, nat.NMG_ALGO_TENSOR_DENSE, 0) >= 4096 * 4096 * 2
    # replicated output: argument validation happens before any CUDA call
    one = ctypes.c_void_p(16)
    outs = (ctypes.c_void_p * 1)(16)
    assert L.nmg_spmm_replicated(one, one, 4096, 4096, 2, 4, 16, BF, one, 4096, 2048, None, outs, 0, None, 2048, None, 0, None) == 1
    assert L.nmg_spmm_replicated(one, one, 4096, 4096, 2, 4, 16, BF, one, 4090, 32, None, outs, 1, None, 32, None, 0, None) == 1  # ld_act < K
    assert L.nmg_spmm_replicated_workspace_bytes(4096, 4096, 100, 2, 4, 16, BF) >= 4096 * 4096 * 2
    assert L.nmg_memcpy_2d_async(None, 8, one, 8, 8, 1, None) == 1
