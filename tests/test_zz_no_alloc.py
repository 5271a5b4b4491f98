"""nmg_spmm_noalloc: the matmul entry point for callers that cannot allocate device memory (graph capture,
pre-partitioned memory pools, allocator-free callbacks).  Its scratch is a fixed array inside the library, shared by
every call, so the test makes two different calls in a row and checks each against the ordinary entry point
(nmg_spmm with a caller-provided workspace), which runs the same kernels, and against a float64 product on the
densified weight, which does not; the device status must read 0 afterwards.  Then it checks the size limit.

Collected last on purpose: a failure here must not hide the result of any other test."""
import numpy as np
import pytest
import torch

from gpu_util import cuda, np_of, rel_fro, seeded_normal

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5


def _noalloc(val, idx, M, K, n, m, g, act, bias, layout):
    from sten_b200 import _native as nat
    token_major = layout == nat.NMG_ACT_TOKEN_MAJOR
    tokens = act.shape[0] if token_major else act.shape[1]
    out = torch.full((tokens, M) if token_major else (M, tokens), float("nan"), dtype=val.dtype, device=val.device)
    code = {torch.float32: nat.NMG_F32, torch.float16: nat.NMG_F16, torch.bfloat16: nat.NMG_BF16}[val.dtype]
    rc = nat.lib().nmg_spmm_noalloc(val.data_ptr(), idx.data_ptr(), M, K, n, m, g, code, act.data_ptr(), act.shape[1],
                                    tokens, bias.data_ptr() if bias is not None else None, out.data_ptr(), out.shape[1],
                                    layout, torch.cuda.current_stream().cuda_stream)
    return rc, out


def _case(M, K, n, m, g, tokens, seed, dtype=torch.float32):
    from sten_b200 import ops
    w = seeded_normal((M, K), seed).to(dtype).to(cuda())
    val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    x = seeded_normal((tokens, K), seed + 1).to(dtype).to(cuda())
    bias = seeded_normal((M,), seed + 2).to(dtype).to(cuda())
    return val, idx, x, bias


def _ref64(val, idx, M, K, n, m, g, x2d, bias):
    """float64 x W^T (+ bias) on the densified weight: independent of every kernel of the matmul."""
    from sten_b200 import ops
    dense = np_of(ops.densify(val, idx, 1, M, K, n, m, g)[0]).astype(np.float64)
    y = np_of(x2d).astype(np.float64) @ dense.T
    return y + np_of(bias).astype(np.float64) if bias is not None else y


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    from sten_b200 import _native as nat, ops
    # call 1: large-ish problem, token-major, with bias
    M, K, n, m, g, tokens = 256, 1000, 2, 4, 16, 200
    val, idx, x, bias = _case(M, K, n, m, g, tokens, 11)
    rc, got = _noalloc(val, idx, M, K, n, m, g, x, bias, nat.NMG_ACT_TOKEN_MAJOR)
    assert rc == 0, nat.lib().nmg_last_error()
    want = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_SIMT)
    assert rel_fro(np_of(got), np_of(want)) <= TOL_F32
    assert rel_fro(np_of(got), _ref64(val, idx, M, K, n, m, g, x, bias)) <= TOL_F32
    # call 2: smaller problem of another pattern and layout, so stale scratch of call 1 lies right behind its data
    M2, K2, n2, m2, g2, tokens2 = 96, 300, 1, 8, 4, 40
    val2, idx2, x2, _ = _case(M2, K2, n2, m2, g2, tokens2, 23)
    b2 = x2.t().contiguous()
    rc, got2 = _noalloc(val2, idx2, M2, K2, n2, m2, g2, b2, None, nat.NMG_ACT_K_MAJOR)
    assert rc == 0, nat.lib().nmg_last_error()
    want2 = ops.spmm(val2, idx2, M2, K2, n2, m2, g2, b2, layout=nat.NMG_ACT_K_MAJOR, algo=nat.NMG_ALGO_SIMT)
    assert rel_fro(np_of(got2), np_of(want2)) <= TOL_F32
    assert rel_fro(np_of(got2), _ref64(val2, idx2, M2, K2, n2, m2, g2, x2, None).T) <= TOL_F32
    # and the first problem again: same answer as before
    rc, again = _noalloc(val, idx, M, K, n, m, g, x, bias, nat.NMG_ACT_TOKEN_MAJOR)
    assert rc == 0 and torch.equal(again, got)
    # half precision goes through the same scratch
    valh, idxh, xh, biash = _case(128, 512, 2, 8, 16, 64, 31, torch.bfloat16)
    rc, goth = _noalloc(valh, idxh, 128, 512, 2, 8, 16, xh, biash, nat.NMG_ACT_TOKEN_MAJOR)
    assert rc == 0
    wanth = ops.spmm(valh, idxh, 128, 512, 2, 8, 16, xh, bias=biash, algo=nat.NMG_ALGO_SIMT)
    assert rel_fro(np_of(goth), np_of(wanth)) <= 1e-2
    assert rel_fro(np_of(goth), _ref64(valh, idxh, 128, 512, 2, 8, 16, xh, biash)) <= 1e-2
    # the kernels of this entry point report a timed-out wait in the first word of the built-in array: it must read 0
    assert ops.read_status() == 0
    torch.cuda.synchronize()


def test_oversized_and_unspecialised_problems_are_rejected_with_a_message():
    from sten_b200 import _native as nat
    L = nat.lib()
    M, K, n, m, g = 64, 4096, 2, 4, 16
    tokens = nat.NMG_NOALLOC_SCRATCH_BYTES // (K * 4) + 128  # one token tile too many
    val, idx, _, _ = _case(M, K, n, m, g, 8, 5)
    x = torch.zeros(tokens, K, device=cuda())
    rc, _ = _noalloc(val, idx, M, K, n, m, g, x, None, nat.NMG_ACT_TOKEN_MAJOR)
    assert rc == 2 and b"NMG_NOALLOC_SCRATCH_BYTES" in L.nmg_last_error()
    val3, idx3, x3, _ = _case(16, 150, 4, 8, 1, 8, 6)
    rc, _ = _noalloc(val3, idx3, 16, 150, 4, 8, 1, x3, None, nat.NMG_ACT_TOKEN_MAJOR)
    assert rc == 2 and b"table" in L.nmg_last_error()
