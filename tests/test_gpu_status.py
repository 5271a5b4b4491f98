"""The bounded device-side waits: a wait that runs out is reported as a status, the context stays usable.

Every mbarrier wait of the library's kernels gives up after a time limit, records a code in a device status word and
lets the kernel return.  Here one such wait is made to run out on purpose in the mildest possible way: a one-thread
kernel waits one millisecond on a barrier nothing arrives at.  Nothing faults, nothing hangs."""
import ctypes

import pytest
import torch

from gpu_util import cuda, np_of, rel_fro, seeded_normal

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_and_the_next_call_succeeds():
    from sten_b200 import _native as nat, ops
    L = nat.lib()
    assert ops.read_status() == 0
    st = torch.cuda.current_stream().cuda_stream
    assert L.nmg_selftest_wait(1_000_000, st) == 0  # 1 ms
    code = ctypes.c_int(0)
    rc = L.nmg_read_status(st, ctypes.byref(code))
    assert rc == 5 and code.value == 90, (rc, code.value)      # NMG_ERR_TIMEOUT, code of the self-test wait
    assert b"bounded wait" in L.nmg_last_error()
    assert ops.read_status() == 0                               # reported once, then cleared
    # the context is intact: an ordinary tensor-core call right afterwards gives the right numbers
    M, K, n, m, g, tokens = 256, 512, 2, 4, 16, 256
    w = seeded_normal((M, K), 1).bfloat16().to(cuda())
    x = seeded_normal((tokens, K), 2).bfloat16().to(cuda())
    val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    dense = ops.densify(val, idx, 1, M, K, n, m, g)[0]
    y = ops.spmm(val, idx, M, K, n, m, g, x, algo=nat.NMG_ALGO_TENSOR)
    assert rel_fro(np_of(y), np_of(x).astype("float64") @ np_of(dense).astype("float64").T) <= 1e-2
    assert ops.read_status() == 0


def test_limit_is_validated_on_the_host():
    from sten_b200 import _native as nat
    L = nat.lib()
    assert L.nmg_selftest_wait(0, None) == 1
    assert L.nmg_selftest_wait(5_000_000_000, None) == 1
