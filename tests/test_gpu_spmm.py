"""Parity of the CUDA matmuls (forward in both activation layouts, transposed backward), through the C ABI.

fp32: relative Frobenius error <= 1e-5 against (a) the CPU oracle, which follows the reference micro-kernel's
accumulation structure, (b) float64 matmul on the densified weight, and (c) stored outputs of the reference's own
AVX micro-kernels.  fp16 / bf16: <= 1e-2 against float64 matmul of the rounded operands."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from gpu_util import cuda, np_of, rel_fro, seeded_normal
from oracle import nmg_oracle as orc

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_HALF = 1e-2


def _problem(M, K, n, m, g, tokens, seed, dtype=torch.float32):
    from sten_b200 import ops
    w = seeded_normal((M, K), seed).to(dtype)
    x = seeded_normal((tokens, K), seed + 1).to(dtype)
    val, idx = ops.sparsify(w.to(cuda()).unsqueeze(0), n, m, g)
    dense = ops.densify(val, idx, 1, M, K, n, m, g)[0]
    return val, idx, x.to(cuda()), dense


CASES = [
    # n, m, g, M, K, tokens   (remainders in M, K and tokens on purpose)
    (2, 4, 4, 1024, 1024, 256),      # the 1024 x 1024 plumbing configuration
    (2, 4, 16, 256, 1000, 200),
    (1, 4, 16, 130, 512, 77),
    (1, 8, 16, 96, 1024, 128),
    (2, 8, 16, 72, 900, 130),
    (1, 16, 16, 100, 777, 64),
    (3, 6, 4, 60, 336, 56),
    (2, 4, 64, 64, 2000, 33),
    (4, 8, 1, 16, 150, 40),          # not specialised: generic kernels
    (5, 12, 2, 24, 1600, 9),         # generic, C = 792 patterns
    (1, 4, 1, 9, 7, 1),
]


@pytest.mark.parametrize("n,m,g,M,K,tokens", CASES)
def test_forward_token_major_fp32(n, m, g, M, K, tokens):
    from sten_b200 import ops
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 10 * n + m + g)
    bias = seeded_normal((M,), 5).to(cuda())
    y = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias)
    ref64 = np_of(x).astype(np.float64) @ np_of(dense).astype(np.float64).T + np_of(bias).astype(np.float64)
    assert rel_fro(np_of(y), ref64) <= TOL_F32
    y_nb = ops.spmm(val, idx, M, K, n, m, g, x)
    want = orc.spmm(np_of(val), np_of(idx), np_of(x), M, K, n, m, g)[:, :M]
    assert rel_fro(np_of(y_nb), want) <= TOL_F32
    assert torch.equal(y_nb, ops.spmm(val, idx, M, K, n, m, g, x))  # deterministic


@pytest.mark.parametrize("n,m,g,M,K,tokens", CASES[:8])
def test_forward_k_major_fp32(n, m, g, M, K, tokens):
    from sten_b200 import _native as nat, ops
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 20 * n + m + g)
    b = x.t().contiguous()  # [K, tokens]
    c = ops.spmm(val, idx, M, K, n, m, g, b, layout=nat.NMG_ACT_K_MAJOR)
    ref64 = np_of(dense).astype(np.float64) @ np_of(b).astype(np.float64)
    assert c.shape == (M, tokens)
    assert rel_fro(np_of(c), ref64) <= TOL_F32


@pytest.mark.parametrize("n,m,g,M,K,tokens", CASES)
def test_transposed_fp32(n, m, g, M, K, tokens):
    from sten_b200 import ops
    val, idx, _, dense = _problem(M, K, n, m, g, tokens, 30 * n + m + g)
    dy = seeded_normal((tokens, M), 99).to(cuda())
    dx = ops.spmm_t(val, idx, M, K, n, m, g, dy)
    ref64 = np_of(dy).astype(np.float64) @ np_of(dense).astype(np.float64)
    assert dx.shape == (tokens, K)
    assert rel_fro(np_of(dx), ref64) <= TOL_F32


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,m,g,M,K,tokens", [(2, 4, 16, 256, 1000, 200), (1, 4, 16, 128, 512, 64), (2, 8, 16, 72, 900, 130)])
def test_half_precision(dtype, n, m, g, M, K, tokens):
    from sten_b200 import ops
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 40 * n + m, dtype)
    y = ops.spmm(val, idx, M, K, n, m, g, x)
    assert y.dtype == dtype
    ref64 = np_of(x).astype(np.float64) @ np_of(dense).astype(np.float64).T
    assert rel_fro(np_of(y), ref64) <= TOL_HALF
    dy = seeded_normal((tokens, M), 98).to(dtype).to(cuda())
    dx = ops.spmm_t(val, idx, M, K, n, m, g, dy)
    assert rel_fro(np_of(dx), np_of(dy).astype(np.float64) @ np_of(dense).astype(np.float64)) <= TOL_HALF


TC_CASES = [
    # n, m, g, M, K, tokens: multiples of the 128 x 256 x 64 tile, and every kind of remainder
    (2, 4, 16, 256, 512, 512),
    (2, 4, 16, 200, 1000, 300),
    (1, 4, 16, 128, 520, 77),
    (1, 8, 16, 96, 1024, 256),
    (2, 8, 16, 264, 904, 130),
    (1, 16, 16, 400, 776, 64),
    (2, 4, 4, 1024, 1024, 256),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,m,g,M,K,tokens", TC_CASES)
def test_tensor_core_forward_and_transposed(dtype, n, m, g, M, K, tokens):
    from sten_b200 import _native as nat, ops
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 50 * n + m + g, dtype)
    bias = seeded_normal((M,), 6).to(dtype).to(cuda())
    y = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR)
    ref64 = np_of(x).astype(np.float64) @ np_of(dense).astype(np.float64).T + np_of(bias).astype(np.float64)
    assert rel_fro(np_of(y), ref64) <= TOL_HALF
    # same numbers whether the column-ordered copy is built per call or once
    packed = ops.pack(val, idx, M, K, n, m, g)
    assert torch.equal(ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR, packed=packed), y)
    # the SIMT kernels agree with the tensor cores to half-precision rounding
    y_simt = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_SIMT)
    assert rel_fro(np_of(y), np_of(y_simt)) <= TOL_HALF
    dy = seeded_normal((tokens, M), 97).to(dtype).to(cuda())
    dx = ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_TENSOR, packed=packed)
    assert rel_fro(np_of(dx), np_of(dy).astype(np.float64) @ np_of(dense).astype(np.float64)) <= TOL_HALF
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_major_input_with_row_major_output(dtype):
    """C = W X^T written as [M, tokens] (what a row shard needs for an in-place gather), into a slab of a larger buffer."""
    from sten_b200 import _native as nat, ops
    M, K, n, m, g, tokens = 256, 520, 2, 8, 16, 200
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 61, dtype)
    full = torch.zeros(3 * M, tokens, dtype=dtype, device=cuda())
    ops.spmm(val, idx, M, K, n, m, g, x, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS, out=full[M:2 * M])
    ref64 = np_of(dense).astype(np.float64) @ np_of(x).astype(np.float64).T
    assert rel_fro(np_of(full[M:2 * M]), ref64) <= (TOL_F32 if dtype == torch.float32 else TOL_HALF)
    assert float(full[:M].abs().max()) == 0 and float(full[2 * M:].abs().max()) == 0
    # aligned case takes the vectorised stores: 256 tokens, ld multiple of 8
    x2 = seeded_normal((256, K), 62).to(dtype).to(cuda())
    c2 = ops.spmm(val, idx, M, K, n, m, g, x2, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS)
    y2 = ops.spmm(val, idx, M, K, n, m, g, x2)
    assert torch.equal(c2, y2.t())


@pytest.mark.parametrize("n,m,g,M,K,tokens", TC_CASES + [(2, 4, 16, 512, 4096, 512)])
def test_fp32_on_tensor_cores_by_exact_bf16_splitting(n, m, g, M, K, tokens):
    """fp32 operands as sums of three bf16 pieces, six partial products in the fp32 accumulator: fp32 tolerance holds."""
    from sten_b200 import _native as nat, ops
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 70 * n + m + g)
    bias = seeded_normal((M,), 8).to(cuda())
    y = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR)
    ref64 = np_of(x).astype(np.float64) @ np_of(dense).astype(np.float64).T + np_of(bias).astype(np.float64)
    err = rel_fro(np_of(y), ref64)
    print(f"split-bf16 forward {n}:{m} K={K}: rel. Frobenius error {err:.2e}")
    assert err <= TOL_F32
    packed = ops.pack(val, idx, M, K, n, m, g)
    assert torch.equal(ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR, packed=packed), y)
    dy = seeded_normal((tokens, M), 96).to(cuda())
    dx = ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_TENSOR, packed=packed)
    assert rel_fro(np_of(dx), np_of(dy).astype(np.float64) @ np_of(dense).astype(np.float64)) <= TOL_F32
    # the SIMT transposed kernel reads the fp32 section of the same packed copy
    dx_simt = ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_SIMT, packed=packed)
    assert rel_fro(np_of(dx_simt), np_of(dx)) <= TOL_F32
    assert ops.read_status() == 0


def test_tensor_core_is_the_default_for_half_precision():
    from sten_b200 import _native as nat, ops
    M, K, n, m, g, tokens = 256, 512, 2, 4, 16, 256
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 3, torch.bfloat16)
    auto = ops.spmm(val, idx, M, K, n, m, g, x)
    assert torch.equal(auto, ops.spmm(val, idx, M, K, n, m, g, x, algo=nat.NMG_ALGO_TENSOR))
    # 3:6 has no fused tensor-core kernel (6 does not divide the 128-row tile): the two-pass variant takes it
    val36, idx36, x36, dense36 = _problem(60, 336, 3, 6, 4, 50, 3, torch.bfloat16)
    y36 = ops.spmm(val36, idx36, 60, 336, 3, 6, 4, x36, algo=nat.NMG_ALGO_TENSOR)
    assert rel_fro(np_of(y36), np_of(x36).astype(np.float64) @ np_of(dense36).astype(np.float64).T) <= TOL_HALF
    # 16-bit activation rows that are not 16-byte aligned cannot be read by TMA: the forced tensor path refuses them
    val_o, idx_o, x_o, _ = _problem(60, 333, 3, 6, 4, 50, 3, torch.bfloat16)
    with pytest.raises(nat.NmgError) as e:
        ops.spmm(val_o, idx_o, 60, 333, 3, 6, 4, x_o, algo=nat.NMG_ALGO_TENSOR)
    assert e.value.status == 2


TWO_PASS_CASES = [
    # n, m, g, M, K, tokens: from 1280 tokens on (256 in fp32, and always for patterns without a fused kernel) the weight is
    # expanded once into a dense 16-bit matrix and multiplied by the persistent TMA-fed kernel
    (2, 4, 16, 256, 512, 1536),
    (2, 8, 16, 264, 904, 1700),
    (1, 16, 16, 400, 776, 1542),
    (1, 4, 16, 128, 520, 1537),
    (2, 4, 1, 136, 72, 2048),
    (3, 6, 8, 304, 704, 1200),
    (3, 6, 4, 64, 336, 56),
    (1, 8, 3, 1000, 304, 2048),
    (2, 8, 16, 203, 333, 1029),   # rows of 16-bit operands would not be 16-byte aligned: fp32 only
    (1, 4, 5, 77, 130, 1500),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,m,g,M,K,tokens", TWO_PASS_CASES)
def test_two_pass_tensor_core_forward_and_transposed(dtype, n, m, g, M, K, tokens):
    from sten_b200 import _native as nat, ops
    tol = TOL_F32 if dtype == torch.float32 else TOL_HALF
    if dtype != torch.float32 and (K % 8 or M % 8):
        pytest.skip("TMA needs 16-byte aligned activation rows")
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 90 * n + m + g, dtype)
    bias = seeded_normal((M,), 16).to(dtype).to(cuda())
    y = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR)
    ref64 = np_of(x).astype(np.float64) @ np_of(dense).astype(np.float64).T + np_of(bias).astype(np.float64)
    assert rel_fro(np_of(y), ref64) <= tol
    c = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS)
    assert torch.equal(c.t(), y)
    dy = seeded_normal((tokens, M), 197).to(dtype).to(cuda())
    dx = ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_TENSOR)
    assert rel_fro(np_of(dx), np_of(dy).astype(np.float64) @ np_of(dense).astype(np.float64)) <= tol
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,K,tokens,tight", [(264, 904, 1100, False), (512, 512, 2048, False), (130, 336, 1027, False), (130, 336, 1027, True)])
def test_replicated_output_matches_the_plain_matmul(dtype, M, K, tokens, tight):
    """The epilogue that writes every destination buffer (peer GPUs in the sharded layer; here three local buffers)."""
    from sten_b200 import _native as nat, ops
    n, m, g = 2, 8, 16
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 123, dtype)
    bias = seeded_normal((M,), 17).to(dtype).to(cuda())
    ld = tokens if tight else tokens + (8 - tokens % 8) % 8 + 16  # tight: rows are not 16-byte aligned, scalar stores
    bufs = [torch.full((M + 2, ld), 7.0, dtype=dtype, device=cuda()) for _ in range(3)]
    ops.spmm_replicated(val, idx, M, K, n, m, g, x, [b[1:].data_ptr() for b in bufs], ld, bias=bias)
    ref = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS, algo=nat.NMG_ALGO_TENSOR)
    ref64 = np_of(dense).astype(np.float64) @ np_of(x).astype(np.float64).T + np_of(bias).astype(np.float64)[:, None]
    assert rel_fro(np_of(ref), ref64) <= (TOL_F32 if dtype == torch.float32 else TOL_HALF)
    for b in bufs:
        # every destination receives the same bits; the plain call may run another variant (fused, split reduction axis),
        # whose fp32 summation order differs
        assert torch.equal(b[1:M + 1, :tokens], bufs[0][1:M + 1, :tokens])
        assert rel_fro(np_of(b[1:M + 1, :tokens]), np_of(ref).astype(np.float64)) <= (1e-6 if dtype == torch.float32 else 2e-3)
        assert rel_fro(np_of(b[1:M + 1, :tokens]), ref64) <= (TOL_F32 if dtype == torch.float32 else TOL_HALF)
        # nothing outside the panel is touched
        assert float((b[0] - 7).abs().max()) == 0 and float((b[M + 1] - 7).abs().max()) == 0
        assert ld == tokens or float((b[1:M + 1, tokens:] - 7).abs().max()) == 0
    assert ops.read_status() == 0
    # few tokens run on the same variant
    ops.spmm_replicated(val, idx, M, K, n, m, g, x[:32], [bufs[0][1:].data_ptr()], ld, bias=bias)
    assert rel_fro(np_of(bufs[0][1:M + 1, :32]), ref64[:, :32]) <= (TOL_F32 if dtype == torch.float32 else TOL_HALF)


def test_against_stored_reference_microkernel_outputs():
    from sten_b200 import ops
    data = np.load(os.path.join(GOLDEN, "spmm_cases.npz"))
    names = sorted({k.split("/")[0] for k in data.files})
    for name in names:
        n, m, g, shape, ntok = name.split("_")
        n, m, g = int(n), int(m), int(g)
        M, K = map(int, shape.split("x"))
        w = torch.from_numpy(data[name + "/w"]).to(cuda())
        x = torch.from_numpy(data[name + "/x"]).to(cuda())
        val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
        y = ops.spmm(val, idx, M, K, n, m, g, x)
        for isa in ("avx2", "avx512"):
            if f"{name}/{isa}" in data.files:
                assert rel_fro(np_of(y), data[f"{name}/{isa}"][:, :M]) <= TOL_F32, (name, isa)


def test_linearity_and_strided_operands():
    from sten_b200 import ops
    M, K, n, m, g, tokens = 128, 600, 2, 4, 16, 96
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 77)
    x2 = seeded_normal((tokens, K), 78).to(cuda())
    a = ops.spmm(val, idx, M, K, n, m, g, x) + 2 * ops.spmm(val, idx, M, K, n, m, g, x2)
    b = ops.spmm(val, idx, M, K, n, m, g, x + 2 * x2)
    assert rel_fro(np_of(a), np_of(b)) <= 1e-5
    wide = torch.zeros(tokens, K + 24, device=cuda())
    wide[:, 8:8 + K] = x
    y = ops.spmm(val, idx, M, K, n, m, g, wide[:, 8:8 + K])  # leading dimension != K, unaligned start
    assert torch.equal(y, ops.spmm(val, idx, M, K, n, m, g, x))


def test_workspace_and_argument_errors():
    from sten_b200 import _native as nat, ops
    M, K, n, m, g, tokens = 64, 96, 2, 4, 4, 32
    val, idx, x, _ = _problem(M, K, n, m, g, tokens, 5)
    L = nat.lib()
    out = torch.empty(tokens, M, device=cuda())
    st = torch.cuda.current_stream().cuda_stream
    rc = L.nmg_spmm(val.data_ptr(), idx.data_ptr(), None, M, K, n, m, g, nat.NMG_F32, x.data_ptr(), K, tokens, None,
                    out.data_ptr(), M, 0, 0, None, 0, st)
    assert rc == 4 and b"workspace" in L.nmg_last_error()
    with pytest.raises(ValueError):
        ops.spmm(val, idx, M, K, n, m, g, x[:, :-1])
    with pytest.raises(TypeError):
        ops.spmm(val, idx, M, K, n, m, g, x.half())
    # a caller-supplied `out` the kernel could not write safely is refused before any launch
    for bad in (torch.empty(tokens, M, device=cuda(), dtype=torch.float16),      # wrong dtype
                torch.empty(tokens, M - 1, device=cuda()),                        # wrong shape
                torch.empty(M, tokens, device=cuda()).t(),                        # transposed view: rows not contiguous
                torch.empty(tokens, 1, device=cuda()).expand(tokens, M)):         # overlapping rows
        with pytest.raises(ValueError):
            ops.spmm(val, idx, M, K, n, m, g, x, out=bad)
    wide = torch.zeros(tokens, M + 8, device=cuda())
    ops.spmm(val, idx, M, K, n, m, g, x, out=wide[:, :M])                         # a column slice is fine: ld_out = stride(0)
    assert torch.equal(wide[:, :M], ops.spmm(val, idx, M, K, n, m, g, x)) and float(wide[:, M:].abs().max()) == 0
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tokens,algo", [(1536, "tensor"), (200, "tensor"), (200, "simt")])
def test_fused_activation_and_residual(dtype, tokens, algo):
    """out = gelu(x W^T + b) + residual in one call, on the two-pass tensor-core path (fused into the epilogue; CTA pairs
    for 16-bit), the fused-expansion kernel and the SIMT kernel (each followed by one elementwise pass)."""
    from sten_b200 import _native as nat, ops
    M, K, n, m, g = 392, 520, 2, 4, 16
    tol = TOL_F32 if dtype == torch.float32 else TOL_HALF
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 123, dtype)
    bias = seeded_normal((M,), 7).to(dtype).to(cuda())
    res = seeded_normal((tokens, M), 8).to(dtype).to(cuda())
    a = nat.NMG_ALGO_TENSOR if algo == "tensor" else nat.NMG_ALGO_SIMT
    pre = np_of(x).astype(np.float64) @ np_of(dense).astype(np.float64).T + np_of(bias).astype(np.float64)
    gelu = torch.nn.functional.gelu(torch.from_numpy(pre)).numpy()
    y = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=a, activation="gelu", residual=res)
    assert rel_fro(np_of(y), gelu + np_of(res).astype(np.float64)) <= tol
    y2 = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=a, activation="gelu")
    assert rel_fro(np_of(y2), gelu) <= tol
    y3 = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=a, residual=res)
    assert rel_fro(np_of(y3), pre + np_of(res).astype(np.float64)) <= tol
    # feature-major output with a feature-major residual (the staged epilogue)
    c = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=a, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS, activation="gelu",
                 residual=res.t().contiguous())
    assert rel_fro(np_of(c), (gelu + np_of(res).astype(np.float64)).T) <= tol
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,tokens", [(1000, 1390), (264, 1281), (1032, 4100)])
def test_fused_epilogue_ragged_edges_of_the_bulk_store_path(dtype, M, tokens):
    """Token-major result of the CTA-pair kernel (operands exchanged, bias along the accumulator's columns, residual rows
    fetched in 16-byte pieces, tiled bulk stores) when neither the token count nor the feature count fills the last tile:
    the copy engine clips the stores, the residual's ragged slices take the element-wise path."""
    from sten_b200 import _native as nat, ops
    K, n, m, g = 520, 2, 4, 16
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 321, dtype)
    bias = seeded_normal((M,), 17).to(dtype).to(cuda())
    res = seeded_normal((tokens, M), 18).to(dtype).to(cuda())
    pre = np_of(x).astype(np.float64) @ np_of(dense).astype(np.float64).T + np_of(bias).astype(np.float64)
    gelu = torch.nn.functional.gelu(torch.from_numpy(pre)).numpy()
    # guard rows behind the result: nothing may be written past the last token
    buf = torch.full((tokens + 8, M), 7.0, dtype=dtype, device=cuda())
    y = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR, activation="gelu", residual=res, out=buf[:tokens])
    assert rel_fro(np_of(y), gelu + np_of(res).astype(np.float64)) <= TOL_HALF
    assert bool((buf[tokens:] == 7.0).all())
    y2 = ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR)
    assert rel_fro(np_of(y2), pre) <= TOL_HALF
    # a result that is a column block of a wider matrix (row pitch larger than M): the neighbouring columns stay untouched
    wide = torch.full((tokens, M + 16), 3.0, dtype=dtype, device=cuda())
    ops.spmm(val, idx, M, K, n, m, g, x, bias=bias, algo=nat.NMG_ALGO_TENSOR, residual=res, out=wide[:, :M])
    assert rel_fro(np_of(wide[:, :M]), pre + np_of(res).astype(np.float64)) <= TOL_HALF
    assert bool((wide[:, M:] == 3.0).all())
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,m,g,M,K,tokens", [TC_CASES[1], TC_CASES[4], TWO_PASS_CASES[1], TWO_PASS_CASES[7], (2, 4, 16, 2176, 512, 1536)])
def test_k_major_activations_on_tensor_cores(dtype, n, m, g, M, K, tokens):
    """C = W B with B[K][tokens] (the torch.mm orientation): one transpose pre-pass, then the token-major tensor-core kernels
    with row-major output.  Against float64, and the default (AUTO) takes this path."""
    from sten_b200 import _native as nat, ops
    tol = TOL_F32 if dtype == torch.float32 else TOL_HALF
    val, idx, x, dense = _problem(M, K, n, m, g, tokens, 222 + n + m, dtype)
    b = x.t().contiguous()  # [K, tokens]
    bias = seeded_normal((M,), 9).to(dtype).to(cuda())
    c = ops.spmm(val, idx, M, K, n, m, g, b, bias=bias, layout=nat.NMG_ACT_K_MAJOR, algo=nat.NMG_ALGO_TENSOR)
    ref64 = np_of(dense).astype(np.float64) @ np_of(b).astype(np.float64) + np_of(bias).astype(np.float64)[:, None]
    assert c.shape == (M, tokens) and rel_fro(np_of(c), ref64) <= tol
    assert torch.equal(c, ops.spmm(val, idx, M, K, n, m, g, b, bias=bias, layout=nat.NMG_ACT_K_MAJOR))
    # a strided B (column slice of a wider matrix) and the SIMT kernel agree
    wide = torch.zeros(K, tokens + 24, dtype=dtype, device=cuda())
    wide[:, 8:8 + tokens] = b
    c2 = ops.spmm(val, idx, M, K, n, m, g, wide[:, 8:8 + tokens], bias=bias, layout=nat.NMG_ACT_K_MAJOR)
    assert torch.equal(c2, c)
    c_simt = ops.spmm(val, idx, M, K, n, m, g, b, bias=bias, layout=nat.NMG_ACT_K_MAJOR, algo=nat.NMG_ALGO_SIMT)
    assert rel_fro(np_of(c_simt), ref64) <= tol
    assert ops.read_status() == 0
