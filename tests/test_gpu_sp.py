"""The transposed product on the structured-sparse tensor cores (tcgen05.mma.sp).

dX = dY W reduces over the weight's rows, the axis the n:m blocks run along, so W^T is 2:4-structured along the
reduction whenever n <= 2 and m is a multiple of 4.  From 1280 tokens on, 16-bit weights take that path by default.
Checked here against float64 on the densified weight (tolerance 1e-2, as for every 16-bit product) and against the
dense-rate tensor-core kernels (NMG_ALGO_TENSOR_DENSE), which multiply the same operands including the zeros."""
import numpy as np
import pytest
import torch

from gpu_util import cuda, seeded_normal

pytestmark = pytest.mark.gpu

TOL_HALF = 1e-2


def _rel(got, want):
    got, want = got.double(), want.double()
    return float((got - want).norm() / want.norm())


CASES = [
    # n, m, g, M, K, tokens
    (2, 4, 16, 128, 128, 1280),     # one metadata atom, one tile
    (2, 4, 16, 256, 512, 1536),
    (1, 4, 16, 128, 520, 1537),     # single kept value per group of four: the pair is completed with a zero
    (2, 8, 16, 264, 904, 1700),     # 2:8: both kept values may fall into one group of four, or one into each
    (1, 8, 3, 1000, 304, 2048),     # M = 1000: reduction padded to 1024, last metadata atom partly empty
    (1, 16, 16, 400, 776, 1542),
    (2, 4, 1, 136, 72, 2048),       # K = 72 < one feature tile
    (1, 32, 2, 192, 200, 1300),     # m = 32: eight groups of four per block, seven of them empty
    (2, 4, 16, 2048, 384, 1280),    # long reduction: 16 A-ring slots per tile
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,m,g,M,K,tokens", CASES)
def test_structured_sparse_transposed_product(dtype, n, m, g, M, K, tokens):
    from sten_b200 import _native as nat, ops
    w = seeded_normal((M, K), 400 + n + m + g).to(dtype).to(cuda())
    val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    dense = ops.densify(val, idx, 1, M, K, n, m, g)[0].double()
    dy = seeded_normal((tokens, M), 401).to(dtype).to(cuda())
    want = dy.double() @ dense
    dx = ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_TENSOR)
    assert dx.shape == (tokens, K)
    assert _rel(dx, want) <= TOL_HALF
    dx_dense = ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_TENSOR_DENSE)
    assert _rel(dx_dense, want) <= TOL_HALF
    # both accumulate the same products in fp32; only the order of the additions differs
    assert _rel(dx, dx_dense) <= 2e-3
    assert torch.equal(dx, ops.spmm_t(val, idx, M, K, n, m, g, dy))  # the default takes the same path, deterministically
    assert ops.read_status() == 0


def test_kept_compressed_copy_and_plugin_backward():
    """nmg_pack_sp24 + nmg_spmm_t_sp24 (the copy kept across calls) give the bits of nmg_spmm_t (the copy built per call),
    and the plugin's F.linear backward uses it: dX of a bf16 layer with 1536 tokens against float64."""
    import sten_b200 as sten
    from sten_b200 import _native as nat, ops
    M, K, tokens, n, m, g = 384, 520, 1536, 2, 8, 16
    w = seeded_normal((M, K), 31).bfloat16().to(cuda())
    val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    dy = seeded_normal((tokens, M), 32).bfloat16().to(cuda())
    sp24 = ops.pack_sp24(val, idx, M, K, n, m, g)
    assert sp24.numel() == ops.sp24_bytes(M, K, n, m, g, torch.bfloat16) >= M * K
    a = ops.spmm_t(val, idx, M, K, n, m, g, dy, sp24=sp24)
    assert torch.equal(a, ops.spmm_t(val, idx, M, K, n, m, g, dy))
    assert ops.sp24_bytes(M, K, n, m, g, torch.float32) == 0 and ops.sp24_bytes(60, 336, 3, 6, 4, torch.bfloat16) == 0
    # few tokens: the kept copy is ignored, the fused kernel runs as before
    few = ops.spmm_t(val, idx, M, K, n, m, g, dy[:200].contiguous(), sp24=sp24)
    assert torch.equal(few, ops.spmm_t(val, idx, M, K, n, m, g, dy[:200].contiguous()))
    # through the plugin
    sten.set_dispatch_failure("raise")
    lin = torch.nn.Linear(K, M, device=cuda(), dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    sb = sten.SparsityBuilder()
    sb.set_weight("weight", initial_sparsifier=sten.GroupedNMSparsifier(n, m, g), out_format=sten.GroupedNMTensor)
    sparse = sb.get_sparse_model(lin)
    x = seeded_normal((tokens, K), 33).bfloat16().to(cuda()).requires_grad_(True)
    sparse(x).backward(dy)
    gnm = sparse.weight.wrapped_tensor
    assert gnm.__dict__.get("_sp24_cache") is not None, "the backward pass did not take the structured-sparse path"
    dense = gnm.to_dense().double()
    assert _rel(x.grad, dy.double() @ dense) <= TOL_HALF
    assert torch.equal(x.grad, a)
    assert set(gnm.__getstate__()) == {"val", "idx", "nm_strides"}  # the cache is never pickled
    assert ops.read_status() == 0


def test_zeros_among_the_kept_values_and_exact_small_integers():
    """Weights of small integers: many exact zeros among the kept values (groups with fewer non-zeros than slots), and a
    product that is exact in bf16 x bf16 -> fp32, so the structured-sparse result must equal the float64 one bit for bit
    after rounding to bf16."""
    from sten_b200 import _native as nat, ops
    M, K, tokens, n, m, g = 256, 256, 1280, 2, 4, 4
    gen = torch.Generator().manual_seed(9)
    w = torch.randint(-2, 3, (M, K), generator=gen).to(torch.bfloat16).to(cuda())
    dy = torch.randint(-2, 3, (tokens, M), generator=gen).to(torch.bfloat16).to(cuda())
    val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    dense = ops.densify(val, idx, 1, M, K, n, m, g)[0]
    dx = ops.spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_TENSOR)
    want = (dy.double() @ dense.double()).to(torch.bfloat16)
    assert torch.equal(dx, want)
    assert ops.read_status() == 0


def test_patterns_outside_the_structure_fall_back_to_the_dense_rate_kernels():
    from sten_b200 import _native as nat, ops
    # 3:6 (blocks are not made of groups of four) and fp32 stay on the dense-rate kernels, with the same results as before
    M, K, tokens = 96, 336, 1300
    w = seeded_normal((M, K), 77).bfloat16().to(cuda())
    val, idx = ops.sparsify(w.unsqueeze(0), 3, 6, 4)
    dy = seeded_normal((tokens, M), 78).bfloat16().to(cuda())
    a = ops.spmm_t(val, idx, M, K, 3, 6, 4, dy, algo=nat.NMG_ALGO_TENSOR)
    b = ops.spmm_t(val, idx, M, K, 3, 6, 4, dy, algo=nat.NMG_ALGO_TENSOR_DENSE)
    assert torch.equal(a, b)
