"""Parity at the sizes the benchmark times, and on tile counts that exercise the persistent kernels' tile order.

The persistent tensor-core matmul walks output tiles in bands of 16 feature tiles; everything up to 2048 output
features is a single band.  The cases here have 17 and 33 feature tiles (a ragged last band of one tile), several token
tiles per CTA, both accumulator modes (16-bit: double-buffered; fp32: promoted chunks), every output orientation, the
transposed product and the replicated epilogue -- each against a float64 product on the densified weight.

The full-size configurations (4096 x 4096 x 4096 tokens, five patterns; 16384 x 16384 x 16384 tokens, 2:8, bf16) are
checked on 256 sampled output features x all tokens: float64 dot products of the densified rows, which costs a
fraction of the full float64 product and still touches every band, every token tile and both ends of the output."""
import numpy as np
import pytest
import torch

from gpu_util import cuda, seeded_normal

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_HALF = 1e-2
G = 16


def _rel(got, want):
    got, want = got.double(), want.double()
    return float((got - want).norm() / want.norm())


def _weight(M, K, n, m, g, seed, dtype, scale=1.0):
    from sten_b200 import ops
    w = (seeded_normal((M, K), seed) * scale).to(dtype).to(cuda())
    val, idx = ops.sparsify(w.unsqueeze(0), n, m, g)
    del w
    return val, idx


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("n,m,M,K,tokens", [
    (2, 4, 2176, 512, 1536),    # 17 feature tiles: one full band + a band of a single tile
    (2, 8, 4200, 520, 1536),    # 33 feature tiles (two bands + one), ragged last tile (4200 = 32 * 128 + 104)
    (1, 4, 2304, 512, 3000),    # 18 feature tiles x 12 token tiles = 216 tiles > 148 CTAs: several tiles per CTA, ragged tokens
])
def test_multi_band_tile_order_forward(dtype, n, m, M, K, tokens):
    from sten_b200 import _native as nat, ops
    tol = TOL_F32 if dtype == torch.float32 else TOL_HALF
    val, idx = _weight(M, K, n, m, G, 300 + n + m, dtype)
    dense = ops.densify(val, idx, 1, M, K, n, m, G)[0].double()
    x = seeded_normal((tokens, K), 301).to(dtype).to(cuda())
    bias = seeded_normal((M,), 302).to(dtype).to(cuda())
    want = x.double() @ dense.t() + bias.double()
    y = ops.spmm(val, idx, M, K, n, m, G, x, bias=bias, algo=nat.NMG_ALGO_TENSOR)
    assert _rel(y, want) <= tol
    c = ops.spmm(val, idx, M, K, n, m, G, x, bias=bias, algo=nat.NMG_ALGO_TENSOR, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS)
    assert torch.equal(c.t(), y)
    # the replicated epilogue (what a row shard runs): two destination buffers, identical bits, same numbers
    bufs = [torch.zeros(M, tokens, dtype=dtype, device=cuda()) for _ in range(2)]
    ops.spmm_replicated(val, idx, M, K, n, m, G, x, [b.data_ptr() for b in bufs], tokens, bias=bias)
    assert torch.equal(bufs[0], bufs[1]) and torch.equal(bufs[0], c)
    assert ops.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,m,M,K,tokens", [
    (2, 4, 512, 2176, 1536),    # transposed product: the output features are the weight's COLUMNS: 17 feature tiles
    (2, 8, 520, 4200, 1536),    # 33 feature tiles, ragged
])
def test_multi_band_tile_order_transposed(dtype, n, m, M, K, tokens):
    from sten_b200 import _native as nat, ops
    tol = TOL_F32 if dtype == torch.float32 else TOL_HALF
    val, idx = _weight(M, K, n, m, G, 310 + n + m, dtype)
    dense = ops.densify(val, idx, 1, M, K, n, m, G)[0].double()
    dy = seeded_normal((tokens, M), 311).to(dtype).to(cuda())
    dx = ops.spmm_t(val, idx, M, K, n, m, G, dy, algo=nat.NMG_ALGO_TENSOR)
    assert _rel(dx, dy.double() @ dense) <= tol
    assert ops.read_status() == 0


def _sampled_rows(M, count, seed):
    g = torch.Generator().manual_seed(seed)
    rows = torch.randperm(M, generator=g)[:count - 2]
    return torch.cat([rows, torch.tensor([0, M - 1])]).sort().values.to(cuda())


SWEEP = [(1, 4), (2, 4), (1, 8), (2, 8), (1, 16)]


@pytest.mark.parametrize("variant", ["f32-simt", "f32-tensor", "bf16-tensor"])
@pytest.mark.parametrize("n,m", SWEEP)
def test_density_sweep_at_full_size(n, m, variant):
    """4096 x 4096 weight N(0,1) seed 0, 4096 tokens seed 1, g = 16: the configuration of the per-pattern table."""
    from sten_b200 import _native as nat, ops
    M = K = tokens = 4096
    dtype = torch.bfloat16 if variant.startswith("bf16") else torch.float32
    algo = nat.NMG_ALGO_SIMT if variant.endswith("simt") else nat.NMG_ALGO_TENSOR
    tol = TOL_F32 if dtype == torch.float32 else TOL_HALF
    val, idx = _weight(M, K, n, m, G, 0, dtype)
    x = seeded_normal((tokens, K), 1).to(dtype).to(cuda())
    y = ops.spmm(val, idx, M, K, n, m, G, x, algo=algo)
    rows = _sampled_rows(M, 256, 5)
    dense_rows = ops.densify(val, idx, 1, M, K, n, m, G)[0][rows].double()
    assert _rel(y[:, rows], x.double() @ dense_rows.t()) <= tol
    # transposed product on sampled output columns (features of dX are weight columns)
    dy = seeded_normal((tokens, M), 2).to(dtype).to(cuda())
    dx = ops.spmm_t(val, idx, M, K, n, m, G, dy, algo=algo)
    cols = _sampled_rows(K, 256, 6)
    dense_cols = ops.densify(val, idx, 1, M, K, n, m, G)[0][:, cols].double()
    assert _rel(dx[:, cols], dy.double() @ dense_cols) <= tol
    assert ops.read_status() == 0


def test_sharded_benchmark_configuration_at_full_size():
    """16384 x 16384 bf16 weight N(0, 0.02) seed 0 at 2:8 g = 16, 16384 tokens N(0,1) seed 1: C = W X^T as the benchmark
    computes it (one call, output rows follow weight rows), and the transposed product, on sampled rows / columns."""
    from sten_b200 import _native as nat, ops
    M = K = tokens = 16384
    n, m = 2, 8
    val, idx = _weight(M, K, n, m, G, 0, torch.bfloat16, scale=0.02)
    x = seeded_normal((tokens, K), 1).bfloat16().to(cuda())
    c = ops.spmm(val, idx, M, K, n, m, G, x, layout=nat.NMG_ACT_TOKEN_MAJOR_OUT_ROWS)
    dense = ops.densify(val, idx, 1, M, K, n, m, G)[0]
    rows = _sampled_rows(M, 256, 7)
    assert _rel(c[rows], dense[rows].double() @ x.double().t()) <= TOL_HALF
    del c
    dx = ops.spmm_t(val, idx, M, K, n, m, G, x)  # any [tokens, M] bf16 matrix serves as dY; M == K here
    cols = _sampled_rows(K, 256, 8)
    assert _rel(dx[:, cols], x.double() @ dense[:, cols].double()) <= TOL_HALF
    assert ops.read_status() == 0
