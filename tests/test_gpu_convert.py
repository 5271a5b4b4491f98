"""Parity of the CUDA sparsifier / densifier (called through the C ABI) with the reference.

Bit-exact (val and idx) against fixtures produced by the reference's own CPU sparsifier, against the CPU oracle on
fresh seeded inputs, and -- at the benchmark sizes -- against sha256 digests of the reference's output."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from gpu_util import cuda, np_of, seeded_normal, sha
from oracle import nmg_oracle as orc

pytestmark = pytest.mark.gpu


def _small():
    with open(os.path.join(GOLDEN, "small_cases.json")) as f:
        meta = json.load(f)
    return meta, np.load(os.path.join(GOLDEN, "small_cases.npz"))


def test_sparsify_and_densify_match_reference_fixtures():
    import sten_b200 as sten
    meta, data = _small()
    for c in meta:
        name = c["name"]
        dense = torch.from_numpy(data[name + "/dense"]).to(cuda())
        t = sten.GroupedNMTensor.from_dense(dense, c["n"], c["m"], sparse_dim=c["sparse_dim"], group_size=c["g"],
                                            group_dim=c["group_dim"])
        assert t.val.shape == data[name + "/val"].shape and t.idx.shape == data[name + "/idx"].shape, name
        assert np.array_equal(np_of(t.idx), data[name + "/idx"]), name
        assert np.array_equal(np_of(t.val).view(np.uint32), data[name + "/val"].view(np.uint32)), name
        back = t.to_dense()
        assert tuple(back.shape) == tuple(dense.shape)
        assert np.array_equal(np_of(back).view(np.uint32), data[name + "/to_dense"].view(np.uint32)), name
        assert t.nm_strides["kernel"] == "sm100" and set(t.__getstate__()) == {"val", "idx", "nm_strides"}


@pytest.mark.parametrize("n,m,g,M,K", [
    (2, 4, 16, 256, 1000), (1, 4, 16, 130, 512), (1, 8, 16, 96, 1024), (2, 8, 16, 72, 900), (1, 16, 16, 100, 777),
    (3, 6, 4, 60, 333), (2, 4, 64, 64, 2000), (2, 8, 4, 40, 500), (1, 4, 1, 9, 7), (4, 8, 1, 16, 150),
])
def test_sparsify_matches_oracle_on_seeded_inputs(n, m, g, M, K):
    from sten_b200 import ops
    w = seeded_normal((M, K), 1000 + n * 100 + m + g)
    val_o, idx_o = orc.sparsify(w.numpy(), n, m, g)
    val, idx = ops.sparsify(w.to(cuda()).unsqueeze(0), n, m, g)
    assert np.array_equal(np_of(idx), idx_o)
    assert np.array_equal(np_of(val).view(np.uint32), val_o.view(np.uint32))
    # idempotence: sparsifying the densified result selects the same entries
    d = ops.densify(val, idx, 1, M, K, n, m, g)
    val2, idx2 = ops.sparsify(d, n, m, g)
    assert torch.equal(ops.densify(val2, idx2, 1, M, K, n, m, g), d)
    # determinism
    val3, idx3 = ops.sparsify(w.to(cuda()).unsqueeze(0), n, m, g)
    assert torch.equal(idx3, idx) and torch.equal(val3, val)


def test_ties_zeros_and_strided_input():
    from sten_b200 import ops
    g_ = torch.Generator().manual_seed(7)
    w = torch.randint(-1, 2, (40, 200), generator=g_).float()
    for (n, m, g) in [(2, 4, 4), (1, 8, 2), (2, 8, 1)]:
        val_o, idx_o = orc.sparsify(w.numpy(), n, m, g)
        val, idx = ops.sparsify(w.to(cuda()).unsqueeze(0), n, m, g)
        assert np.array_equal(np_of(idx), idx_o) and np.array_equal(np_of(val), val_o)
    # a column slice of a wider matrix: leading dimension larger than K
    wide = seeded_normal((32, 300), 3).to(cuda())
    view = wide[:, 17:217]
    val_o, idx_o = orc.sparsify(view.cpu().numpy(), 2, 4, 4)
    val, idx = ops.sparsify(view.unsqueeze(0), 2, 4, 4)
    assert np.array_equal(np_of(idx), idx_o) and np.array_equal(np_of(val), val_o)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_precision_selection_is_done_on_fp32_magnitudes(dtype):
    from sten_b200 import ops
    w = seeded_normal((64, 300), 11).to(dtype)
    val_o, idx_o = orc.sparsify(w.float().numpy(), 2, 8, 4)
    val, idx = ops.sparsify(w.to(cuda()).unsqueeze(0), 2, 8, 4)
    assert val.dtype == dtype
    assert np.array_equal(np_of(idx), idx_o)
    assert np.array_equal(np_of(val), val_o)
    d = ops.densify(val, idx, 1, 64, 300, 2, 8, 4)
    assert np.array_equal(np_of(d)[0], orc.densify(val_o, idx_o, (64, 300), 2, 8, 4))


def test_benchmark_size_weights_match_reference_digests():
    """Every listed case must be checked: the 1024^2 and 4096^2 fp32 weights of the plumbing case and the density sweep,
    and the 16384^2 bf16 2:8 weight of the sharded benchmark (75 776 tiles of 448 columns, a 256-column remainder chunk)."""
    from sten_b200 import ops
    with open(os.path.join(GOLDEN, "big_hashes.json")) as f:
        cases = json.load(f)
    assert len(cases) >= 8 and any(c["M"] == 16384 for c in cases)
    for c in cases:
        w = seeded_normal((c["M"], c["K"]), c["seed"], c.get("scale", 1.0))
        half = c.get("dtype") == "bf16"
        if half:
            w = w.bfloat16()
        bits = (lambda t: t.view(torch.int16).cpu().numpy()) if half else (lambda t: t.cpu().numpy())
        # the fixtures record the digest of their input: torch's CPU generator must reproduce it, else nothing below means anything
        assert sha(bits(w)) == c["dense_sha256"], f"seeded input of {c['M']}x{c['K']} differs from the one the digests were made from"
        wd = w.to(cuda())
        val, idx = ops.sparsify(wd.unsqueeze(0), c["n"], c["m"], c["g"])
        assert list(val.shape) == c["val_shape"] and list(idx.shape) == c["idx_shape"]
        assert sha(np_of(idx)) == c["idx_sha256"], c
        assert sha(bits(val)) == c["val_sha256"], c
        # round trip at full size: densify keeps exactly the selected entries
        d = ops.densify(val, idx, 1, c["M"], c["K"], c["n"], c["m"], c["g"])[0]
        assert bool(((d == wd) | (d == 0)).all())
        assert int((d != 0).sum()) <= c["M"] * c["K"] * c["n"] // c["m"]
        del w, wd, val, idx, d


def test_reference_conversion_properties_all_permutations():
    """The reference's own conversion test (tests/test_nmg.py:33-86), same shapes, n=5 m=12 g=2, every layout."""
    import itertools
    import sten_b200 as sten
    from sten_b200.grouped_nm_tensor import is_correct_nm
    torch.manual_seed(123)
    dims = [17, 5, 1]
    n, m, g = 5, 12, 2
    for shape in itertools.product(dims, dims):
        shape = (3, *shape)
        for perm in itertools.permutations("abc"):
            layout = "".join(perm)
            dense = torch.einsum(f"abc->{layout}", torch.rand(shape, device=cuda()))
            sd, gd = layout.index("c"), layout.index("b")
            t = sten.GroupedNMTensor.from_dense(dense, n=n, m=m, sparse_dim=sd, group_size=g, group_dim=gd)
            sp = t.to_dense()
            assert is_correct_nm(dense, sp, sparse_dim=sd, n=n, m=m)
            kept = sp.abs().sum() / dense.abs().sum()
            assert kept > n / m
            perfect = sten.PerfectNMTensor.from_dense(dense, n=n, m=m, sparse_dim=sd).to_dense()
            assert is_correct_nm(dense, perfect, sparse_dim=sd, n=n, m=m)
            assert perfect.abs().sum() / dense.abs().sum() >= kept - 1e-5


def test_errors_are_status_codes():
    from sten_b200 import _native as nat, ops
    w = torch.randn(8, 8, device=cuda())
    with pytest.raises(nat.NmgError) as e:
        ops.sparsify(w.unsqueeze(0), 2, 8, 2000)
    assert e.value.status == 1
    with pytest.raises(TypeError):
        ops.sparsify(w.double().unsqueeze(0), 2, 4, 2)
    assert ops.read_status() == 0


def test_perfect_nm_matches_reference_fixtures():
    """PerfectNMTensor (per-block top-n, no group constraint) on CUDA against what the reference computed with
    pad / reshape / argsort / gather: val, idx (int64, descending magnitude) and to_dense(), bit for bit."""
    import sten_b200 as sten
    with open(os.path.join(GOLDEN, "perfect_cases.json")) as f:
        meta = json.load(f)
    data = np.load(os.path.join(GOLDEN, "perfect_cases.npz"))
    for c in meta:
        name = c["name"]
        dense = torch.from_numpy(data[name + "/dense"]).to(cuda())
        t = sten.PerfectNMTensor.from_dense(dense, c["n"], c["m"], c["sparse_dim"])
        assert t.idx.dtype == torch.int64 and tuple(t.val.shape) == data[name + "/val"].shape, name
        assert np.array_equal(t.idx.cpu().numpy(), data[name + "/idx"]), name
        assert np.array_equal(t.val.cpu().numpy().view(np.uint32), data[name + "/val"].view(np.uint32)), name
        assert np.array_equal(t.to_dense().cpu().numpy().view(np.uint32), data[name + "/to_dense"].view(np.uint32)), name
    # half precision, the contiguous-block (16-byte load) path, and a negative sparse_dim
    w = seeded_normal((128, 256), 77).bfloat16().to(cuda())
    t = sten.PerfectNMTensor.from_dense(w, 2, 8, -1)
    blocks = w.reshape(128, 32, 8)
    order = blocks.float().abs().argsort(dim=2, descending=True, stable=True)[:, :, :2]
    assert torch.equal(t.idx, order) and torch.equal(t.val, blocks.gather(2, order))
    back = t.to_dense()
    assert torch.equal(back != 0, torch.zeros_like(blocks, dtype=torch.bool).scatter_(2, order, True).reshape(128, 256) & (w != 0))
