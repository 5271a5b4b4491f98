"""The CPU oracle against fixtures produced by the reference itself (tests/golden/gen_golden.py)."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import nmg_oracle as orc


def _small():
    with open(os.path.join(GOLDEN, "small_cases.json")) as f:
        meta = json.load(f)
    data = np.load(os.path.join(GOLDEN, "small_cases.npz"))
    return meta, data


def _to_kernel_view(dense, sparse_dim, group_dim):
    """[..., rows(n:m axis), cols(group axis)] contiguous, other dims kept in their original order."""
    nd = dense.ndim
    others = [d for d in range(nd) if d not in (sparse_dim, group_dim)]
    return np.ascontiguousarray(np.transpose(dense, others + [sparse_dim, group_dim]))


def test_sparsify_bit_exact_on_reference_fixtures():
    meta, data = _small()
    assert len(meta) >= 20
    for c in meta:
        name = c["name"]
        view = _to_kernel_view(data[name + "/dense"], c["sparse_dim"], c["group_dim"])
        val, idx = orc.sparsify(view, c["n"], c["m"], c["g"])
        assert np.array_equal(idx, data[name + "/idx"]), name
        assert np.array_equal(val.view(np.uint32), data[name + "/val"].view(np.uint32)), name


def test_densify_bit_exact_on_reference_fixtures():
    meta, data = _small()
    for c in meta:
        name = c["name"]
        dense = data[name + "/dense"]
        view_shape = _to_kernel_view(dense, c["sparse_dim"], c["group_dim"]).shape
        out = orc.densify(data[name + "/val"], data[name + "/idx"], view_shape, c["n"], c["m"], c["g"])
        nd = dense.ndim
        others = [d for d in range(nd) if d not in (c["sparse_dim"], c["group_dim"])]
        back = np.transpose(out, np.argsort(others + [c["sparse_dim"], c["group_dim"]]))
        assert np.array_equal(back.view(np.uint32), data[name + "/to_dense"].view(np.uint32)), name


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("limit", [4096])
def test_sparsify_bit_exact_on_benchmark_weights(limit):
    with open(os.path.join(GOLDEN, "big_hashes.json")) as f:
        cases = json.load(f)
    for c in cases:
        if c["M"] > limit:
            continue
        g = torch.Generator().manual_seed(c["seed"])
        w = torch.randn(c["M"], c["K"], generator=g, dtype=torch.float32).numpy()
        if _sha(w) != c["dense_sha256"]:
            pytest.skip("torch.randn stream differs from the one the fixtures were made with")
        val, idx = orc.sparsify(w, c["n"], c["m"], c["g"])
        assert list(val.shape) == c["val_shape"] and list(idx.shape) == c["idx_shape"]
        assert _sha(idx) == c["idx_sha256"], c
        assert _sha(val) == c["val_sha256"], c


def test_spmm_against_reference_microkernels_and_float64():
    data = np.load(os.path.join(GOLDEN, "spmm_cases.npz"))
    names = sorted({k.split("/")[0] for k in data.files})
    assert names
    for name in names:
        n, m, g, shape, ntok = name.split("_")
        n, m, g, ntok = int(n), int(m), int(g), int(ntok)
        M, K = map(int, shape.split("x"))
        w, x = data[name + "/w"], data[name + "/x"]
        val, idx = orc.sparsify(w, n, m, g)
        y = orc.spmm(val, idx, x, M, K, n, m, g)
        dense = orc.densify(val, idx, (M, K), n, m, g)
        ref64 = x.astype(np.float64) @ dense.astype(np.float64).T
        err = np.linalg.norm(y[:, :M] - ref64) / np.linalg.norm(ref64)
        assert err < 1e-6, (name, err)
        assert np.all(y[:, M:] == 0)
        for isa in ("avx2", "avx512"):
            key = f"{name}/{isa}"
            if key in data.files:
                ref = data[key]
                e = np.linalg.norm(y - ref) / np.linalg.norm(ref)
                assert e < 1e-6, (name, isa, e)


def test_oracle_properties_of_the_reference_test():
    """Properties the reference's own conversion test checks (tests/test_nmg.py:33-86): kept values are
    unchanged, at most n survivors per block of m, and more magnitude is kept than a random n/m choice."""
    rng = np.random.default_rng(123)
    n, m, g = 5, 12, 2
    for (M, K) in [(17, 5), (5, 17), (17, 17), (1, 5)]:
        w = rng.random((3, M, K), dtype=np.float32)
        val, idx = orc.sparsify(w, n, m, g)
        d = orc.densify(val, idx, w.shape, n, m, g)
        assert np.all((d == w) | (d == 0))
        pad = (-M) % m
        dp = np.pad(d, ((0, 0), (0, pad), (0, 0))).reshape(3, -1, m, K)
        assert (dp != 0).sum(axis=2).max() <= n
        assert np.abs(d).sum() / np.abs(w).sum() > n / m
