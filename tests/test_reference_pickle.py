"""A pickle written by the reference runtime loads here (serialization row of the format contract).

``tests/golden/reference_linear.pkl`` was written by the reference's own ``torch.save`` of a ``torch.nn.Linear`` whose
weight its ``SparsityBuilder`` turned into a ``SparseParameterWrapper`` around a ``GroupedNMTensor`` (n:m = 2:4, g = 2;
generator: tests/golden/gen_golden.py).  The file names the reference's modules (``sten.sten``,
``sten.grouped_nm.grouped_nm_tensor``); aliasing those names to this package is all it takes, because the pickled state
is the same three attributes (reference: src/sten/sten.py:178-189, 413-420)."""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN


def _alias(monkeypatch):
    import sten_b200
    import sten_b200.dispatch
    import sten_b200.grouped_nm_tensor
    import sten_b200.nmg_impls
    for name, mod in {"sten": sten_b200, "sten.sten": sten_b200.dispatch, "sten.grouped_nm": sten_b200,
                      "sten.grouped_nm.grouped_nm_tensor": sten_b200.grouped_nm_tensor,
                      "sten.grouped_nm.sten_impls": sten_b200.nmg_impls}.items():
        monkeypatch.setitem(sys.modules, name, mod)


def _load(monkeypatch):
    _alias(monkeypatch)
    model = torch.load(os.path.join(GOLDEN, "reference_linear.pkl"), weights_only=False)
    return model, np.load(os.path.join(GOLDEN, "reference_linear.npz"))


def test_reference_pickle_loads_into_this_package(monkeypatch):
    import sten_b200 as sten
    model, data = _load(monkeypatch)
    w = model.weight
    assert isinstance(w, sten.SparseParameterWrapper) and isinstance(w.wrapped_tensor, sten.GroupedNMTensor)
    gnm = w.wrapped_tensor
    assert np.array_equal(gnm.val.numpy(), data["val"]) and np.array_equal(gnm.idx.numpy(), data["idx"])
    s = gnm.nm_strides
    assert (s["n"], s["m"], s["group_size"], s["sparse_dim"], s["group_dim"]) == (2, 4, 2, 0, 1)
    assert tuple(s["dense_shape"]) == (24, 100)
    assert w.requires_grad and len(w.grad_fmt) == 4


@pytest.mark.gpu
def test_reference_pickle_runs_on_the_gpu(monkeypatch):
    """.to('cuda') of the loaded weight, F.linear through the plugin, densify: all against what the reference stored."""
    import sten_b200 as sten
    model, data = _load(monkeypatch)
    sten.set_dispatch_failure("raise")
    dev = torch.device("cuda", 0)
    model = model.to(dev)
    gnm = model.weight.wrapped_tensor
    assert gnm.val.is_cuda and gnm.idx.is_cuda
    assert np.array_equal(gnm.to_dense().cpu().numpy(), data["to_dense"])
    x = torch.from_numpy(data["x"]).to(dev)
    with torch.no_grad():
        y = model(x)
    want = data["x"].astype(np.float64) @ data["to_dense"].astype(np.float64).T + data["b"].astype(np.float64)
    err = np.linalg.norm(y.cpu().numpy().astype(np.float64) - want) / np.linalg.norm(want)
    assert err <= 1e-5
    # and back: what this package pickles, the same aliasing loads again with identical tensors
    import io
    buf = io.BytesIO()
    torch.save(model, buf)
    buf.seek(0)
    again = torch.load(buf, weights_only=False)
    assert torch.equal(again.weight.wrapped_tensor.val, gnm.val) and torch.equal(again.weight.wrapped_tensor.idx, gnm.idx)
