"""Layout bookkeeping against tables dumped from the reference (tests/golden/layout.json)."""
import json
import os

import torch

from conftest import GOLDEN
from sten_b200.layout import compute_nm_strides, is_valid_n_m, make_n_m


def _load():
    with open(os.path.join(GOLDEN, "layout.json")) as f:
        return json.load(f)


def test_make_n_m_matches_reference_tables():
    for key, table in _load()["make_n_m"].items():
        n, m = map(int, key.split(":"))
        got = make_n_m(n, m)
        assert [list(t) for t in got] == table, key
        assert is_valid_n_m(got, n, m) or n in (0, m)


def test_make_n_m_known_answers():
    assert make_n_m(2, 4) == [(0, 1), (0, 2), (1, 2), (1, 3), (0, 3), (2, 3)]
    assert make_n_m(1, 4) == [(1,), (0,), (2,), (3,)]


def test_compute_nm_strides_matches_reference():
    for case in _load()["nm_strides"]:
        a = case["args"]
        got = compute_nm_strides(torch.Size(a["shape"]), a["n"], a["m"], a["sparse_dim"], a["group_dim"],
                                 a["group_size"])
        assert [list(t) for t in got["order"]] == case["order"]
        # the reference mutates its cached dict in set_spmm_opt (:899-902); those four knobs are not layout
        want = {k: v for k, v in case["result"].items() if k not in ("tile_a", "acc_width", "tile_b", "kernel")}
        assert set(want) == set(got) - {"order"}
        for k, v in want.items():
            g = got[k]
            g = list(g) if isinstance(g, (list, tuple, torch.Size)) else g
            assert g == v, (a, k, g, v)
        # key order matters for nobody, but the pickled dict must carry exactly the reference's keys
        assert isinstance(got["dense_shape"], torch.Size)


def test_compute_nm_strides_is_cached_object():
    a = compute_nm_strides(torch.Size((8, 30)), 2, 4, 0, 1, 2)
    b = compute_nm_strides(torch.Size((8, 30)), 2, 4, 0, 1, 2)
    assert a is b
