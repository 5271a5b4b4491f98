"""Generate the golden fixtures of tests/golden/ from the reference implementation itself.

Run where the reference tree is available, naming it on the command line or in NMG_REFERENCE_ROOT:

    python tests/golden/gen_golden.py /path/to/reference [small|big|layout|spmm|pickle ...]

It imports the reference package (a stub stands in for the third-party ``dace`` module, which the
sparsifier / densifier never touch), runs the reference's own CPU sparsifier
(``GroupedNMTensor.from_dense``, src/sten/grouped_nm/grouped_nm_tensor.py:883-890 -> :220-305) and densifier
(``to_dense``, :953-958) on seeded inputs and stores

  * ``small_cases.npz``   inputs, ``val``, ``idx`` and ``to_dense()`` of small 2-D and 3-D cases that cover every
                          remainder (M %% m, K %% (C*g)), ties, zeros, and all dim permutations;
  * ``big_hashes.json``   sha256 of ``val`` / ``idx`` for the 1024 x 1024 and 4096 x 4096 benchmark weights and for the
                          16384 x 16384 bf16 2:8 weight of the sharded benchmark (N(0, 0.02) rounded to bf16, selection
                          on the fp32 magnitudes of the rounded values; ``val`` hashed as bf16 bits) --
                          inputs come from ``torch.Generator().manual_seed``; their sha256 is stored too;
  * ``reference_linear.pkl``  a pickle WRITTEN BY THE REFERENCE: a ``torch.nn.Linear`` whose weight is the reference's
                          ``SparseParameterWrapper`` around a ``GroupedNMTensor`` (made by its ``SparsityBuilder``), plus the
                          input and the dense weight it was made from in ``reference_linear.npz``;
  * ``perfect_cases.npz`` ``val`` / ``idx`` / ``to_dense()`` of the reference's ``PerfectNMTensor`` on tie-free random tensors;
  * ``layout.json``       ``make_n_m`` tables and every key of ``compute_nm_strides`` for a list of shapes;
  * ``spmm_cases.npz``    outputs of the reference's AVX micro-kernels (built by oracle/build_ref.py) on small
                          problems with k-remainders.

The fixtures travel with the repository; the reference tree does not.
"""
import hashlib
import itertools
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402


def sha(t):
    return hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest()


def seeded_normal(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def main(ref_root=None, *parts):
    ref_root = build_ref.reference_root(ref_root)
    if ref_root is None:
        raise SystemExit("no reference tree: pass its path or set NMG_REFERENCE_ROOT")
    parts = set(parts) or {"small", "big", "layout", "spmm", "pickle", "perfect"}
    build_ref.import_reference(ref_root)
    import tempfile
    os.chdir(tempfile.gettempdir())  # the reference JIT writes ./.compile_cache
    from sten.grouped_nm.grouped_nm_tensor import GroupedNMTensor, compute_nm_strides, make_n_m
    if "small" in parts:
        gen_small(GroupedNMTensor)
    if "big" in parts:
        gen_big(GroupedNMTensor)
    if "layout" in parts:
        gen_layout(compute_nm_strides, make_n_m)
    if "spmm" in parts:
        gen_spmm(GroupedNMTensor)
    if "pickle" in parts:
        gen_pickle()
    if "perfect" in parts:
        gen_perfect()
    print("done")


def gen_perfect():
    """PerfectNMTensor.from_dense / to_dense of the reference (grouped_nm_tensor.py:1010-1066) on tie-free random tensors:
    every position of the sparse dimension, ragged block counts, n = m, and the 3-D shapes of its conversion test."""
    from sten.grouped_nm.grouped_nm_tensor import PerfectNMTensor
    out, meta = {}, []
    seed = 900
    for (shape, n, m, sd) in [((64, 100), 2, 4, 0), ((64, 100), 2, 4, 1), ((30, 50), 1, 4, 1), ((37, 120), 2, 8, 0),
                              ((50, 64), 1, 16, 1), ((3, 5, 17), 5, 12, 2), ((3, 17, 5), 5, 12, 1), ((17, 3, 5), 2, 4, 0),
                              ((9, 10), 4, 4, 1), ((7, 13), 3, 6, 1), ((2, 3, 16, 40), 1, 8, 2)]:
        seed += 1
        dense = seeded_normal(shape, seed)
        t = PerfectNMTensor.from_dense(dense, n, m, sd)
        name = f"perfect_{n}_{m}_{sd}_" + "x".join(map(str, shape))
        out[name + "/dense"] = dense.numpy()
        out[name + "/val"] = t.val.contiguous().numpy()
        out[name + "/idx"] = t.idx.contiguous().numpy()
        out[name + "/to_dense"] = t.to_dense().contiguous().numpy()
        meta.append(dict(name=name, n=n, m=m, sparse_dim=sd, shape=list(shape)))
    np.savez_compressed(os.path.join(HERE, "perfect_cases.npz"), **out)
    with open(os.path.join(HERE, "perfect_cases.json"), "w") as f:
        json.dump(meta, f, indent=1)


def gen_pickle():
    """A model pickled by the reference runtime itself (sten.py:178-189, 413-420 define what lands in the file)."""
    import sten
    torch.manual_seed(7)
    lin = torch.nn.Linear(100, 24)
    x = seeded_normal((9, 100), 8)
    sb = sten.SparsityBuilder()
    sb.set_weight("weight", initial_sparsifier=sten.GroupedNMSparsifier(2, 4, 2), out_format=sten.GroupedNMTensor)
    dense_w = lin.weight.detach().clone().numpy()
    sparse = sb.get_sparse_model(lin)
    torch.save(sparse, os.path.join(HERE, "reference_linear.pkl"))
    gnm = sparse.weight.wrapped_tensor
    np.savez_compressed(os.path.join(HERE, "reference_linear.npz"), w=dense_w, b=lin.bias.detach().numpy(), x=x.numpy(),
                        val=gnm.val.numpy(), idx=gnm.idx.numpy(), to_dense=gnm.to_dense().contiguous().numpy())
    print("pickled a reference-made sparse Linear:", type(sparse.weight).__module__, type(gnm).__module__)


def gen_small(GroupedNMTensor):
    # ---------------------------------------------------------------- small cases
    small = {}
    meta = []

    def add_case(name, dense, n, m, g, sparse_dim, group_dim):
        t = GroupedNMTensor.from_dense(dense, n, m, sparse_dim=sparse_dim, group_size=g, group_dim=group_dim)
        small[name + "/dense"] = dense.numpy()
        small[name + "/val"] = t.val.numpy()
        small[name + "/idx"] = t.idx.numpy()
        small[name + "/to_dense"] = t.to_dense().contiguous().numpy()
        meta.append(dict(name=name, n=n, m=m, g=g, sparse_dim=sparse_dim, group_dim=group_dim,
                         shape=list(dense.shape)))

    seed = 100
    for (n, m, g, M, K) in [
        (2, 4, 4, 64, 100), (2, 4, 16, 32, 200), (1, 4, 3, 30, 50), (1, 4, 16, 16, 128), (1, 8, 2, 40, 70),
        (2, 8, 2, 37, 120), (1, 16, 2, 50, 64), (3, 6, 4, 18, 96), (2, 4, 1, 7, 13), (4, 4, 3, 9, 10),
        (5, 12, 2, 17, 40), (1, 2, 5, 6, 33),
    ]:
        seed += 1
        add_case(f"randn_{n}_{m}_{g}_{M}x{K}", seeded_normal((M, K), seed), n, m, g, 0, 1)
    # ties: small-integer weights, many equal scores and exact zeros
    for (n, m, g, M, K) in [(2, 4, 4, 16, 60), (1, 8, 2, 24, 50), (2, 8, 1, 16, 60)]:
        seed += 1
        gen = torch.Generator().manual_seed(seed)
        w = torch.randint(-2, 3, (M, K), generator=gen).to(torch.float32)
        add_case(f"ties_{n}_{m}_{g}_{M}x{K}", w, n, m, g, 0, 1)
    add_case("zeros_2_4_2_8x20", torch.zeros(8, 20), 2, 4, 2, 0, 1)
    # 3-D tensors, every dim permutation (the shape family of the reference's conversion test)
    base = "abc"
    for perm in itertools.permutations(base):
        layout = "".join(perm)
        seed += 1
        g_ = torch.Generator().manual_seed(seed)
        src = torch.rand(3, 5, 17, generator=g_)
        dense = torch.einsum(f"{base}->{layout}", src)
        add_case(f"perm_{layout}", dense, 2, 4, 2, layout.index("c"), layout.index("b"))
    np.savez_compressed(os.path.join(HERE, "small_cases.npz"), **small)
    with open(os.path.join(HERE, "small_cases.json"), "w") as f:
        json.dump(meta, f, indent=1)



def gen_big(GroupedNMTensor):
    # ---------------------------------------------------------------- benchmark-size hashes
    big = []
    for (M, K, n, m, g, seed_) in [
        (1024, 1024, 2, 4, 4, 0), (1024, 1024, 2, 4, 16, 0),
        (4096, 4096, 1, 4, 16, 0), (4096, 4096, 2, 4, 16, 0), (4096, 4096, 1, 8, 16, 0),
        (4096, 4096, 2, 8, 16, 0), (4096, 4096, 1, 16, 16, 0),
    ]:
        w = seeded_normal((M, K), seed_)
        t = GroupedNMTensor.from_dense(w, n, m, sparse_dim=0, group_size=g, group_dim=1)
        big.append(dict(M=M, K=K, n=n, m=m, g=g, seed=seed_, dense_sha256=sha(w.numpy()),
                        val_sha256=sha(t.val.numpy()), idx_sha256=sha(t.idx.numpy()),
                        val_shape=list(t.val.shape), idx_shape=list(t.idx.shape)))
        print("hashed", M, K, n, m, g)
    # the sharded benchmark's weight: N(0, 0.02) rounded to bf16; the reference sees the rounded values as fp32
    M = K = 16384
    n, m, g, seed_ = 2, 8, 16, 0
    w = (seeded_normal((M, K), seed_) * 0.02).bfloat16()
    t = GroupedNMTensor.from_dense(w.float(), n, m, sparse_dim=0, group_size=g, group_dim=1)
    val16 = t.val.bfloat16()
    assert torch.equal(val16.float(), t.val)  # kept values are the bf16 inputs, exactly
    big.append(dict(M=M, K=K, n=n, m=m, g=g, seed=seed_, scale=0.02, dtype="bf16",
                    dense_sha256=sha(w.view(torch.int16).numpy()), val_sha256=sha(val16.view(torch.int16).numpy()),
                    idx_sha256=sha(t.idx.numpy()), val_shape=list(t.val.shape), idx_shape=list(t.idx.shape)))
    print("hashed", M, K, n, m, g, "bf16")
    with open(os.path.join(HERE, "big_hashes.json"), "w") as f:
        json.dump(big, f, indent=1)


def gen_layout(compute_nm_strides, make_n_m):
    # ---------------------------------------------------------------- layout tables
    layout = {"make_n_m": {}, "nm_strides": []}
    for (n, m) in [(1, 4), (2, 4), (3, 4), (1, 8), (2, 8), (4, 8), (1, 16), (2, 16), (3, 6), (5, 12), (2, 2), (0, 3)]:
        layout["make_n_m"][f"{n}:{m}"] = [list(t) for t in make_n_m(n, m)]
    for (shape, n, m, sd, gd, g) in [
        ((8, 30), 2, 4, 0, 1, 2), ((1024, 1024), 2, 4, 0, 1, 16), ((30, 8), 2, 4, 1, 0, 2),
        ((3, 5, 17), 2, 4, 2, 1, 2), ((3, 17, 5), 2, 4, 1, 2, 2), ((17, 3, 5), 1, 8, 0, 2, 3),
        ((5, 17, 3), 2, 8, 1, 0, 1), ((2, 3, 16, 40), 1, 4, 2, 3, 4), ((4096, 4096), 2, 8, 0, 1, 16),
    ]:
        d = compute_nm_strides(torch.Size(shape), n, m, sd, gd, g)
        layout["nm_strides"].append(dict(
            args=dict(shape=list(shape), n=n, m=m, sparse_dim=sd, group_dim=gd, group_size=g),
            result={k: (list(v) if isinstance(v, (list, tuple, torch.Size)) else v) for k, v in d.items()
                    if k != "order"},
            order=[list(t) for t in d["order"]]))
    with open(os.path.join(HERE, "layout.json"), "w") as f:
        json.dump(layout, f)



def gen_spmm(GroupedNMTensor):
    # ---------------------------------------------------------------- matmul through the reference micro-kernels
    spmm = {}
    seed = 500
    for (n, m, g, K, M, ntok) in [(2, 4, 2, 100, 24, 64), (1, 4, 3, 50, 30, 64), (2, 8, 2, 120, 37, 128),
                                  (3, 6, 4, 96, 18, 64)]:
        seed += 1
        w = seeded_normal((M, K), seed)
        x = seeded_normal((ntok, K), seed + 1000)
        t = GroupedNMTensor.from_dense(w, n, m, sparse_dim=0, group_size=g, group_dim=1)
        for isa in ("avx2", "avx512"):
            try:
                y = build_ref.spmm(t.val.numpy(), t.idx.numpy(), x.numpy(), M, K, n, m, g, isa=isa)
            except OSError:
                continue
            spmm[f"{n}_{m}_{g}_{M}x{K}_{ntok}/{isa}"] = y
        spmm[f"{n}_{m}_{g}_{M}x{K}_{ntok}/w"] = w.numpy()
        spmm[f"{n}_{m}_{g}_{M}x{K}_{ntok}/x"] = x.numpy()
    np.savez_compressed(os.path.join(HERE, "spmm_cases.npz"), **spmm)


if __name__ == "__main__":
    main(*sys.argv[1:])
