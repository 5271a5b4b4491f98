"""Index arithmetic of the grouped n:m ("nmg") format.

A weight is cut into blocks of ``m`` consecutive entries along ``sparse_dim`` and chunks of ``C*g``
consecutive entries along ``group_dim`` (``C = comb(m, n)``).  Inside one (block, chunk) tile every
position along ``group_dim`` keeps ``n`` of its ``m`` entries; the kept-entry pattern is one of the ``C``
n-subsets of ``[0, m)`` and exactly ``g`` positions use each pattern.  Positions are stored sorted by
pattern, in the fixed order returned by :func:`make_n_m`.

This module mirrors the bookkeeping of the reference (src/sten/grouped_nm/grouped_nm_tensor.py:37-50
``make_n_m`` and :71-217 ``compute_nm_strides``): same function names, same dictionary keys and values,
because the dictionary is pickled together with the tensor and reference pickles must stay loadable.
"""
import functools
import math


@functools.lru_cache(maxsize=None)
def _revolving_door(n, m, flip):
    """All sorted n-subsets of range(m) such that neighbours differ in exactly one element.

    ``flip`` reverses the part of the list that does not contain ``m - 1``; the recursion alternates it so
    that the two halves join with a one-element change.
    """
    if n == 0 or n == m:
        return (tuple(range(n)),)
    without_last = _revolving_door(n, m - 1, True)
    if flip:
        without_last = without_last[::-1]
    with_last = tuple(t + (m - 1,) for t in _revolving_door(n - 1, m - 1, not flip))
    return without_last + with_last


def make_n_m(n, m, special=False):
    """Pattern order of the format: list of ``comb(m, n)`` sorted n-tuples (reference :37-50)."""
    if not (0 <= n <= m):
        raise ValueError(f"need 0 <= n <= m, got n={n}, m={m}")
    return list(_revolving_door(int(n), int(m), bool(special)))


def is_valid_n_m(patterns, n, m):
    """True when ``patterns`` lists every n-subset once, sorted, neighbours one element apart (:24-34)."""
    if len(patterns) != math.comb(m, n):
        return False
    if any(list(p) != sorted(set(p)) for p in patterns):
        return False
    return all(sum(a != b for a, b in zip(p, q)) == 1 for p, q in zip(patterns[:-1], patterns[1:]))


def _prod(seq):
    return math.prod(seq)


def compute_nm_strides(dense_shape, n, m, sparse_dim, group_dim, group_size):
    """Shapes, strides and permutations that take a dense tensor to its tile view and back (:71-217).

    The padded tensor is viewed with ``sparse_dim`` split into ``[num_blocks, m]`` and ``group_dim`` split into
    ``[num_chunks, C, g]``; the five new axes are moved last, in the order
    ``[num_chunks, num_blocks, C, g, m]``, and everything in front of the last three is merged into one tile
    axis.  The result is cached per argument tuple and, like in the reference, the *same* dictionary object
    is handed out again for equal arguments.
    """
    return _compute_nm_strides_cached(dense_shape, int(n), int(m), int(sparse_dim), int(group_dim), int(group_size))


@functools.lru_cache(maxsize=None)
def _compute_nm_strides_cached(dense_shape, n, m, sparse_dim, group_dim, group_size):
    if sparse_dim == group_dim:
        raise ValueError("sparse_dim and group_dim must differ")
    C = math.comb(m, n)
    num_chunks = math.ceil(dense_shape[group_dim] / (C * group_size))
    num_blocks = math.ceil(dense_shape[sparse_dim] / m)
    split = {sparse_dim: [num_blocks, m], group_dim: [num_chunks, C, group_size]}

    padded = list(dense_shape)
    padded[sparse_dim] = num_blocks * m
    padded[group_dim] = num_chunks * C * group_size

    expanded, first_axis = [], {}
    for d, size in enumerate(padded):
        first_axis[d] = len(expanded)
        expanded.extend(split.get(d, [size]))
    es, eg = first_axis[sparse_dim], first_axis[group_dim]
    s_end, g_end = es + 2, eg + 3                       # one past the split axes of each dim
    lo_from, lo_to, hi_from, hi_to = (es, s_end, eg, g_end) if sparse_dim < group_dim else (eg, g_end, es, s_end)

    def with_block_len(k):
        return expanded[: es + 1] + [k] + expanded[es + 2:]

    val_shape, idx_shape = with_block_len(n), with_block_len(1)
    views = {"dense": expanded, "sparse": val_shape, "idx": idx_shape}

    moved_last = [eg, es, eg + 1, eg + 2, es + 1]
    perm = [a for a in range(len(expanded)) if a not in moved_last] + moved_last
    inv = sorted(range(len(perm)), key=perm.__getitem__)
    permuted = [expanded[a] for a in perm]

    out = {
        "n": n, "m": m, "sparse_dim": sparse_dim, "group_dim": group_dim, "group_size": group_size,
        "dense_shape": dense_shape,
        "padded_dense_shape": padded,
        "expanded_dense_shape": expanded,
        "chunk_size": C, "num_chunks": num_chunks, "num_blocks": num_blocks,
        "exp_sparse_dim": es, "exp_group_dim": eg,
        "smaller_dim_from": lo_from, "smaller_dim_to": lo_to, "larger_dim_from": hi_from, "larger_dim_to": hi_to,
        "sparse_val_shape": val_shape, "sparse_idx_shape": idx_shape,
        "loop_outer_size": _prod(expanded[: lo_from + 1]),
        "loop_middle_size": _prod(expanded[lo_to: hi_from + 1]),
        "loop_inner_size": _prod(expanded[hi_to:]),
        "order": make_n_m(n, m),
    }
    for name, view in views.items():
        out[f"{name}_block_stride"] = _prod(view[s_end:])
        out[f"{name}_group_stride"] = _prod(view[g_end:])
    for name, view in views.items():
        out[f"{name}_loop_middle_stride"] = _prod(view[hi_from + 1:])
        out[f"{name}_loop_outer_stride"] = _prod(view[lo_from + 1:])
    out.update({
        "padded_sparse_dim": num_blocks * m,
        "padded_group_dim": num_chunks * C * group_size,
        "dim_permutation": perm,
        "inverse_dim_permutation": inv,
        "permuted_shape": permuted,
        "merged_shape": [_prod(permuted[:-3]), *permuted[-3:]],
    })
    return out


def tile_geometry(rows, cols, n, m, g):
    """Sizes of the 2-D kernel view: rows along the n:m axis, cols along the group axis."""
    C = math.comb(m, n)
    cc = C * g
    nb, nc = -(-rows // m), -(-cols // cc)
    return {"C": C, "cc": cc, "nb": nb, "nc": nc, "Mp": nb * m, "Kp": nc * cc}
