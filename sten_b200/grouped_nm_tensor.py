"""``GroupedNMTensor`` and friends: the tensor types of the grouped n:m format.

Same public surface as the reference module (src/sten/grouped_nm/grouped_nm_tensor.py:877-1091): the object holds
``val`` (kept values, ``[tiles, C, g, n]``), ``idx`` (int16 column positions, ``[tiles, C, g, 1]``) and ``nm_strides``
(the layout dictionary), and these three attributes are all that is pickled.  Conversion in both directions is
one CUDA kernel each (``nmg_sparsify`` / ``nmg_densify`` of the C ABI) that reads / writes the dense tensor in
place; there is no run-time code generation and no CPU path.
"""
import math

import torch

from . import ops
from .layout import compute_nm_strides, make_n_m  # noqa: F401  (re-exported like the reference module does)


def pad_to(tensor, new_shape):
    pads = []
    for have, want in zip(reversed(tensor.shape), reversed(list(new_shape))):
        pads += [0, want - have]
    return torch.nn.functional.pad(tensor, pads)


def unpad_to(tensor, new_shape):
    if tensor.ndim != len(new_shape):
        raise ValueError("rank mismatch")
    for d, length in enumerate(new_shape):
        tensor = tensor.narrow(d, 0, length)
    return tensor


def _kernel_view(tensor, sparse_dim, group_dim):
    """[B, rows, cols] view of ``tensor`` with the n:m axis as rows and the group axis as cols.

    The remaining dims keep their order and are flattened into B, which is the tile order of the format."""
    others = [d for d in range(tensor.ndim) if d not in (sparse_dim, group_dim)]
    moved = tensor.permute(*others, sparse_dim, group_dim)
    rows, cols = moved.shape[-2], moved.shape[-1]
    if moved.ndim == 2:
        return moved.unsqueeze(0), others
    if moved.ndim > 3:
        moved = moved.reshape(-1, rows, cols)  # copies only when the leading dims cannot be merged
    return moved, others


def dense_to_grouped_n_m(tensor, n, m, sparse_dim, group_size, group_dim):
    """dense -> (val, idx, nm_strides); reference: grouped_nm_tensor.py:701-710."""
    sparse_dim %= tensor.ndim
    group_dim %= tensor.ndim
    nm_strides = compute_nm_strides(tensor.shape, n, m, sparse_dim, group_dim, group_size)
    view3, _ = _kernel_view(tensor.detach(), sparse_dim, group_dim)
    val, idx = ops.sparsify(view3, n, m, group_size)
    return val, idx, nm_strides


def grouped_n_m_to_dense(nm_strides, val, idx):
    """(val, idx) -> dense tensor of ``nm_strides['dense_shape']``; reference: grouped_nm_tensor.py:848-874."""
    shape = list(nm_strides["dense_shape"])
    sd, gd = nm_strides["sparse_dim"], nm_strides["group_dim"]
    others = [d for d in range(len(shape)) if d not in (sd, gd)]
    B = math.prod(shape[d] for d in others) if others else 1
    out3 = ops.densify(val, idx, B, shape[sd], shape[gd], nm_strides["n"], nm_strides["m"], nm_strides["group_size"])
    moved = out3.reshape([shape[d] for d in others] + [shape[sd], shape[gd]])
    order = others + [sd, gd]
    inverse = sorted(range(len(order)), key=order.__getitem__)
    return moved.permute(*inverse)


class GroupedNMTensor:
    def __init__(self, val, idx, nm_strides):
        self.val = val
        self.idx = idx
        self.nm_strides = nm_strides

    @staticmethod
    def from_dense(tensor, n, m, sparse_dim, group_size, group_dim):
        val, idx, nm_strides = dense_to_grouped_n_m(tensor, n, m, sparse_dim, group_size, group_dim)
        ten = GroupedNMTensor(val, idx, nm_strides)
        ten.set_spmm_opt()
        return ten

    def set_spmm_opt(self, tile_a=None, acc_width=None, tile_b=None, kernel=None):
        """The reference tunes its CPU micro-kernel with these knobs (:892-902); the CUDA kernels choose their own tiling,
        so ``tile_a`` / ``acc_width`` / ``tile_b`` are only recorded (pickles carry the same keys as reference pickles).

        ``kernel`` names the kernel family: ``"sm100"`` (default: the weight stays compressed, large batches expand it into
        a transient workspace on every call) or ``"sm100-expanded"`` (opt-in for compute-bound serving of 16-bit weights:
        the expanded weight is kept after first use, which skips the per-call expansion pass and gives up the format's
        memory saving)."""
        self.nm_strides["tile_a"] = tile_a or 3
        self.nm_strides["acc_width"] = acc_width or 4
        self.nm_strides["tile_b"] = tile_b or 16
        self.nm_strides["kernel"] = kernel or "sm100"

    def clone_layout(self, dense_tensor):
        """A tensor with THIS tensor's layout (same ``idx``, shared) holding ``dense_tensor``'s values at the kept
        positions: no new magnitude selection.  The reference sketches this (grouped_nm_tensor.py:904-951) and leaves it
        disabled; it is what keeps a weight gradient, or an optimizer update, in the weight's own layout."""
        s = self.nm_strides
        if tuple(dense_tensor.shape) != tuple(s["dense_shape"]):
            raise ValueError(f"expected a tensor of shape {tuple(s['dense_shape'])}, got {tuple(dense_tensor.shape)}")
        view3, _ = _kernel_view(dense_tensor.detach(), s["sparse_dim"], s["group_dim"])
        val = ops.gather_layout(view3, self.idx, s["n"], s["m"], s["group_size"])
        return GroupedNMTensor(val, self.idx, s)

    def to_dense(self):
        return grouped_n_m_to_dense(self.nm_strides, self.val, self.idx)

    # -- conveniences the reference object lacks (its wrapper densifies just to learn dtype / device) ----------
    @property
    def dtype(self):
        return self.val.dtype

    @property
    def device(self):
        return self.val.device

    @property
    def shape(self):
        return torch.Size(self.nm_strides["dense_shape"])

    def packed(self):
        """Column-ordered device copy used by the tensor-core and transposed kernels (``nmg_pack``).

        Built on first use and kept while ``val`` / ``idx`` are the same tensors at the same version; it is a
        cache, never pickled."""
        s = self.nm_strides
        if len(s["dense_shape"]) != 2 or s["sparse_dim"] != 0:
            raise ValueError("the packed copy exists for 2-D weights with n:m blocks along dim 0")
        key = (self.val.data_ptr(), self.val._version, self.idx.data_ptr(), self.idx._version, self.val.dtype)
        cache = self.__dict__.get("_packed_cache")
        if cache is None or cache[0] != key:
            M, K = s["dense_shape"]
            cache = (key, ops.pack(self.val, self.idx, int(M), int(K), s["n"], s["m"], s["group_size"]))
            self.__dict__["_packed_cache"] = cache
        return cache[1]

    def expanded(self):
        """Kept dense 16-bit copy for ``kernel="sm100-expanded"`` (``nmg_expand``), or None when there is none (fp32,
        weights that are not 2-D with n:m blocks along dim 0).  Cached like ``packed()``; never pickled."""
        s = self.nm_strides
        if len(s["dense_shape"]) != 2 or s["sparse_dim"] != 0 or not self.val.is_cuda or self.val.dtype == torch.float32:
            return None
        key = (self.val.data_ptr(), self.val._version, self.idx.data_ptr(), self.idx._version, self.val.dtype)
        cache = self.__dict__.get("_expanded_cache")
        if cache is None or cache[0] != key:
            M, K = (int(v) for v in s["dense_shape"])
            cache = (key, ops.expand(self.val, self.idx, M, K, s["n"], s["m"], s["group_size"]))
            self.__dict__["_expanded_cache"] = cache
        return cache[1]

    def packed_sp24(self):
        """Compressed transposed copy for the structured-sparse backward product (``nmg_pack_sp24``), or None when the
        weight is outside the 2:4 structure (fp32, n > 2, m not a power of two >= 4).  Cached like ``packed()``."""
        s = self.nm_strides
        if len(s["dense_shape"]) != 2 or s["sparse_dim"] != 0:
            return None
        M, K = (int(v) for v in s["dense_shape"])
        if not self.val.is_cuda or ops.sp24_bytes(M, K, s["n"], s["m"], s["group_size"], self.val.dtype) == 0:
            return None
        key = (self.val.data_ptr(), self.val._version, self.idx.data_ptr(), self.idx._version, self.val.dtype)
        cache = self.__dict__.get("_sp24_cache")
        if cache is None or cache[0] != key:
            cache = (key, ops.pack_sp24(self.val, self.idx, M, K, s["n"], s["m"], s["group_size"]))
            self.__dict__["_sp24_cache"] = cache
        return cache[1]

    def to(self, device=None, dtype=None, non_blocking=False, copy=False):
        """Same layout on another device / in another floating dtype (indices are dtype independent)."""
        val = self.val.to(device=device, dtype=dtype, non_blocking=non_blocking, copy=copy)
        idx = self.idx.to(device=device, non_blocking=non_blocking, copy=copy)
        return GroupedNMTensor(val, idx, self.nm_strides)

    def __getstate__(self):
        return {"val": self.val, "idx": self.idx, "nm_strides": self.nm_strides}

    def __setstate__(self, state):
        self.__dict__.update(state)

    def __repr__(self):
        s = self.nm_strides
        return (f"GroupedNMTensor(shape={tuple(s['dense_shape'])}, n={s['n']}, m={s['m']}, g={s['group_size']}, "
                f"dtype={self.val.dtype}, device={self.val.device})")


class PerfectNMTensor:
    """Per-block top-n by magnitude without the group constraint (reference :1010-1066): ``val`` / ``idx`` of shape
    ``[..., blocks, n, ...]`` with ``idx`` the int64 positions inside each block of m, by descending magnitude.
    Both directions are one CUDA kernel each (``nmg_perfect_nm_select`` / ``nmg_perfect_nm_densify``)."""

    def __init__(self, val, idx, n, m, sparse_dim, sparse_dim_size):
        self.val = val
        self.idx = idx
        self.n = n
        self.m = m
        self.sparse_dim = sparse_dim
        self.sparse_dim_size = sparse_dim_size

    @staticmethod
    def from_dense(dense_tensor, n, m, sparse_dim):
        sparse_dim %= dense_tensor.ndim
        val, idx = ops.perfect_nm_select(dense_tensor.detach(), n, m, sparse_dim)
        return PerfectNMTensor(val, idx, n, m, sparse_dim, dense_tensor.shape[sparse_dim])

    def to_dense(self):
        return ops.perfect_nm_densify(self.val, self.idx, self.n, self.m, self.sparse_dim, self.sparse_dim_size)


def is_correct_nm(original_dense, sparsified_dense, sparse_dim, n, m):
    """Property check of the reference tests (:1069-1091): survivors are unchanged, at most n per block of m."""
    untouched = (original_dense == sparsified_dense) | (sparsified_dense == 0)
    if not bool(untouched.all()):
        return False
    size = original_dense.shape[sparse_dim]
    blocks = math.ceil(size / m)
    padded_shape = list(original_dense.shape)
    padded_shape[sparse_dim] = blocks * m
    split = pad_to(sparsified_dense, padded_shape).reshape(
        *original_dense.shape[:sparse_dim], blocks, m, *original_dense.shape[sparse_dim + 1:])
    return bool((split.bool().sum(dim=sparse_dim + 1) <= n).all())
