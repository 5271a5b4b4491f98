"""Fused epilogues for grouped n:m linears inside transformer blocks (inference).

The reference runs ``F.linear`` and leaves bias, activation and residual to separate passes over the output
(src/sten/grouped_nm/sten_impls.py:170-173 adds the bias itself, the model code does the rest).  ``nmg_spmm_fused`` does
``activation(x W^T + b) + residual`` in the matmul's epilogue, so the intermediate is written once.  ``fuse_linear_epilogues``
rewires the two module shapes every BERT-style encoder is made of:

* ``dense`` + ``intermediate_act_fn`` (exact GELU)            -> one call with ``activation="gelu"``
* ``dense`` + ``dropout`` + ``LayerNorm(hidden + input)``     -> one call with ``residual=input`` followed by the LayerNorm

Only modules whose ``dense.weight`` is a grouped n:m parameter are touched, and only while gradients are disabled and
dropout is inactive; otherwise the module's own forward runs.
"""
import types

import torch

from . import _native as nat
from . import ops
from .dispatch import SparseTensorWrapper
from .grouped_nm_tensor import GroupedNMTensor


def _nmg_weight(linear):
    w = getattr(linear, "weight", None)
    if isinstance(w, SparseTensorWrapper) and isinstance(w.wrapped_tensor, GroupedNMTensor):
        s = w.wrapped_tensor.nm_strides
        if len(s["dense_shape"]) == 2 and s["sparse_dim"] == 0 and s["group_dim"] == 1:
            return w.wrapped_tensor
    return None


def sparse_linear_fused(x, gnm, bias=None, activation=None, residual=None):
    """``activation(x W^T + bias) + residual`` for a grouped n:m weight in one library call (no autograd)."""
    s = gnm.nm_strides
    M, K = (int(v) for v in s["dense_shape"])
    n, m, g = s["n"], s["m"], s["group_size"]
    x2d = x.reshape(-1, K)
    tokens = x2d.shape[0]
    res2d = residual.reshape(-1, M) if residual is not None else None
    from .nmg_impls import _wants_expanded
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    if _wants_expanded(gnm, x2d, tokens):
        return ops.spmm_expanded(gnm.expanded(), M, K, x2d, bias=bias, activation=activation, residual=res2d).reshape(*x.shape[:-1], M)
    packed = gnm.packed() if tokens and ops.uses_packed(M, K, tokens, n, m, g, gnm.val.dtype, nat.NMG_ACT_TOKEN_MAJOR) else None
    y = ops.spmm(gnm.val, gnm.idx, M, K, n, m, g, x2d, bias=bias, packed=packed, activation=activation, residual=res2d)
    return y.reshape(*x.shape[:-1], M)


def _is_exact_gelu(fn):
    name = type(fn).__name__ if not isinstance(fn, types.FunctionType) else fn.__name__
    return name in ("GELUActivation", "GELU", "gelu") and not getattr(fn, "approximate", "none") == "tanh"


def _fused_intermediate_forward(self, hidden_states):
    gnm = _nmg_weight(self.dense)
    if gnm is None or torch.is_grad_enabled() or not hidden_states.is_cuda:
        return self._sten_unfused_forward(hidden_states)
    return sparse_linear_fused(hidden_states, gnm, self.dense.bias, activation="gelu")


def _fused_output_forward(self, hidden_states, input_tensor):
    gnm = _nmg_weight(self.dense)
    dropout_off = (not self.training) or getattr(self.dropout, "p", 0.0) == 0.0
    if gnm is None or torch.is_grad_enabled() or not dropout_off or not hidden_states.is_cuda:
        return self._sten_unfused_forward(hidden_states, input_tensor)
    return self.LayerNorm(sparse_linear_fused(hidden_states, gnm, self.dense.bias, residual=input_tensor))


def fuse_linear_epilogues(model):
    """Rewire ``dense`` + GELU and ``dense`` + residual + LayerNorm modules of ``model`` whose dense weight is grouped n:m.
    Returns the number of modules rewired.  Idempotent."""
    count = 0
    for mod in model.modules():
        dense = getattr(mod, "dense", None)
        if not isinstance(dense, torch.nn.Linear) or _nmg_weight(dense) is None or hasattr(mod, "_sten_unfused_forward"):
            continue
        if hasattr(mod, "intermediate_act_fn") and _is_exact_gelu(mod.intermediate_act_fn):
            mod._sten_unfused_forward = mod.forward
            mod.forward = types.MethodType(_fused_intermediate_forward, mod)
            count += 1
        elif hasattr(mod, "LayerNorm") and hasattr(mod, "dropout"):
            mod._sten_unfused_forward = mod.forward
            mod.forward = types.MethodType(_fused_output_forward, mod)
            count += 1
    return count
