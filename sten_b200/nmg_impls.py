"""The grouped n:m plugin: sparsifier and operator registrations (reference: src/sten/grouped_nm/sten_impls.py).

Registered here, all backed by ``libnmg_b200.so``:

* ``GroupedNMSparsifier`` : ``torch.Tensor -> GroupedNMTensor``                    (reference sten_impls.py:13-37)
* ``F.linear``  forward for ``(Tensor, GroupedNMTensor, Tensor)`` -- the reference's only operator (:143-174) -- and for
  ``(Tensor, GroupedNMTensor)``: a bias-free linear has two tensor inputs and would otherwise miss the registration
  and silently densify;
* ``torch.mm`` / ``torch.matmul`` forward for ``(GroupedNMTensor, Tensor)``;
* the matching backward entries (``dX = dY W`` through the transposed kernel); the reference has none and installs a
  failing stub (sten.py:1690-1693).

Unlike the reference (sten_impls.py:53, which derives the transpose flag from contiguity and ends up reading a
contiguous ``[tokens, K]`` activation as ``[K, tokens]``), the activation layout is stated explicitly:
``F.linear`` is ``y = x W^T + b`` on ``x[tokens, K]``.
"""
import torch

from . import _native as nat
from . import dispatch as sten
from . import ops
from .grouped_nm_tensor import GroupedNMTensor


class GroupedNMSparsifier:
    def __init__(self, n, m, g):
        self.n = n
        self.m = m
        self.g = g


class WeightLayoutSparsifier:
    """Inline gradient sparsifier of a grouped n:m weight: the gradient keeps the weight's own layout (same ``idx``),
    only the kept positions are stored.  Declared per weight with::

        sb.set_weight_grad(name, inline_sparsifier=WeightLayoutSparsifier(), tmp_format=GroupedNMTensor,
                           external_sparsifier=KeepAll(), out_format=GroupedNMTensor)

    The reference leaves this open (``clone_layout`` is disabled, grouped_nm_tensor.py:904-951; its linear backward
    returns dense gradients only).  With it the gradient, the optimizer's view of it and the bytes a data-parallel
    all-reduce moves are n/m of the dense size, and the layout is identical on every rank."""


@sten.register_sparsifier_implementation(sparsifier=GroupedNMSparsifier, inp=torch.Tensor, out=GroupedNMTensor)
def dense_to_grouped_nm(sparsifier, tensor, grad_fmt=None):
    gnm = GroupedNMTensor.from_dense(tensor, sparsifier.n, sparsifier.m, sparse_dim=tensor.ndim - 2,
                                     group_size=sparsifier.g, group_dim=tensor.ndim - 1)
    return sten.SparseTensorWrapper.wrapped_from_dense(gnm, tensor, grad_fmt)


@sten.register_sparsifier_implementation(sparsifier=sten.SameFormatSparsifier, inp=torch.Tensor, out=GroupedNMTensor)
def dense_to_same_grouped_nm(sparsifier, tensor, grad_fmt=None):
    """Re-sparsify a dense result with the (n, m, g, dims) of the reference tensor (fresh magnitude selection)."""
    ref = sparsifier.ref_sp_ten
    s = ref.wrapped_tensor.nm_strides
    gnm = GroupedNMTensor.from_dense(tensor, s["n"], s["m"], sparse_dim=s["sparse_dim"], group_size=s["group_size"],
                                     group_dim=s["group_dim"])
    return sten.SparseTensorWrapper.wrapped_from_dense(gnm, tensor, grad_fmt if grad_fmt is not None else ref.grad_fmt)


def _weight_geometry(weight):
    gnm = weight.wrapped_tensor
    s = gnm.nm_strides
    if len(s["dense_shape"]) != 2 or s["sparse_dim"] != 0 or s["group_dim"] != 1:
        raise sten.DispatchError("grouped n:m matmul needs a 2-D weight with n:m blocks along dim 0 and groups along dim 1")
    M, K = s["dense_shape"]
    return gnm, int(M), int(K), s["n"], s["m"], s["group_size"]


def _packed_or_none(gnm, geometry, tokens, layout=nat.NMG_ACT_TOKEN_MAJOR, transposed=False):
    """The cached column-ordered copy when the kernel that will run reads it, else None (nothing is built)."""
    M, K, n, m, g = geometry
    if not gnm.val.is_cuda or not ops.uses_packed(M, K, tokens, n, m, g, gnm.val.dtype, layout, transposed=transposed):
        return None
    return gnm.packed()


def _sp24_or_none(gnm, tokens):
    """The cached compressed transposed copy when the backward product of this many tokens runs on the structured-sparse
    tensor cores (16-bit weight inside the 2:4 structure), else None (nothing is built)."""
    return gnm.packed_sp24() if tokens >= ops.SP24_MIN_TOKENS else None


def _wants_expanded(gnm, x2d, tokens, layout=nat.NMG_ACT_TOKEN_MAJOR):
    """The opt-in of ``set_spmm_opt(kernel="sm100-expanded")`` applies: 16-bit weight, token-major activation whose rows TMA
    can read, and a batch large enough for the two-pass regime (fewer tokens stay on the compressed-weight kernel)."""
    return (gnm.nm_strides.get("kernel") == "sm100-expanded" and layout == nat.NMG_ACT_TOKEN_MAJOR and tokens >= ops.SP24_MIN_TOKENS
            and gnm.val.dtype != torch.float32 and x2d.stride(-1) == 1 and x2d.data_ptr() % 16 == 0 and x2d.stride(0) % 8 == 0
            and gnm.expanded() is not None)


def sparse_dense_mul_dispatch(weight, dense2d, bias, layout):
    """One C-ABI call; replaces the compile-or-load + ctypes call of the reference (sten_impls.py:44-140)."""
    gnm, M, K, n, m, g = _weight_geometry(weight)
    tokens = dense2d.shape[1] if layout == nat.NMG_ACT_K_MAJOR else dense2d.shape[0]
    if _wants_expanded(gnm, dense2d, tokens, layout):
        return ops.spmm_expanded(gnm.expanded(), M, K, dense2d, bias=bias)
    packed = _packed_or_none(gnm, (M, K, n, m, g), tokens, layout) if tokens else None
    return ops.spmm(gnm.val, gnm.idx, M, K, n, m, g, dense2d, bias=bias, layout=layout, packed=packed)


def _linear_fwd(ctx, inputs, output_sparsifiers):
    if len(inputs) == 3:
        x, weight, bias = inputs
    else:
        (x, weight), bias = inputs, None
    ctx.save_for_backward(x, weight, bias) if bias is not None else ctx.save_for_backward(x, weight)
    x2d = x.reshape(-1, x.shape[-1])
    y = sparse_dense_mul_dispatch(weight, x2d, bias, nat.NMG_ACT_TOKEN_MAJOR)
    return y.reshape(*x.shape[:-1], y.shape[-1])


_LIN_OUT = [(sten.KeepAll, torch.Tensor)]
sparse_torch_nn_functional_linear = sten.register_fwd_op_impl(
    operator=torch.nn.functional.linear, inp=(torch.Tensor, GroupedNMTensor, torch.Tensor), out=_LIN_OUT)(_linear_fwd)
sten.register_fwd_op_impl(operator=torch.nn.functional.linear, inp=(torch.Tensor, GroupedNMTensor), out=_LIN_OUT)(_linear_fwd)


def _linear_bwd(ctx, grad_outputs, input_sparsifiers):
    saved = ctx.saved_tensors
    x, weight = saved[0], saved[1]
    has_bias = len(saved) == 3
    [dy] = grad_outputs
    needs = tuple(ctx.needs_input_grad[1:]) + (False,) * 3
    gnm, M, K, n, m, g = _weight_geometry(weight)
    dy2d = dy.reshape(-1, M)
    dx = dw = db = None
    if needs[0]:
        sp24 = _sp24_or_none(gnm, dy2d.shape[0])
        dx = ops.spmm_t(gnm.val, gnm.idx, M, K, n, m, g, dy2d, sp24=sp24,
                        packed=None if sp24 is not None else _packed_or_none(gnm, (M, K, n, m, g), dy2d.shape[0], transposed=True)).reshape(x.shape)
    if needs[1]:
        # dense weight gradient (training of nmg weights is outside the inference hot path): plain GEMM
        dw = dy2d.t().mm(x.reshape(-1, K))
    if has_bias and needs[2]:
        db = dy2d.sum(dim=0)
    return (dx, dw, db) if has_bias else (dx, dw)


def _linear_bwd_weight_layout(ctx, grad_outputs, input_sparsifiers):
    """Same products as ``_linear_bwd``; dW leaves as a GroupedNMTensor in the weight's layout.  dY^T X runs on the tensor
    cores at the dense rate into a transient buffer (a sampled product on the FP32 pipes would be an order of magnitude
    slower on this hardware) and one gather pass keeps the layout's positions."""
    grads = list(_linear_bwd(ctx, grad_outputs, input_sparsifiers))
    if grads[1] is not None:
        weight = ctx.saved_tensors[1]
        masked = weight.wrapped_tensor.clone_layout(grads[1])
        grads[1] = sten.SparseTensorWrapper.wrapped_from_dense(masked, grads[1], None)
    return tuple(grads)


_DENSE_GRAD = (sten.KeepAll, torch.Tensor)
_LAYOUT_GRAD = (WeightLayoutSparsifier, GroupedNMTensor)
for _inp in ((torch.Tensor, GroupedNMTensor, torch.Tensor), (torch.Tensor, GroupedNMTensor)):
    sten.register_bwd_op_impl(operator=torch.nn.functional.linear, grad_out=(torch.Tensor,),
                              grad_inp=tuple(_DENSE_GRAD for _ in _inp), inp=_inp)(_linear_bwd)
    sten.register_bwd_op_impl(operator=torch.nn.functional.linear, grad_out=(torch.Tensor,),
                              grad_inp=tuple(_LAYOUT_GRAD if f is GroupedNMTensor else _DENSE_GRAD for f in _inp),
                              inp=_inp)(_linear_bwd_weight_layout)


def _mm_fwd(ctx, inputs, output_sparsifiers):
    weight, b = inputs
    ctx.save_for_backward(weight, b)
    if b.dim() != 2:
        raise sten.DispatchError("grouped n:m matmul expects a 2-D right operand")
    return sparse_dense_mul_dispatch(weight, b, None, nat.NMG_ACT_K_MAJOR)


def _mm_bwd(ctx, grad_outputs, input_sparsifiers):
    weight, b = ctx.saved_tensors
    [dc] = grad_outputs  # [M, N]
    needs = tuple(ctx.needs_input_grad[1:]) + (False,) * 2
    gnm, M, K, n, m, g = _weight_geometry(weight)
    dw = db = None
    if needs[0]:
        dw = dc.mm(b.t())
    if needs[1]:
        # dB = W^T dC : the transposed kernel computes (dC^T W)[N, K]; hand back its transpose
        dct = dc.t().contiguous()
        sp24 = _sp24_or_none(gnm, dct.shape[0])
        db = ops.spmm_t(gnm.val, gnm.idx, M, K, n, m, g, dct, sp24=sp24,
                        packed=None if sp24 is not None else _packed_or_none(gnm, (M, K, n, m, g), dct.shape[0], transposed=True)).t()
    return dw, db


for _op in (torch.mm, torch.matmul):
    sten.register_fwd_op_impl(operator=_op, inp=(GroupedNMTensor, torch.Tensor), out=_LIN_OUT)(_mm_fwd)
    sten.register_bwd_op_impl(operator=_op, grad_out=(torch.Tensor,), grad_inp=(_DENSE_GRAD, _DENSE_GRAD),
                              inp=(GroupedNMTensor, torch.Tensor))(_mm_bwd)
