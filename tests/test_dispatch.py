"""Host logic of the plugin boundary on CPU, with a toy format standing in for the CUDA-backed one
(the way the reference's own tests register private formats: tests/test_api.py, tests/test_dispatch.py)."""
import io
import warnings

import pytest
import torch

import sten_b200 as sten


class ToyTensor:
    def __init__(self, data):
        self.data = data

    def to_dense(self):
        return self.data.clone()


class ToySparsifier:
    pass


def _register_once():
    key = (ToySparsifier, torch.Tensor, ToyTensor)
    if key in sten.SPARSIFIER_IMPLEMENTATIONS:
        return

    @sten.register_sparsifier_implementation(sparsifier=ToySparsifier, inp=torch.Tensor, out=ToyTensor)
    def to_toy(sparsifier, tensor, grad_fmt=None):
        return sten.SparseTensorWrapper.wrapped_from_dense(ToyTensor(tensor.detach().clone()), tensor, grad_fmt)

    @sten.register_sparsifier_implementation(sparsifier=sten.SameFormatSparsifier, inp=torch.Tensor, out=ToyTensor)
    def to_toy_again(sparsifier, tensor, grad_fmt=None):
        return sten.SparseTensorWrapper.wrapped_from_dense(ToyTensor(tensor.detach().clone()), tensor, grad_fmt)


_register_once()
CALLS = []


@sten.register_fwd_op_impl(operator=torch.mm, inp=(ToyTensor, torch.Tensor), out=[(sten.KeepAll, torch.Tensor)])
def toy_mm(ctx, inputs, output_sparsifiers):
    a, b = inputs
    ctx.save_for_backward(a, b)
    CALLS.append("mm_fwd")
    return a.wrapped_tensor.data @ b


@sten.register_bwd_op_impl(operator=torch.mm, grad_out=(torch.Tensor,),
                           grad_inp=((sten.KeepAll, torch.Tensor), (sten.KeepAll, torch.Tensor)),
                           inp=(ToyTensor, torch.Tensor))
def toy_mm_bwd(ctx, grad_outputs, input_sparsifiers):
    a, b = ctx.saved_tensors
    [dc] = grad_outputs
    CALLS.append("mm_bwd")
    return dc @ b.t(), a.wrapped_tensor.data.t() @ dc


def _sparse_linear():
    torch.manual_seed(0)
    dense = torch.nn.Linear(8, 4)
    sb = sten.SparsityBuilder()
    sb.set_weight("weight", initial_sparsifier=ToySparsifier(), out_format=ToyTensor)
    return dense, sb.get_sparse_model(dense)


def test_builder_wraps_weight_and_keeps_original():
    dense, sparse = _sparse_linear()
    assert isinstance(sparse.weight, sten.SparseParameterWrapper)
    assert isinstance(sparse.weight.wrapped_tensor, ToyTensor)
    assert isinstance(dense.weight, torch.nn.Parameter) and not isinstance(dense.weight, sten.SparseTensorWrapper)
    assert sparse.weight.grad_fmt[3] is sten.DenseTensor
    assert len(sparse.weight.grad_fmt) == 4


def test_registered_mm_forward_backward_and_no_grad_shortcut():
    CALLS.clear()
    w = sten.SparseTensorWrapper.wrapped_from_dense(ToyTensor(torch.randn(4, 6)), torch.zeros(1, requires_grad=True))
    b = torch.randn(6, 3, requires_grad=True)
    c = torch.mm(w, b)
    assert torch.allclose(c, w.wrapped_tensor.data @ b)
    c.sum().backward()
    assert CALLS == ["mm_fwd", "mm_bwd"]
    assert torch.allclose(b.grad, w.wrapped_tensor.data.t() @ torch.ones(4, 3))
    assert isinstance(w.grad, sten.SparseTensorWrapper) and isinstance(w.grad.wrapped_tensor, sten.DenseTensor)
    with torch.no_grad():
        torch.mm(w, b)
    assert CALLS[-1] == "mm_fwd"


def test_missing_impl_falls_back_to_dense_with_warning_and_backward_works():
    dense, sparse = _sparse_linear()
    x = torch.randn(5, 8, requires_grad=True)
    with pytest.warns(sten.DispatchWarning):
        y = sparse(x)
    assert torch.allclose(y, dense(x))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        y.sum().backward()
    assert x.grad is not None and sparse.weight.grad is not None


def test_raise_mode_raises_dispatch_error():
    _, sparse = _sparse_linear()
    sten.set_dispatch_failure("raise")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with pytest.raises(sten.DispatchError):
            sparse(torch.randn(2, 8))
    with pytest.raises(ValueError):
        sten.set_dispatch_failure("explode")


def test_registry_keys_are_canonicalised():
    assert sten.canonicalize_list_of_tensor_formats((torch.Tensor, torch.Tensor)) is None
    assert sten.canonicalize_list_of_sparsifier_ten_fmt_pairs([(sten.KeepAll, torch.Tensor)]) is None
    assert sten.get_fwd_op_impl(torch.mm, (ToyTensor, torch.Tensor), [(sten.KeepAll, torch.Tensor)]) is toy_mm
    with pytest.raises(sten.DispatchError):
        sten.get_fwd_op_impl(torch.mm, (torch.Tensor, ToyTensor), None)
    with pytest.raises(Exception, match="second time"):
        sten.register_sparsifier_implementation(sparsifier=ToySparsifier, inp=torch.Tensor, out=ToyTensor)(lambda *a: None)


def test_inplace_update_resparsifies_into_same_format_and_optimizer_steps():
    dense, sparse = _sparse_linear()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with torch.no_grad():
            sparse.weight.mul_(2.0)
        assert isinstance(sparse.weight.wrapped_tensor, ToyTensor)
        assert torch.allclose(sparse.weight.wrapped_tensor.to_dense(), dense.weight * 2)
        x = torch.randn(3, 8)
        sparse(x).sum().backward()
        before = sparse.weight.wrapped_tensor.to_dense()
        torch.optim.SGD(sparse.parameters(), lr=0.5).step()
        assert not torch.equal(before, sparse.weight.wrapped_tensor.to_dense())


def test_pickle_round_trip_of_module_and_wrapper():
    dense, sparse = _sparse_linear()
    buf = io.BytesIO()
    torch.save(sparse, buf)
    buf.seek(0)
    again = torch.load(buf, weights_only=False)
    assert isinstance(again.weight, sten.SparseParameterWrapper)
    assert torch.equal(again.weight.wrapped_tensor.data, sparse.weight.wrapped_tensor.data)
    fn, args = sparse.weight.__reduce_ex__(2)
    assert fn is sten.dispatch.sparse_tensor_builder and args[0] is sten.SparseParameterWrapper and len(args) == 4


def test_clone_detach_and_grad_fmt_survive():
    _, sparse = _sparse_linear()
    w = sparse.weight
    d = w.detach()
    assert isinstance(d, sten.SparseTensorWrapper) and not d.requires_grad and d.wrapped_tensor is w.wrapped_tensor
    c = w.clone()
    assert c.wrapped_tensor is not w.wrapped_tensor and torch.equal(c.wrapped_tensor.data, w.wrapped_tensor.data)
    assert c.grad_fmt[1] is torch.Tensor


def test_sparsified_op_output_format():
    op = sten.sparsified_op(torch.add, [(sten.KeepAll(), torch.Tensor, ToySparsifier(), ToyTensor)],
                            [(sten.KeepAll(), torch.Tensor, sten.KeepAll(), torch.Tensor)])
    out = op(torch.ones(2, 2), torch.ones(2, 2))
    assert isinstance(out, sten.SparseTensorWrapper) and isinstance(out.wrapped_tensor, ToyTensor)
    assert torch.equal(out.wrapped_tensor.data, torch.full((2, 2), 2.0))
    assert out.grad_fmt[3] is sten.DenseTensor  # dense gradient of a sparse tensor is wrapped automatically


def test_plugin_registrations_exist_for_both_linear_arities_and_mm():
    G = sten.GroupedNMTensor
    lin = torch.nn.functional.linear
    out = [(sten.KeepAll, torch.Tensor)]
    assert sten.get_fwd_op_impl(lin, (torch.Tensor, G, torch.Tensor), out)
    assert sten.get_fwd_op_impl(lin, (torch.Tensor, G), out)
    assert sten.get_fwd_op_impl(torch.mm, (G, torch.Tensor), out)
    dense = (sten.KeepAll, torch.Tensor)
    assert sten.get_bwd_op_impl(lin, (torch.Tensor,), (dense, dense, dense), (torch.Tensor, G, torch.Tensor))
    assert sten.get_bwd_op_impl(torch.mm, (torch.Tensor,), (dense, dense), (G, torch.Tensor))
    assert (sten.GroupedNMSparsifier, torch.Tensor, G) in sten.SPARSIFIER_IMPLEMENTATIONS
    s = sten.GroupedNMSparsifier(2, 4, 16)
    assert (s.n, s.m, s.g) == (2, 4, 16)


def test_patch_rebinds_function_in_scope():
    import types
    mod = types.ModuleType("scope_mod")

    def old():
        return "old"

    mod.f = old
    mod.K = type("K", (), {"g": staticmethod(old)})
    sten.patch(old, lambda: "new", [mod])
    assert mod.f() == "new" and mod.K.g() == "new"


def test_module_to_moves_the_payload_without_densifying():
    """nn.Module.to() on a module with a sparse parameter: the dtype / device questions PyTorch asks on the way
    (is_floating_point, _has_compatible_shallow_copy_type) are answered from the wrapper, the payload's own .to() does
    the move, and to_dense() is never called."""
    import sten_b200 as sten
    from sten_b200 import dispatch

    class Payload:
        def __init__(self, t):
            self.t, self.densified = t, 0

        def to_dense(self):
            self.densified += 1
            return self.t

        def to(self, device=None, dtype=None, non_blocking=False, copy=False):
            assert isinstance(non_blocking, bool) and isinstance(copy, bool)
            return Payload(self.t.to(device=device, dtype=dtype))

        dtype = property(lambda self: self.t.dtype)
        device = property(lambda self: self.t.device)

    sten.set_dispatch_failure("raise")
    lin = torch.nn.Linear(4, 4)
    first = Payload(torch.randn(4, 4))
    lin.weight = dispatch.SparseParameterWrapper(dispatch.SparseTensorWrapper([first], True, dispatch._DEFAULT_GRAD_FMT()))
    lin = lin.to(torch.float64)
    assert isinstance(lin.weight, dispatch.SparseParameterWrapper)
    assert lin.weight.dtype == torch.float64 and lin.weight.wrapped_tensor.t.dtype == torch.float64
    assert first.densified == 0 and lin.weight.wrapped_tensor.densified == 0
