"""Dispatch runtime: the host of the plugin boundary.

This module re-creates, with its own implementation, the public surface of the reference runtime
(src/sten/sten.py) that the grouped n:m plugin and its users touch:

* ``SparseTensorWrapper`` / ``SparseParameterWrapper`` -- ``torch.Tensor`` subclasses that carry an arbitrary
  format object in ``.wrapped_tensor`` and a gradient-format 4-tuple in ``.grad_fmt`` (sten.py:91-270);
* the three registries and their decorators ``register_sparsifier_implementation`` (sten.py:1071-1104),
  ``register_fwd_op_impl`` (:1162-1195), ``register_bwd_op_impl`` (:1257-1298) with the same keys, the same
  callable signatures ``f(sparsifier, tensor, grad_fmt=None)``, ``f(ctx, inputs, output_sparsifiers)``,
  ``f(ctx, grad_outputs, input_sparsifiers)`` and the same key canonicalisation (all-dense -> ``None``);
* ``sparsified_op`` (:1875-1928), the dense fall-back with ``DispatchWarning`` / ``DispatchError`` and
  ``set_dispatch_failure`` (:54-76, :1586-1601, :1676-1693);
* ``SparsityBuilder`` (:720-1019) and pickling through ``sparse_tensor_builder`` (:178-189, :413-420).

Differences that are deliberate: when no participating tensor needs a gradient the registered forward
implementation is called directly instead of through ``autograd.Function`` (saves host time per call), and
``Tensor.to`` of a wrapper uses the format object's own ``to`` when it has one.
"""
import copy
import functools
import inspect
import types
import warnings

import torch
import torch.fx

# ------------------------------------------------------------------------------------------------ failure policy
DISPATCH_RAISE = "raise"
DISPATCH_WARN = "warn"
DISPATCH_FAILURE = DISPATCH_WARN


def set_dispatch_failure(action):
    """'warn': missing implementations fall back to dense with a DispatchWarning; 'raise': they raise."""
    global DISPATCH_FAILURE
    if action not in (DISPATCH_RAISE, DISPATCH_WARN):
        raise ValueError("Unknown action")
    DISPATCH_FAILURE = action


class DispatchWarning(Warning):
    pass


class DispatchError(Warning):  # a Warning subclass that is *raised*, as in the reference (sten.py:75)
    pass


# ------------------------------------------------------------------------------------------------ profiling switches
CUDA_PROFILING = [False]
profile_entries = {}


def set_cuda_profiling(value=True):
    if torch.cuda.is_available():
        CUDA_PROFILING[0] = value


def sync_cuda():
    if CUDA_PROFILING[0]:
        torch.cuda.synchronize()


def reset_profile():
    for v in profile_entries.values():
        v.clear()


# ------------------------------------------------------------------------------------------------ trivial formats
class DenseTensor:
    """Dense data behind the wrapper interface: lets a dense tensor have a gradient in a custom format."""

    def __init__(self, data):
        self.data = data

    def to_dense(self):
        return self.data


class KeepAll:
    """The sparsifier that keeps everything."""

    def __eq__(self, other):
        return type(other) is type(self)

    def __hash__(self):
        return hash(type(self))


class SameFormatSparsifier:
    """Re-sparsify a dense result into the format (and layout) of ``ref_sp_ten``; used after in-place ops."""

    def __init__(self, ref_sp_ten):
        self.ref_sp_ten = ref_sp_ten


_DEFAULT_GRAD_FMT = lambda: (KeepAll(), torch.Tensor, KeepAll(), DenseTensor)  # noqa: E731


# ------------------------------------------------------------------------------------------------ pytree helpers
class TensorIdx:
    """Placeholder for the i-th tensor of a flattened argument structure."""

    __slots__ = ("idx",)

    def __init__(self, idx):
        self.idx = idx

    def __eq__(self, other):
        return isinstance(other, TensorIdx) and self.idx == other.idx

    def __hash__(self):
        return hash(("TensorIdx", self.idx))


def _map_structure(fn, obj):
    if type(obj) in (list, tuple):
        return type(obj)(_map_structure(fn, o) for o in obj)
    if type(obj) is dict:
        return {k: _map_structure(fn, v) for k, v in obj.items()}
    return fn(obj)


def flatten_list_of_tensors_in_args(args):
    flat = []

    def visit(x):
        if isinstance(x, torch.Tensor):
            flat.append(x)
            return TensorIdx(len(flat) - 1)
        return x

    return _map_structure(visit, args), flat


def unflatten_list_of_tensors_in_args(args_with_stubs, flat_tensors):
    return _map_structure(lambda x: flat_tensors[x.idx] if isinstance(x, TensorIdx) else x, args_with_stubs)


def flattened_tensors(args):
    return flatten_list_of_tensors_in_args(args)[1]


def flattened_sparse_tensors(args):
    return [t for t in flattened_tensors(args) if isinstance(t, SparseTensorWrapper)]


def densify(args):
    return _map_structure(lambda x: x.wrapped_tensor.to_dense() if isinstance(x, SparseTensorWrapper) else x, args)


def torch_name(op):
    name = torch.overrides.resolve_name(op) if hasattr(torch.overrides, "resolve_name") else None
    if name:
        return name
    if hasattr(op, "__module__") and op.__module__:
        return f"{op.__module__}.{op.__name__}"
    if hasattr(op, "__objclass__"):
        return f"{op.__objclass__}.{op.__name__}"
    return getattr(op, "__name__", str(op))


def pretty_name(obj):
    if isinstance(obj, list):
        return "[" + ", ".join(pretty_name(o) for o in obj) + "]"
    if isinstance(obj, tuple):
        return "(" + ", ".join(pretty_name(o) for o in obj) + ")"
    if inspect.isclass(obj):
        return obj.__qualname__ if obj.__module__ in ("builtins", "__main__") else f"{obj.__module__}.{obj.__qualname__}"
    return str(obj)


# ------------------------------------------------------------------------------------------------ registries
SPARSIFIER_IMPLEMENTATIONS = {}
FWD_OP_IMPLS = {}
BWD_OP_IMPLS = {}


def canonicalize_list_of_tensor_formats(fmts):
    if fmts is None or all(f is torch.Tensor for f in fmts):
        return None
    return tuple(fmts)


def canonicalize_list_of_sparsifier_ten_fmt_pairs(pairs):
    if pairs is None or all(p is not None and p[0] is KeepAll and p[1] is torch.Tensor for p in pairs):
        return None
    return tuple(tuple(p) if p is not None else None for p in pairs)


def register_sparsifier_implementation(sparsifier, inp, out):
    """Decorator: ``f(sparsifier, tensor, grad_fmt=None) -> SparseTensorWrapper`` for (sparsifier class, input
    format class, output format class).  Registering the same key twice raises."""

    def decorator(func):
        key = (sparsifier, inp, out)
        if key in SPARSIFIER_IMPLEMENTATIONS:
            raise Exception("Trying to register sparsifier implementation second time! "
                            "Use unregister_sparsifier_implementation to remove existing implementation.")
        SPARSIFIER_IMPLEMENTATIONS[key] = func
        return func

    return decorator


def unregister_sparsifier_implementation(sparsifier, inp, out):
    del SPARSIFIER_IMPLEMENTATIONS[(sparsifier, inp, out)]


def get_sparsifier_implementation(sparsifier, inp, out):
    if (sparsifier, inp, out) == (type(None), None, None) or (sparsifier is KeepAll and inp is out):
        return lambda sp, ten, grad_fmt=None: ten
    if sparsifier in (KeepAll, SameFormatSparsifier) and inp is torch.Tensor and out is DenseTensor:
        return lambda sp, ten, grad_fmt=None: SparseTensorWrapper.wrapped_from_dense(
            DenseTensor(ten.clone().detach()), ten, grad_fmt)
    impl = SPARSIFIER_IMPLEMENTATIONS.get((sparsifier, inp, out))
    if impl is not None:
        return impl
    msg = ("Sparsifier implementation is not registered:\n"
           "@sten.register_sparsifier_implementation(\n"
           f"    sparsifier={pretty_name(sparsifier)}, inp={pretty_name(inp)}, out={pretty_name(out)}\n)\n"
           "def my_sparsifier_implementation(sparsifier, tensor, grad_fmt=None):\n    return sparsified_tensor_wrapper")
    if DISPATCH_FAILURE == DISPATCH_WARN and inp is not torch.Tensor:
        warnings.warn(f"{msg}\nUsing the implementation for dense input after densifying.", DispatchWarning)
        from_dense = get_sparsifier_implementation(sparsifier, torch.Tensor, out)
        return lambda sp, ten, grad_fmt=None: from_dense(sp, ten.wrapped_tensor.to_dense(), grad_fmt)
    raise DispatchError(msg)


def register_fwd_op_impl(operator, inp, out):
    """Decorator: ``f(ctx, inputs, output_sparsifiers)`` for (operator, input formats, [(sparsifier class, format)])."""
    key = (operator, canonicalize_list_of_tensor_formats(inp), canonicalize_list_of_sparsifier_ten_fmt_pairs(out))

    def decorator(func):
        FWD_OP_IMPLS[key] = func
        return func

    return decorator


def get_fwd_op_impl(operator, inp, out):
    inp = canonicalize_list_of_tensor_formats(inp)
    out = canonicalize_list_of_sparsifier_ten_fmt_pairs(out)
    impl = FWD_OP_IMPLS.get((operator, inp, out))
    if impl is None:
        raise DispatchError(
            "Sparse operator implementation is not registered (fwd):\n"
            "@sten.register_fwd_op_impl(\n"
            f"    operator={torch_name(operator)},\n    inp={pretty_name(inp)},\n    out={pretty_name(out)},\n)\n"
            "def my_operator(ctx, inputs, output_sparsifiers):\n    return outputs")
    return impl


def register_bwd_op_impl(operator, grad_out, grad_inp, inp):
    """Decorator: ``f(ctx, grad_outputs, input_sparsifiers)`` returning one gradient per forward tensor input."""
    key = (operator, canonicalize_list_of_tensor_formats(grad_out),
           canonicalize_list_of_sparsifier_ten_fmt_pairs(grad_inp), canonicalize_list_of_tensor_formats(inp))

    def decorator(func):
        BWD_OP_IMPLS[key] = func
        return func

    return decorator


def get_bwd_op_impl(operator, grad_out, grad_inp, inp):
    grad_out = canonicalize_list_of_tensor_formats(grad_out)
    grad_inp = canonicalize_list_of_sparsifier_ten_fmt_pairs(grad_inp)
    inp = canonicalize_list_of_tensor_formats(inp)
    impl = BWD_OP_IMPLS.get((operator, grad_out, grad_inp, inp))
    if impl is None:
        raise DispatchError(
            "Sparse operator implementation is not registered (bwd):\n"
            "@sten.register_bwd_op_impl(\n"
            f"    operator={torch_name(operator)},\n    grad_out={pretty_name(grad_out)},\n"
            f"    grad_inp={pretty_name(grad_inp)},\n    inp={pretty_name(inp)},\n)\n"
            "def my_operator(ctx, grad_outputs, input_sparsifiers):\n    return grad_inputs")
    return impl


def get_format(tensor):
    if isinstance(tensor, SparseTensorWrapper):
        return tensor.wrapped_tensor.__class__
    if isinstance(tensor, torch.Tensor):
        return torch.Tensor
    return None


def has_format(tensor, fmt):
    if not isinstance(tensor, SparseTensorWrapper):
        return (isinstance(tensor, torch.Tensor) and fmt is torch.Tensor) or fmt is None
    return tensor.wrapped_tensor.__class__ is fmt


def find_gradient_fmt(tensor):
    if isinstance(tensor, SparseTensorWrapper):
        return tensor.grad_fmt
    if isinstance(tensor, torch.Tensor):
        return (KeepAll(), torch.Tensor, KeepAll(), torch.Tensor)
    return (None, None, None, None)


def _is_dense_fmt(f):
    return f in (None, torch.Tensor, DenseTensor)


def check_dense_inputs(fmts):
    return fmts is None or all(_is_dense_fmt(f) for f in fmts)


def check_dense_outputs(pairs):
    if pairs is None:
        return True
    return all(p is None or (p[0] is KeepAll and _is_dense_fmt(p[1])) for p in pairs)


# ------------------------------------------------------------------------------------------------ wrappers
HANDLED_FUNCTIONS = {}


def implements(*torch_functions):
    def decorator(fn):
        for f in torch_functions:
            HANDLED_FUNCTIONS[f] = fn
        return fn

    return decorator


class SparseTensorWrapper(torch.Tensor):
    """A tensor whose payload is ``self.wrapped_tensor`` (any object with ``to_dense()``).

    The underlying storage is a one-element dummy of the payload's dtype on the payload's device, so autograd,
    ``nn.Module`` and optimizers can carry the object around; every torch function applied to it is routed
    through ``__torch_function__`` to the registries."""

    @staticmethod
    def wrapped_from_dense(wrapped, dense, grad_fmt=None):
        return SparseTensorWrapper([wrapped], dense.requires_grad, grad_fmt if grad_fmt is not None else _DEFAULT_GRAD_FMT())

    def __new__(cls, wrapped_tensor_container, requires_grad, grad_fmt, *, dummy_shape=None):
        payload = wrapped_tensor_container[0]
        assert not isinstance(payload, SparseTensorWrapper)
        meta = payload if hasattr(payload, "dtype") and hasattr(payload, "device") else payload.to_dense()
        dummy = torch.zeros([1], dtype=meta.dtype, device=meta.device)
        self = torch.Tensor._make_subclass(cls, dummy, requires_grad)
        self._wrapped_tensor_container = wrapped_tensor_container
        self.grad_fmt = grad_fmt
        self.update_grad_fix_hook()
        return self

    # autograd hands back gradients as plain views of the subclass; keep the wrapper in .grad
    def grad_fix_hook(self, grad):
        self.grad = grad

    def update_grad_fix_hook(self):
        has = hasattr(self, "grad_fix_hook_handle")
        if self.requires_grad and not has:
            self.grad_fix_hook_handle = self.register_hook(self.grad_fix_hook)
        elif not self.requires_grad and has:
            self.grad_fix_hook_handle.remove()
            del self.grad_fix_hook_handle

    @property
    def wrapped_tensor(self):
        return self._wrapped_tensor_container[0]

    @wrapped_tensor.setter
    def wrapped_tensor(self, value):
        self._wrapped_tensor_container[0] = value

    def init_from_other(self, other, replace_attributes=True):
        assert isinstance(other, SparseTensorWrapper)
        _retarget_dummy(self, other.device, other.dtype)
        self.wrapped_tensor = other.wrapped_tensor
        if replace_attributes:
            self.requires_grad = other.requires_grad
            self.grad_fmt = other.grad_fmt

    def __copy__(self):
        return sparse_tensor_builder(type(self), self._wrapped_tensor_container, self.requires_grad, self.grad_fmt)

    def __deepcopy__(self, memo):
        if id(self) in memo:
            return memo[id(self)]
        result = sparse_tensor_builder(type(self), copy.deepcopy(self._wrapped_tensor_container, memo),
                                       bool(self.requires_grad), copy.deepcopy(self.grad_fmt, memo))
        if self.grad is not None:
            result.grad = copy.deepcopy(self.grad, memo)
        memo[id(self)] = result
        return result

    def __reduce_ex__(self, proto):
        return (sparse_tensor_builder, (type(self), self._wrapped_tensor_container, self.requires_grad, self.grad_fmt))

    def __repr__(self):
        return f"SparseTensorWrapper:\n{self.wrapped_tensor}"

    def __mul__(self, rhs):
        return torch.mul(self, rhs)

    def __rmul__(self, lhs):
        return torch.mul(lhs, self)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        handler = HANDLED_FUNCTIONS.get(func)
        if handler is not None:
            return handler(super().__torch_function__, func, types, *args, **kwargs)
        return sparse_fallback(super().__torch_function__, func, types, *args, **kwargs)


class SparseParameterWrapper(SparseTensorWrapper, torch.nn.parameter.Parameter):
    @staticmethod
    def wrapped_from_dense(wrapped_tensor, dense_tensor, grad_fmt=None):
        raise Exception("Do not use this, instead call wrapped_from_dense of SparseTensorWrapper and then wrap")

    def __new__(cls, sparse_tensor_wrapper):
        assert isinstance(sparse_tensor_wrapper, SparseTensorWrapper)
        return super().__new__(cls, wrapped_tensor_container=sparse_tensor_wrapper._wrapped_tensor_container,
                               requires_grad=sparse_tensor_wrapper.requires_grad,
                               grad_fmt=sparse_tensor_wrapper.grad_fmt)

    def __repr__(self):
        return "SparseParameterWrapper containing:\n" + super().__repr__()

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        base = tuple(SparseTensorWrapper if t is SparseParameterWrapper else t for t in types)
        return SparseTensorWrapper.__torch_function__(func, base, args, kwargs or {})


def sparse_tensor_builder(wrapper_type, wrapped_tensor_container, requires_grad, grad_fmt):
    """Unpickling / copying constructor; its module path and argument order are part of the pickle format."""
    assert issubclass(wrapper_type, SparseTensorWrapper)
    result = SparseTensorWrapper(wrapped_tensor_container, requires_grad, grad_fmt)
    if wrapper_type is SparseParameterWrapper:
        result = SparseParameterWrapper(result)
    return result


def _as_plain(tensor):
    class _Plain:
        def __enter__(self_inner):
            self_inner.cls = tensor.__class__
            tensor.__class__ = torch.Tensor
            return tensor

        def __exit__(self_inner, *exc):
            tensor.__class__ = self_inner.cls

    return _Plain()


def get_dummy_shape(tensor):
    with _as_plain(tensor) as t:
        return t.shape


def _retarget_dummy(tensor, device, dtype):
    with _as_plain(tensor) as t:
        t.data = t.data.to(device=device, dtype=dtype)


def change_wrapper_metadata(tensor, device, dtype):
    _retarget_dummy(tensor, device, dtype)


# ---- functions answered by the base class on the dummy storage
@implements(
    torch.Tensor.register_hook,
    torch.Tensor.requires_grad.__get__,
    torch.Tensor._backward_hooks.__set__,
    torch.Tensor.grad.__set__,
    torch.Tensor.grad.__get__,
    torch.Tensor.is_leaf.__get__,
    torch.Tensor.grad_fn.__get__,
    torch.Tensor.__hash__,
    torch.Tensor.is_sparse.__get__,
    torch.Tensor.backward,
    # dtype / device questions are answered by the one-element dummy, which carries the payload's dtype and device: no
    # reason to densify a weight (what the generic fallback would do) because nn.Module.to() asks whether it is floating point
    torch.Tensor.is_floating_point,
    torch.Tensor.is_complex,
    torch.Tensor.is_cuda.__get__,
)
def _base_impl(base_impl, func, types, *args, **kwargs):
    return base_impl(func, types, args, kwargs)


@implements(torch.Tensor.requires_grad_, torch.Tensor.requires_grad.__set__)
def _requires_grad_(base_impl, func, types, self, requires_grad=True):
    res = base_impl(func, types, (self, requires_grad))
    self.update_grad_fix_hook()
    return res


@implements(torch.Tensor.data.__get__, torch.Tensor.detach)
def _shallow_detached(base_impl, func, types, *args, **kwargs):
    [inp] = flattened_tensors(args) + flattened_tensors(kwargs)
    return copy.copy(inp).requires_grad_(False)


@implements(torch.Tensor.clone, torch.clone)
def _clone(base_impl, func, types, *args, **kwargs):
    [inp] = flattened_tensors(args)
    return copy.deepcopy(inp)


@implements(torch.Tensor.data.__set__)
def _data_set(base_impl, func, types, lhs, rhs):
    if isinstance(lhs, SparseTensorWrapper) and isinstance(rhs, SparseTensorWrapper):
        lhs.wrapped_tensor = rhs.wrapped_tensor
        _retarget_dummy(lhs, rhs.device, rhs.dtype)
    else:
        make_sparse_catcher(torch.Tensor.data.__set__, handle_inplace_modifications=True)(lhs, rhs)


@implements(torch._has_compatible_shallow_copy_type)
def _compatible_shallow_copy(base_impl, func, types, a, b):
    """nn.Module._apply asks this before ``param.data = fn(param)``: two sparse wrappers are interchangeable (the data
    setter swaps the payload), a wrapper and a plain tensor are not.  Answered here without densifying either side."""
    return isinstance(a, SparseTensorWrapper) and isinstance(b, SparseTensorWrapper)


@implements(torch.Tensor.to)
def _to(base_impl, func, types, *args, **kwargs):
    self = args[0]
    rest = list(args[1:])
    device, dtype = kwargs.get("device"), kwargs.get("dtype")
    if rest and isinstance(rest[0], torch.dtype):
        dtype = rest.pop(0)
    elif rest and isinstance(rest[0], torch.Tensor):
        other = rest.pop(0)
        device, dtype = other.device, other.dtype
    elif rest:
        device = rest.pop(0)
        if rest and isinstance(rest[0], torch.dtype):
            dtype = rest.pop(0)
    # nn.Module.to() passes non_blocking positionally and may pass None; Tensor.to() itself only takes booleans
    non_blocking = bool(rest.pop(0) if rest else kwargs.get("non_blocking", False))
    do_copy = bool(rest.pop(0) if rest else kwargs.get("copy", False))
    device = torch.device(device) if device is not None else self.device
    if device.type == "cuda" and device.index is None and self.device.type == "cuda":
        device = torch.device("cuda", torch.cuda.current_device())
    dtype = dtype if dtype is not None else self.dtype
    if device == self.device and dtype == self.dtype and not do_copy:
        return self
    payload = self.wrapped_tensor
    if hasattr(payload, "to") and not isinstance(payload, DenseTensor):
        moved = payload.to(device=device, dtype=dtype, non_blocking=non_blocking, copy=do_copy)
        return sparse_tensor_builder(SparseTensorWrapper, [moved], self.requires_grad, self.grad_fmt)
    fmt = payload.__class__
    return sparse_fallback_with_backprop(
        func, args=[self], kwargs={"device": device, "dtype": dtype, "non_blocking": non_blocking, "copy": do_copy},
        out_fmt=[(SameFormatSparsifier(self), fmt, KeepAll(), fmt)], grad_out_fmt=[self.grad_fmt])


# ------------------------------------------------------------------------------------------------ op semantics
OP_INPLACE_SEMANTICS_OVERRIDES = {}


def is_inplace_op(op):
    if op in OP_INPLACE_SEMANTICS_OVERRIDES:
        return OP_INPLACE_SEMANTICS_OVERRIDES[op]
    name = op.__name__
    if name == "__get__":
        return False
    if name == "__set__":
        return True
    return name.startswith("_") or name.endswith("_")


def _is_attribute(op):
    return op.__name__ in ("__get__", "__set__")


def sparse_fallback(base_impl, func, types, *args, **kwargs):
    inplace = is_inplace_op(func)
    if _is_attribute(func):
        if inplace:
            raise NotImplementedError("Attribute assignment is not supported")
        name = func.__self__.__name__
        self = args[0]
        if hasattr(self.wrapped_tensor, name):
            return getattr(self.wrapped_tensor, name)
        return make_sparse_catcher(func, handle_inplace_modifications=False)(*args, **kwargs)
    if isinstance(func, types_MethodDescriptor):
        self = args[0]
        if isinstance(self, SparseTensorWrapper) and hasattr(type(self.wrapped_tensor), func.__name__):
            return getattr(type(self.wrapped_tensor), func.__name__)(self.wrapped_tensor, *args[1:], **kwargs)
        if inplace:
            return make_sparse_catcher(func, handle_inplace_modifications=isinstance(self, SparseTensorWrapper))(*args, **kwargs)
        return sparse_fallback_with_backprop(func, args, kwargs)
    if inplace:
        return make_sparse_catcher(func, handle_inplace_modifications=True)(*args, **kwargs)
    return sparse_fallback_with_backprop(func, args, kwargs)


types_MethodDescriptor = types.MethodDescriptorType


def sparse_fallback_with_backprop(func, args, kwargs, *, out_fmt=None, grad_out_fmt=None):
    """Run ``func`` through a (cached) SparseOp attached to the participating sparse tensors."""
    for a in args:  # common case: the sparse operand is a top-level positional argument with a cached op
        if isinstance(a, SparseTensorWrapper):
            cached = getattr(a, "sparsified_ops", None)
            if cached is not None:
                op = cached.get(func)
                if op is not None:
                    return op(*args, **kwargs)
    sparse_args = flattened_sparse_tensors(args) + flattened_sparse_tensors(kwargs)
    op = None
    for t in sparse_args:
        op = getattr(t, "sparsified_ops", {}).get(func)
        if op is not None:
            break
    if op is None:
        op = sparsified_op(func, out_fmt, grad_out_fmt)
        for t in sparse_args:
            if not hasattr(t, "sparsified_ops"):
                t.sparsified_ops = {}
            t.sparsified_ops[func] = op
    return op(*args, **kwargs)


# ------------------------------------------------------------------------------------------------ signature binding
PATCHED_OVERRIDES = {
    torch.Tensor.to: lambda self, device=None, dtype=None, non_blocking=False, copy=False, *, memory_format=torch.preserve_format: -1,
}


@functools.lru_cache(maxsize=None)
def _signature_of(op):
    stub = PATCHED_OVERRIDES.get(op)
    if stub is None:
        stub = _testing_overrides().get(op)
    if stub is None:
        return None
    stubs = stub if isinstance(stub, tuple) else (stub,)
    return tuple(inspect.signature(s) for s in stubs)


@functools.lru_cache(maxsize=1)
def _testing_overrides():
    return torch.overrides.get_testing_overrides()


def bind_func_signature(op, args, kwargs):
    """Bind the call to the operator's declared signature so tensor inputs are ordered by parameter position."""
    sigs = _signature_of(op)
    if sigs is None:
        return None, None
    errors = []
    for sig in sigs:
        try:
            bound = sig.bind(*args, **kwargs)
            bound.apply_defaults()
            return bound, sig
        except TypeError as e:
            errors.append(e)
    raise KeyError(f"Failed to bind any of signatures to the args. {errors}")


# ------------------------------------------------------------------------------------------------ operator dispatch
class _NoGradCtx:
    """Stand-in for the autograd context when nothing needs a gradient."""

    needs_input_grad = ()

    def __init__(self, disp_state):
        self.disp_state = disp_state
        self.saved_tensors = ()

    def save_for_backward(self, *tensors):
        pass

    def mark_non_differentiable(self, *tensors):
        pass


def _transpose4(fmts, count):
    if fmts is None:
        return [None] * 4
    return tuple(zip(*fmts))


def _sparsifier_classes(sparsifiers, formats):
    if sparsifiers is None and formats is None:
        return None
    return tuple((s.__class__, f) if s is not None else None for s, f in zip(sparsifiers, formats))


def _exact_formats(fmts, tensors):
    return tuple(torch.Tensor for _ in tensors) if fmts is None else fmts


def _exact_sparsifiers(sps, tensors):
    return tuple(KeepAll() for _ in tensors) if sps is None else sps


def _check_formats(what, tensors, fmts):
    fmts = _exact_formats(fmts, tensors)
    if not all(has_format(t, f) for t, f in zip(tensors, fmts)):
        raise KeyError(f"Operator implementation {what} returned outputs in incorrect formats. "
                       f"Expected: {fmts}. Returned: {tuple(t.__class__ for t in tensors)}.")


def _fallback_fwd(out_fmt1):
    def impl(ctx, flat_inputs, output_sparsifiers):
        st = ctx.disp_state
        dense_inputs = []
        for t in flat_inputs:
            d = (t.wrapped_tensor.to_dense() if isinstance(t, SparseTensorWrapper) else t).detach()
            dense_inputs.append(d.requires_grad_(d.is_floating_point() or d.is_complex()))
        dense_inputs = tuple(dense_inputs)
        # impl inputs are ordered by the operator's signature; the call itself is replayed as it was written
        args, kwargs = unflatten_list_of_tensors_in_args(st["call_stubs"], [dense_inputs[i] for i in st["call_order"]])
        with torch.enable_grad():
            outputs = st["orig_op"](*args, **kwargs)
        out_stubs, flat_out = flatten_list_of_tensors_in_args(outputs)
        st["num_fwd_input_tensors"] = len(dense_inputs)
        ctx.save_for_backward(*dense_inputs, *flat_out)
        fmts = _exact_formats(out_fmt1, flat_out)
        sps = _exact_sparsifiers(output_sparsifiers, flat_out)
        impls = [get_sparsifier_implementation(s.__class__, torch.Tensor, f) for f, s in zip(fmts, sps)]
        return unflatten_list_of_tensors_in_args(out_stubs, [i(s, o.detach()) for i, s, o in zip(impls, sps, flat_out)])

    return impl


def _fallback_bwd(grad_inp_fmts):
    def impl(ctx, grad_outputs, input_sparsifiers):
        st = ctx.disp_state
        k = st["num_fwd_input_tensors"]
        inputs, outputs = ctx.saved_tensors[:k], ctx.saved_tensors[k:]
        pairs = [(o, g) for o, g in zip(outputs, densify(grad_outputs)) if o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], grad_tensors=[g for _, g in pairs])
        res = []
        for fmt, sp, inp in zip(grad_inp_fmts, input_sparsifiers, inputs):
            if inp.grad is None:
                res.append(None)
            else:
                res.append(get_sparsifier_implementation(sp.__class__, torch.Tensor, fmt)(sp, inp.grad))
        return tuple(res)

    return impl


def _failing_bwd(exc):
    def impl(ctx, grad_outputs, input_sparsifiers):
        raise DispatchError(exc)

    return impl


def _resolve_forward(st, flat_inputs):
    """Fill the per-op dispatch state on first use (formats are assumed stable for a given SparseOp)."""
    st["dummy_input_shapes"] = [get_dummy_shape(x) if isinstance(x, SparseTensorWrapper) else None for x in flat_inputs]
    st["inp_fmt"] = tuple(get_format(a) for a in flat_inputs)
    st["grad_inp_fmt"] = tuple(find_gradient_fmt(a) for a in flat_inputs)
    sp1, fmt1, sp2, fmt2 = _transpose4(st["out_fmt"], 4)
    st["out_fmt4"] = (sp1, fmt1, sp2, fmt2)
    st["op_out_fmt"] = _sparsifier_classes(sp1, fmt1)
    st["fwd_impl_fallback"] = False
    try:
        st["op_impl_fwd"] = get_fwd_op_impl(st["orig_op"], st["inp_fmt"], st["op_out_fmt"])
    except DispatchError as e:
        if not (check_dense_inputs(st["inp_fmt"]) and check_dense_outputs(st["op_out_fmt"])):
            warnings.warn(f"{e}\nFallback to dense implementation.", DispatchWarning)
            if DISPATCH_FAILURE == DISPATCH_RAISE:
                raise e
        st["fwd_impl_fallback"] = True
        st["op_impl_fwd"] = _fallback_fwd(fmt1)


def _run_forward(ctx, st, flat_inputs):
    first = "fwd_sp_impls" not in st
    if first:
        _resolve_forward(st, flat_inputs)
    sp1, fmt1, sp2, fmt2 = st["out_fmt4"]
    tmp = st["op_impl_fwd"](ctx, flat_inputs, sp1)
    out_stubs, flat_out = flatten_list_of_tensors_in_args(tmp)
    if first:
        _check_formats(f"{st['orig_op']} (fwd)", flat_out, fmt1)
        assert st["out_fmt"] is None or len(flat_out) == len(st["out_fmt"])
        f1, s2, f2 = _exact_formats(fmt1, flat_out), _exact_sparsifiers(sp2, flat_out), _exact_formats(fmt2, flat_out)
        st["fwd_out_fmt_sp_fmt"] = (f1, s2, f2)
        st["fwd_sp_impls"] = tuple(get_sparsifier_implementation(s.__class__, a, b) for a, s, b in zip(f1, s2, f2))
    _, s2, _ = st["fwd_out_fmt_sp_fmt"]
    outs = tuple(impl(s, t) for impl, t, s in zip(st["fwd_sp_impls"], flat_out, s2))
    return unflatten_list_of_tensors_in_args(out_stubs, outs)


class SparseOperatorDispatcher(torch.autograd.Function):
    @staticmethod
    def forward(ctx, disp_state, *flat_inputs):
        ctx.disp_state = disp_state
        return _run_forward(ctx, disp_state, flat_inputs)

    @staticmethod
    def backward(ctx, *grad_outputs):
        st = ctx.disp_state
        first = "bwd_sparsifier_impls" not in st
        if first:
            actual = tuple(get_format(a) for a in grad_outputs)
            _, _, _, gout_fmt2 = _transpose4(st["grad_out_fmt"], 4)
            if canonicalize_list_of_tensor_formats(gout_fmt2) != canonicalize_list_of_tensor_formats(actual):
                raise ValueError("Backward implementation received output gradients of incorrect format. "
                                 f"Expected: {st['grad_out_fmt']}. Actual: {actual}.")
            st["gout_fmt2"] = gout_fmt2
        gout_fmt2 = st["gout_fmt2"]
        ginp_sp1, ginp_fmt1, ginp_sp2, ginp_fmt2 = zip(*st["grad_inp_fmt"])
        if first:
            op_ginp = _sparsifier_classes(ginp_sp1, ginp_fmt1)
            try:
                impl = get_bwd_op_impl(st["orig_op"], gout_fmt2, op_ginp, st["inp_fmt"])
            except DispatchError as e:
                dense = check_dense_inputs(gout_fmt2) and check_dense_outputs(op_ginp) and check_dense_inputs(st["inp_fmt"])
                if dense or st["fwd_impl_fallback"]:
                    if not dense and DISPATCH_FAILURE == DISPATCH_RAISE:
                        raise e
                    impl = _fallback_bwd(ginp_fmt1)
                elif DISPATCH_FAILURE == DISPATCH_RAISE:
                    raise e
                else:
                    impl = _failing_bwd(e)
            st["op_impl_bwd"] = impl
        tmp = st["op_impl_bwd"](ctx, grad_outputs, ginp_sp1)
        tmp = tmp if isinstance(tmp, (tuple, list)) else (tmp,)
        if first:
            st["bwd_sparsifier_impls"] = tuple(
                get_sparsifier_implementation(s.__class__, a, b) for a, s, b in zip(ginp_fmt1, ginp_sp2, ginp_fmt2))
        grads = []
        for impl, g, s, shape in zip(st["bwd_sparsifier_impls"], tmp, ginp_sp2, st["dummy_input_shapes"]):
            if g is None:
                grads.append(None)
                continue
            g = impl(s, g)
            if isinstance(g, SparseTensorWrapper):  # gradient wrapper must look like the input's dummy
                g = SparseTensorWrapper(g._wrapped_tensor_container, g.requires_grad, g.grad_fmt, dummy_shape=shape)
            grads.append(g)
        return (None, *grads)


class SparseOp:
    def __init__(self, orig_op, out_fmt, grad_out_fmt):
        self.orig_op, self.out_fmt, self.grad_out_fmt = orig_op, out_fmt, grad_out_fmt
        self.clear_disp_state()

    def clear_disp_state(self):
        self.disp_state = {"orig_op": self.orig_op, "out_fmt": self.out_fmt, "grad_out_fmt": self.grad_out_fmt}

    def _run_fast(self, args):
        """Repeat of a call this op has already resolved: positional tensors only, same formats, nothing needs a
        gradient, a registered (not fallback) implementation and one dense output.  Skips flattening and signature
        binding, which dominate the host time of a sparse ``F.linear`` in inference."""
        st = self.disp_state
        fast = st.get("fast")
        if fast is None or len(args) != len(fast):
            return None
        for a, fmt in zip(args, fast):
            if not isinstance(a, torch.Tensor) or get_format(a) != fmt:
                return None
        if torch.is_grad_enabled() and any(a.requires_grad for a in args):
            return None
        tmp = st["op_impl_fwd"](_NoGradCtx(st), args, st["out_fmt4"][0])
        if type(tmp) is not torch.Tensor:
            return None if tmp is None else self._finish_slow_output(tmp)
        return st["fwd_sp_impls"][0](st["fwd_out_fmt_sp_fmt"][1][0], tmp)

    def _finish_slow_output(self, tmp):
        # an implementation that changed its mind about the output type: run the generic post-processing
        st = self.disp_state
        out_stubs, flat_out = flatten_list_of_tensors_in_args(tmp)
        _, s2, _ = st["fwd_out_fmt_sp_fmt"]
        outs = tuple(impl(s, t) for impl, t, s in zip(st["fwd_sp_impls"], flat_out, s2))
        return unflatten_list_of_tensors_in_args(out_stubs, outs)

    def run(self, *args, **kwargs):
        if not kwargs and "fast" in self.disp_state:
            out = self._run_fast(args)
            if out is not None:
                return out
        call_stubs, flat_call = flatten_list_of_tensors_in_args((tuple(args), dict(kwargs)))
        bound, _ = bind_func_signature(self.orig_op, args, kwargs)
        flat, order = flat_call, list(range(len(flat_call)))
        if bound is not None:
            flat_bound = flattened_tensors((tuple(bound.args), dict(bound.kwargs)))
            pos = {id(t): i for i, t in enumerate(flat_bound)}
            if len(flat_bound) == len(flat_call) and all(id(t) in pos for t in flat_call):
                flat, order = flat_bound, [pos[id(t)] for t in flat_call]
        st = self.disp_state
        signature = (call_stubs, tuple(get_format(t) for t in flat))
        if st.get("call_signature") != signature:
            self.clear_disp_state()
            st = self.disp_state
            st["call_signature"] = signature
        st["call_stubs"] = call_stubs
        st["call_order"] = order
        st["bound_args"] = bound

        need_grad = torch.is_grad_enabled() and any(t.requires_grad for t in flat)
        if need_grad:
            outputs = SparseOperatorDispatcher.apply(st, *flat)
        else:
            outputs = _run_forward(_NoGradCtx(st), st, tuple(flat))
        if (not need_grad and not kwargs and type(outputs) is torch.Tensor and not st.get("fwd_impl_fallback")
                and len(flat) == len(args) and all(a is b for a, b in zip(flat, args)) and len(st.get("fwd_sp_impls", ())) == 1):
            st["fast"] = tuple(get_format(t) for t in flat)  # next identical call takes _run_fast
        out_tuple = outputs if isinstance(outputs, (tuple, list)) else (outputs,)
        grad_fmts = _exact_formats(st["grad_out_fmt"], out_tuple)
        for o, gf in zip(out_tuple, grad_fmts):
            if isinstance(o, SparseTensorWrapper):
                o.grad_fmt = gf
        return outputs

    def __call__(self, *args, **kwargs):
        sync_cuda()
        out = self.run(*args, **kwargs)
        sync_cuda()
        return out


def sparsified_op(orig_op, out_fmt, grad_out_fmt):
    """Operator fused with sparsification of its outputs (reference sten.py:1875-1928).

    ``out_fmt`` / ``grad_out_fmt``: one 4-tuple (inline sparsifier, temporary format, external sparsifier, final
    format) per tensor output / per output gradient, or ``None`` for all-dense."""
    if out_fmt is not None or grad_out_fmt is not None:
        dense4 = lambda: [KeepAll(), torch.Tensor, KeepAll(), torch.Tensor]  # noqa: E731
        out_fmt = [list(x) for x in out_fmt] if out_fmt is not None else [dense4() for _ in grad_out_fmt]
        grad_out_fmt = [list(x) for x in grad_out_fmt] if grad_out_fmt is not None else [dense4() for _ in out_fmt]
        for o, g in zip(out_fmt, grad_out_fmt):  # a sparse tensor needs a wrapper on the gradient side too
            if (o[3] is torch.Tensor) != (g[3] is torch.Tensor):
                if o[3] is torch.Tensor:
                    o[3] = DenseTensor
                if g[3] is torch.Tensor:
                    g[3] = DenseTensor
    op = SparseOp(orig_op, out_fmt, grad_out_fmt)

    def wrapper(*args, **kwargs):
        return op(*args, **kwargs)

    wrapper.sparse_op = op
    return wrapper


@functools.lru_cache(maxsize=None)
def make_sparse_catcher(orig_fn, handle_inplace_modifications=True):
    """Run a function that has no sparse implementation on densified arguments; when it modified a sparse
    argument in place, re-sparsify the result into the argument's own format (``SameFormatSparsifier``)."""

    def sparse_catcher(*args, **kwargs):
        stubs, flat = flatten_list_of_tensors_in_args((args, kwargs))
        if not any(isinstance(t, SparseTensorWrapper) for t in flat):
            return orig_fn(*args, **kwargs)
        if any(isinstance(t, SparseTensorWrapper) and not isinstance(t.wrapped_tensor, DenseTensor) for t in flat):
            warnings.warn(f"Catching {torch_name(orig_fn)} called with the sparse arguments!", DispatchWarning)
        dense = densify(flat)
        before = [d.clone() if handle_inplace_modifications and isinstance(o, SparseTensorWrapper) else None
                  for o, d in zip(flat, dense)]
        d_args, d_kwargs = unflatten_list_of_tensors_in_args(stubs, dense)
        d_out = orig_fn(*d_args, **d_kwargs)
        if handle_inplace_modifications:
            for old, orig, now in zip(before, flat, dense):
                if old is None:
                    continue
                if old.dtype == now.dtype and old.device == now.device and old.shape == now.shape and torch.equal(old, now):
                    continue
                impl = get_sparsifier_implementation(SameFormatSparsifier, torch.Tensor, orig.wrapped_tensor.__class__)
                orig.init_from_other(impl(SameFormatSparsifier(orig), now), replace_attributes=False)
        out_stubs, flat_out = flatten_list_of_tensors_in_args(d_out)
        if not flat_out:
            return d_out
        mapped = []
        for o in flat_out:
            hit = [orig for orig, d in zip(flat, dense) if o is d]
            mapped.append(hit[-1] if hit else o)
        return unflatten_list_of_tensors_in_args(out_stubs, mapped)

    return sparse_catcher


# ------------------------------------------------------------------------------------------------ model surgery
def find_direct_container(module, weight_path):
    *parents, leaf = weight_path.split(".")
    for p in parents:
        module = getattr(module, p)
    return module, leaf


class SparsityBuilder:
    """Declare which weights / intermediate tensors (and their gradients) become sparse, then build the model.

    Same methods and defaults as the reference class (sten.py:720-1019)."""

    def __init__(self):
        self.initial_weight_sparsifiers = {}
        self.weights = {}
        self.grad_weights = {}
        self.interms = {}
        self.grad_interms = {}

    def set_weight(self, name, initial_sparsifier=KeepAll(), inline_sparsifier=KeepAll(), tmp_format=torch.Tensor,
                   external_sparsifier=KeepAll(), out_format=DenseTensor):
        self.weights[name] = (inline_sparsifier, tmp_format, external_sparsifier, out_format)
        self.initial_weight_sparsifiers[name] = initial_sparsifier

    def set_weight_grad(self, name, inline_sparsifier=KeepAll(), tmp_format=torch.Tensor,
                        external_sparsifier=KeepAll(), out_format=DenseTensor):
        self.grad_weights[name] = (inline_sparsifier, tmp_format, external_sparsifier, out_format)

    def set_interm(self, name, inline_sparsifier=KeepAll(), tmp_format=torch.Tensor, external_sparsifier=KeepAll(),
                   out_format=DenseTensor):
        self.interms[name] = (inline_sparsifier, tmp_format, external_sparsifier, out_format)

    def set_interm_grad(self, name, inline_sparsifier=KeepAll(), tmp_format=torch.Tensor,
                        external_sparsifier=KeepAll(), out_format=DenseTensor):
        self.grad_interms[name] = (inline_sparsifier, tmp_format, external_sparsifier, out_format)

    def fill_remaining(self):
        for name in set(self.weights) - set(self.grad_weights):
            self.set_weight_grad(name)
        for name in set(self.grad_weights) - set(self.weights):
            self.set_weight(name, KeepAll(), KeepAll(), torch.Tensor, KeepAll(), DenseTensor)
        for name in set(self.grad_interms) - set(self.interms):
            self.set_interm(name)
        for name in set(self.interms) - set(self.grad_interms):
            self.set_interm_grad(name)

    def sparsify_model_inplace(self, module):
        self.fill_remaining()
        with torch.no_grad():
            traced = {}
            for name, fmt in self.interms.items():
                path, _, node_name = name.rpartition(".")
                if path not in traced:
                    sub = module
                    for tok in filter(None, path.split(".")):
                        sub = getattr(sub, tok)
                    traced[path] = torch.fx.symbolic_trace(sub)
                [node] = [n for n in traced[path].graph.nodes if n.name == node_name]
                node.target = sparsified_op(node.target, [fmt], [self.grad_interms[name]])
            for path, gm in sorted(traced.items(), key=lambda kv: len([t for t in kv[0].split(".") if t])):
                gm.recompile()
                if path == "":
                    module = gm
                else:
                    parent, leaf = find_direct_container(module, path)
                    if not hasattr(parent, leaf):
                        raise KeyError(f"Can't find module under {path} path")
                    setattr(parent, leaf, gm)
            for name, (sp1, fmt1, sp2, fmt2) in self.weights.items():
                parent, leaf = find_direct_container(module, name)
                original = getattr(parent, leaf)
                initial = self.initial_weight_sparsifiers[name]
                impl = get_sparsifier_implementation(initial.__class__, torch.Tensor, fmt2)
                sparse = impl(initial, original, self.grad_weights[name])
                setattr(parent, leaf, SparseParameterWrapper(sparse))
        return module

    def sparsify_model_and_optimizer_inplace(self, module, optimizer):
        before = [id(p) for p in module.parameters()]
        where = {id(p): (gi, pi) for gi, grp in enumerate(optimizer.param_groups) for pi, p in enumerate(grp["params"])}
        module = self.sparsify_model_inplace(module)
        for param, old in zip(module.parameters(), before):
            if id(param) != old and old in where:
                gi, pi = where[old]
                optimizer.param_groups[gi]["params"][pi] = param
        return module, optimizer

    def get_sparse_model(self, module):
        return self.sparsify_model_inplace(copy.deepcopy(module))
