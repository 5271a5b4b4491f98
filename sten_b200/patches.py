"""``patch(old, new, module_scope)`` and the data-parallel gradient hook for sparse parameters.

Reference: src/sten/patches.py:21-54 (``patch``) and :125-218 (``sparse_ddp_all_reduce_hook``, ``patch_ddp``).  The Apex
optimizer patches of the reference are outside the grouped n:m path and are not provided.
"""
import inspect
import sys

import torch


def _callables(owner):
    for name, member in inspect.getmembers(owner):
        if callable(member) and not inspect.isclass(member):
            yield name, member


def patch(old, new, module_scope=None):
    """Rebind every module-level name and every class attribute in ``module_scope`` that is ``old`` to ``new``.

    ``module_scope`` defaults to all currently imported ``torch*`` modules, as in the reference."""
    if module_scope is None:
        module_scope = [m for name, m in list(sys.modules.items()) if name.startswith("torch") and m is not None]
    for mod in module_scope:
        for _, cls in inspect.getmembers(mod, inspect.isclass):
            for name, member in _callables(cls):
                if member is old:
                    setattr(cls, name, new)
        for name, member in _callables(mod):
            if member is old:
                setattr(mod, name, new)


def _shares_layout(param, grad):
    """A grouped n:m gradient whose ``idx`` IS the weight's ``idx`` (what ``WeightLayoutSparsifier`` produces): weights
    are replicated under data parallelism, so such a layout is the same on every rank and ``val`` can be reduced as is."""
    from .grouped_nm_tensor import GroupedNMTensor
    w, g = param.wrapped_tensor, grad.wrapped_tensor
    return (isinstance(w, GroupedNMTensor) and isinstance(g, GroupedNMTensor) and g.idx.shape == w.idx.shape
            and (g.idx is w.idx or g.idx.data_ptr() == w.idx.data_ptr()))


def sparse_ddp_all_reduce_hook(state, bucket):
    """DDP communication hook for buckets that contain sparse parameters (reference: patches.py:125-199).

    The reference densifies every sparse gradient, all-reduces the dense copy and re-sparsifies the mean with a fresh
    selection.  That remains the path for a gradient with a layout of its own.  A grouped n:m gradient that carries its
    weight's layout is reduced in packed form instead: only ``val`` travels (n/m of the dense bytes), no densify, no
    re-selection, and the mean keeps the layout exactly.  Dense parameters of the bucket are averaged as DDP would.
    ``state`` may be a process group (None = the default group).  Returns the future DDP expects (the bucket buffer)."""
    import torch.distributed as dist
    from . import dispatch as sten
    group = state if state is not None else dist.group.WORLD
    world = dist.get_world_size(group)
    dense_buf = bucket.buffer()
    sparse_params = [p for p in bucket.parameters() if isinstance(p, sten.SparseTensorWrapper) and p.grad is not None]
    packed, densified = [], []
    for p in sparse_params:
        g = p.grad
        if isinstance(g, sten.SparseTensorWrapper) and _shares_layout(p, g):
            packed.append(g.wrapped_tensor.val)
        else:
            dense = g.wrapped_tensor.to_dense() if isinstance(g, sten.SparseTensorWrapper) else g
            densified.append((p, tuple(dense.shape), dense.flatten()))
    pieces = [v.reshape(-1) for v in packed] + [d for _, _, d in densified]
    futures = []
    flat = None
    if pieces:
        flat = torch.cat(pieces)  # a copy: dividing it leaves the gradients untouched until the mean is written back
        flat /= world
        futures.append(dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True).get_future())
    dense_buf /= world
    futures.append(dist.all_reduce(dense_buf, op=dist.ReduceOp.SUM, group=group, async_op=True).get_future())

    def finish(fut):
        if flat is not None:
            off = 0
            for v in packed:  # the mean goes straight back into the gradient's val: same layout on every rank
                v.copy_(flat[off:off + v.numel()].reshape(v.shape))
                off += v.numel()
            for p, shape, d in densified:  # own layout: re-sparsify the mean into the gradient's format (fresh selection)
                mean = flat[off:off + d.numel()].reshape(shape)
                off += d.numel()
                if isinstance(p.grad, sten.SparseTensorWrapper):
                    impl = sten.get_sparsifier_implementation(sten.SameFormatSparsifier, torch.Tensor, p.grad.wrapped_tensor.__class__)
                    p.grad.init_from_other(impl(sten.SameFormatSparsifier(p.grad), mean))
                else:
                    p.grad.copy_(mean)
        return dense_buf

    return torch.futures.collect_all(futures).then(finish)


def patch_ddp():
    """Make ``DistributedDataParallel`` register the hook above whenever the wrapped module has sparse parameters
    (reference: patches.py:202-218).  Opt-in here: call it once before constructing DDP."""
    from . import dispatch as sten
    ddp = torch.nn.parallel.DistributedDataParallel
    orig_init = ddp.__init__
    if getattr(orig_init, "_sten_b200_patched", False):
        return

    def init_with_hook(self, module, *args, **kwargs):
        orig_init(self, module, *args, **kwargs)
        if any(isinstance(p, sten.SparseParameterWrapper) for p in module.parameters()):
            self.register_comm_hook(state=None, hook=sparse_ddp_all_reduce_hook)

    init_with_hook._sten_b200_patched = True
    ddp.__init__ = init_with_hook
