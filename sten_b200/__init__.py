"""sten_b200 -- the grouped n:m ("nmg") hot path of STen on B200 (sm_100a).

Use it where the reference package is used: ``import sten_b200 as sten``.  The names exported here are the ones
the reference exports at top level (src/sten/__init__.py:1-6) that belong to this path.
"""
from .dispatch import *  # noqa: F401,F403
from .dispatch import (  # noqa: F401  (names with a leading capital are covered by *, listed for clarity)
    DenseTensor, DispatchError, DispatchWarning, KeepAll, SameFormatSparsifier, SparseOperatorDispatcher,
    SparseParameterWrapper, SparseTensorWrapper, SparsityBuilder, get_bwd_op_impl, get_fwd_op_impl,
    get_sparsifier_implementation, make_sparse_catcher, register_bwd_op_impl, register_fwd_op_impl,
    register_sparsifier_implementation, set_dispatch_failure, sparsified_op, unregister_sparsifier_implementation,
)
from .grouped_nm_tensor import GroupedNMTensor, PerfectNMTensor
from .nmg_impls import GroupedNMSparsifier, WeightLayoutSparsifier
from .fusion import fuse_linear_epilogues, sparse_linear_fused
from .patches import patch, patch_ddp, sparse_ddp_all_reduce_hook

__version__ = "0.1.0"
