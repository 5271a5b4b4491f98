"""Row-sharded grouped n:m linear layers for one node of GPUs.

A weight ``W[M, K]`` is split by output rows: rank ``r`` of ``R`` owns rows ``[bounds[r], bounds[r+1])`` (multiples of
``m``, so n:m blocks are never cut), sparsifies only those rows -- the result is identical to slicing the sparsified
full weight because tiles never interact -- and computes its slice of the output.  The slices are combined with one
all-gather per token panel (NCCL over NVLink when the group is a NCCL group); nothing else is communicated.
Activations are replicated.  The reference has no multi-GPU path for this format; its only collective code is the
DDP gradient hook (src/sten/patches.py:125-218), which is unrelated.

The gather of panel ``p`` is issued asynchronously and overlaps the matmul of panel ``p + 1``.
"""
import math

import torch
import torch.distributed as dist

from . import ops
from .grouped_nm_tensor import GroupedNMTensor


def row_shard_bounds(M, world_size, m):
    """Row ranges of the shards: as even as possible in units of whole n:m blocks.  Returns ``world_size + 1`` offsets."""
    if world_size < 1 or M < 1 or m < 1:
        raise ValueError("need M >= 1, m >= 1, world_size >= 1")
    blocks = math.ceil(M / m)
    base, extra = divmod(blocks, world_size)
    bounds = [0]
    for r in range(world_size):
        bounds.append(min(M, bounds[-1] + (base + (1 if r < extra else 0)) * m))
    bounds[-1] = M
    return bounds


def _default_matmul(gnm, x2d, bias):
    s = gnm.nm_strides
    M, K = s["dense_shape"]
    packed = gnm.packed() if gnm.val.dtype in (torch.float16, torch.bfloat16) else None
    return ops.spmm(gnm.val, gnm.idx, int(M), int(K), s["n"], s["m"], s["group_size"], x2d, bias=bias, packed=packed)


class ShardedGroupedNMLinear:
    """``y = x W^T + b`` with ``W`` row-sharded over a process group.

    ``weight_shard``: this rank's rows as a ``GroupedNMTensor`` (``from_full_weight`` builds it).  ``matmul`` computes
    ``x2d @ shard^T + bias``; it defaults to the CUDA kernels and exists so the host logic can be exercised on CPU
    ranks with a stand-in."""

    def __init__(self, weight_shard, bias_shard, M_total, group=None, panels=4, matmul=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.weight_shard = weight_shard
        self.bias_shard = bias_shard
        self.M_total = int(M_total)
        self.panels = max(1, int(panels))
        self.matmul = matmul or _default_matmul
        s = weight_shard.nm_strides
        self.m = s["m"]
        self.bounds = row_shard_bounds(self.M_total, self.world, self.m)
        rows, K = s["dense_shape"]
        self.K = int(K)
        want = self.bounds[self.rank + 1] - self.bounds[self.rank]
        if int(rows) != want:
            raise ValueError(f"rank {self.rank} holds {int(rows)} rows but the row split of M={self.M_total} over "
                             f"{self.world} ranks assigns it {want}")
        self._check_agreement((self.M_total, self.K, s["n"], s["m"], s["group_size"]))

    @classmethod
    def from_full_weight(cls, weight, bias, n, m, g, group=None, panels=4, matmul=None, sparsify=None):
        """Every rank passes the same dense ``weight[M, K]``; each keeps and sparsifies only its rows."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        M = weight.shape[0]
        b = row_shard_bounds(M, world, m)
        rows = weight[b[rank]:b[rank + 1]]
        make = sparsify or (lambda w: GroupedNMTensor.from_dense(w, n, m, sparse_dim=0, group_size=g, group_dim=1))
        shard = make(rows)
        return cls(shard, None if bias is None else bias[b[rank]:b[rank + 1]], M, group, panels, matmul)

    def _check_agreement(self, meta):
        """All ranks must describe the same layer, otherwise the gather would silently mix shapes."""
        if self.world == 1:
            return
        gathered = [None] * self.world
        dist.all_gather_object(gathered, tuple(int(v) for v in meta), group=self.group)
        if any(g != gathered[0] for g in gathered):
            raise ValueError(f"ranks disagree on the sharded layer (M, K, n, m, g): {gathered}")

    def forward_local(self, x2d):
        """This rank's output columns ``[tokens, rows_of_this_rank]``; no communication."""
        return self.matmul(self.weight_shard, x2d, self.bias_shard)

    def forward(self, x):
        """Full output ``[..., M]`` on every rank."""
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.shape[1] != self.K:
            raise ValueError(f"activation has {x2d.shape[1]} features, the layer expects {self.K}")
        tokens = x2d.shape[0]
        if self.world == 1:
            return self.forward_local(x2d).reshape(*x.shape[:-1], self.M_total)
        sizes = [self.bounds[r + 1] - self.bounds[r] for r in range(self.world)]
        even = all(s == sizes[0] for s in sizes)
        out = torch.empty(tokens, self.M_total, dtype=x2d.dtype, device=x2d.device)
        step = math.ceil(tokens / self.panels)
        pending = []
        for t0 in range(0, tokens, step):
            t1 = min(tokens, t0 + step)
            y = self.forward_local(x2d[t0:t1])
            width = max(sizes)
            if not even:  # collectives want equal pieces: pad the ragged last shards, drop the padding after
                y = torch.nn.functional.pad(y, (0, width - y.shape[1]))
            stage = torch.empty(self.world * (t1 - t0), width, dtype=y.dtype, device=y.device)
            work = dist.all_gather_into_tensor(stage, y.contiguous(), group=self.group, async_op=True)
            pending.append((work, stage, width, t0, t1))
        for work, stage, width, t0, t1 in pending:
            work.wait()
            stage = stage.view(self.world, t1 - t0, width)  # [R, tokens_p, rows] -> columns of the row-major output
            if even:
                out[t0:t1].view(t1 - t0, self.world, width).copy_(stage.permute(1, 0, 2))
            else:
                for r in range(self.world):
                    out[t0:t1, self.bounds[r]:self.bounds[r + 1]] = stage[r, :, :sizes[r]]
        return out.reshape(*x.shape[:-1], self.M_total)

    __call__ = forward
