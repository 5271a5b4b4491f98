"""The data-parallel gradient hook for grouped n:m parameters, on two gloo ranks (CPU).

A gradient that carries its weight's layout is all-reduced in packed form: only ``val`` travels and the mean keeps the
layout.  The hook is exercised directly with a stand-in for DDP's bucket (``buffer()`` / ``parameters()``), which is all
it touches; no CUDA kernel is involved in the packed path."""
import os
import socket

import pytest
import torch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Bucket:
    def __init__(self, buf, params):
        self._buf, self._params = buf, params

    def buffer(self):
        return self._buf

    def parameters(self):
        return self._params


def _worker(rank, world, port, q):
    import torch.distributed as dist
    import sten_b200 as sten
    from sten_b200.layout import compute_nm_strides
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, n, m, g = 8, 12, 2, 4, 2
        strides = compute_nm_strides(torch.Size((M, K)), n, m, 0, 1, g)
        tiles, C = strides["sparse_val_shape"][0], strides["chunk_size"]
        gen = torch.Generator().manual_seed(3)
        idx = torch.stack([torch.randperm(C * g, generator=gen) for _ in range(tiles)]).to(torch.int16).reshape(tiles, C, g, 1)
        w_val = torch.randn(tiles, C, g, n, generator=gen)
        weight = sten.SparseParameterWrapper(
            sten.SparseTensorWrapper.wrapped_from_dense(sten.GroupedNMTensor(w_val, idx, strides), torch.zeros(1, requires_grad=True)))
        # this rank's gradient, in the weight's layout (same idx object)
        g_val = torch.full((tiles, C, g, n), float(rank + 1))
        weight.grad = sten.SparseTensorWrapper.wrapped_from_dense(sten.GroupedNMTensor(g_val, idx, strides), torch.zeros(1))
        dense_buf = torch.full((5,), float(10 * (rank + 1)))
        fut = sten.sparse_ddp_all_reduce_hook(None, _Bucket(dense_buf, [weight]))
        out = fut.wait()
        mean = sum(range(1, world + 1)) / world
        ok = torch.allclose(out, torch.full((5,), 10 * mean)) and torch.allclose(weight.grad.wrapped_tensor.val, torch.full_like(g_val, mean))
        ok = ok and weight.grad.wrapped_tensor.idx is idx  # the layout is untouched
        q.put((rank, bool(ok), None))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, False, repr(exc)))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_packed_gradients_are_averaged_without_densifying():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    for rank, ok, exc in got:
        assert exc is None, f"rank {rank}: {exc}"
        assert ok, f"rank {rank}: averaged gradient differs"
