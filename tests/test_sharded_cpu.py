"""Host logic of the row-sharded layer on CPU ranks (gloo, world size 2).  The CUDA kernels cannot run here, so the
layer is given a stand-in matmul / sparsifier; what is tested is the sharding arithmetic, the gather assembly and the
failure handling (inconsistent ranks, a rank that never joins)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sten_b200.sharded import RowShardedNMMatmul, ShardedGroupedNMLinear, row_shard_bounds


class FakeGNM:
    """Stands in for GroupedNMTensor on CPU: dense rows plus the few nm_strides keys the layer reads."""

    def __init__(self, dense, n, m, g):
        self.dense = dense
        self.nm_strides = {"dense_shape": dense.shape, "n": n, "m": m, "group_size": g}


def fake_matmul(gnm, x2d, bias):
    y = x2d @ gnm.dense.t()
    return y if bias is None else y + bias


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _worker_ok(rank, world, port, result_q):
    _init(rank, world, port)
    torch.manual_seed(0)
    ok = True
    for M in (16, 20):  # even shards, then a ragged last shard (padded for the collective)
        w = torch.randn(M, 24)
        b = torch.randn(M)
        x = torch.randn(3, 5, 24)
        layer = ShardedGroupedNMLinear.from_full_weight(w, b, 2, 4, 2, panels=3, matmul=fake_matmul,
                                                        sparsify=lambda rows: FakeGNM(rows, 2, 4, 2))
        y = layer(x)
        ok = ok and torch.allclose(y, x @ w.t() + b, atol=1e-5) and y.shape == (3, 5, M)
        local = layer.forward_local(x.reshape(-1, 24))
        ok = ok and local.shape[1] == layer.bounds[rank + 1] - layer.bounds[rank]
    # torch.mm orientation, block-cyclic panels, in-place gathers
    w = torch.randn(32, 24)
    x = torch.randn(7, 24)
    mm = RowShardedNMMatmul.from_full_weight(w, 2, 4, 2, rounds=2, sparsify=lambda rows: FakeGNM(rows, 2, 4, 2),
                                             matmul=lambda gnm, x2d, out: out.copy_(gnm.dense @ x2d.t()))
    c = mm(x)
    ok = ok and c.shape == (32, 7) and torch.allclose(c, w @ x.t(), atol=1e-5)
    try:
        RowShardedNMMatmul.from_full_weight(torch.randn(20, 24), 2, 4, 2, rounds=2, sparsify=lambda r: FakeGNM(r, 2, 4, 2))
        ok = False
    except ValueError:
        pass
    result_q.put((rank, bool(ok)))
    dist.destroy_process_group()


def _worker_mismatch(rank, world, port, result_q):
    _init(rank, world, port)
    w = torch.randn(16, 8)
    try:
        b = row_shard_bounds(16, world, 4)
        g = 2 if rank == 0 else 3  # ranks disagree on the group size
        ShardedGroupedNMLinear(FakeGNM(w[b[rank]:b[rank + 1]], 2, 4, g), None, 16, matmul=fake_matmul)
        result_q.put((rank, "no error"))
    except ValueError as e:
        result_q.put((rank, "ValueError" if "disagree" in str(e) else str(e)))
    dist.destroy_process_group()


def _worker_absent_peer(rank, world, port, result_q):
    _init(rank, world, port, timeout_s=5)
    if rank == 1:
        result_q.put((rank, "left"))
        return  # leaves between steps, before any collective of the layer is in flight
    w = torch.randn(16, 8)
    try:
        b = row_shard_bounds(16, world, 4)
        layer = ShardedGroupedNMLinear(FakeGNM(w[b[0]:b[1]], 2, 4, 2), None, 16, matmul=fake_matmul)
        layer(torch.randn(4, 8))
        result_q.put((rank, "no error"))
    except Exception as e:  # gloo reports the missing peer as a RuntimeError / DistBackendError after the timeout
        result_q.put((rank, "error:" + type(e).__name__))


def _run(worker, world, *args):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, *args, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    return results


def test_row_shard_bounds():
    assert row_shard_bounds(16384, 8, 8) == [2048 * i for i in range(9)]
    assert row_shard_bounds(10, 2, 4) == [0, 8, 10]          # blocks are never cut; the ragged block goes last
    assert row_shard_bounds(4, 3, 4) == [0, 4, 4, 4]          # more ranks than blocks: empty shards
    b = row_shard_bounds(1000, 7, 4)
    assert b[0] == 0 and b[-1] == 1000 and all((x % 4 == 0) for x in b[:-1]) and b == sorted(b)
    with pytest.raises(ValueError):
        row_shard_bounds(0, 2, 4)


def test_two_rank_forward_matches_dense():
    res = _run(_worker_ok, 2)
    assert res == {0: True, 1: True}


def test_ranks_that_disagree_raise_on_every_rank():
    res = _run(_worker_mismatch, 2)
    assert res == {0: "ValueError", 1: "ValueError"}


def test_absent_peer_ends_in_an_error_not_a_hang():
    res = _run(_worker_absent_peer, 2)
    assert res[1] == "left" and res[0].startswith("error:")


def test_single_process_layer_needs_no_process_group():
    w = torch.randn(12, 8)
    layer = ShardedGroupedNMLinear(FakeGNM(w, 2, 4, 2), None, 12, matmul=fake_matmul)
    x = torch.randn(5, 8)
    assert torch.allclose(layer(x), x @ w.t(), atol=1e-6)
    with pytest.raises(ValueError):
        ShardedGroupedNMLinear(FakeGNM(w[:8], 2, 4, 2), None, 12, matmul=fake_matmul)
