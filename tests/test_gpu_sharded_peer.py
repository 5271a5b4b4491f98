"""Row-sharded matmul on two GPUs: the exchange done by the matmul epilogue (stores into every rank's buffer over
NVLink) against the NCCL all-gather variant and against a dense product.  Needs two GPUs; skipped otherwise.
NVLS is switched off for the NCCL calls of this test (plain rings / trees are enough for a 4-byte all-reduce)."""
import datetime
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_q):
    import torch.distributed as dist
    import sten_b200 as sten
    from sten_b200.sharded import RowShardedNMMatmul
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120), device_id=dev)
    try:
        M, K, tokens, n, m, g = 1024, 520, 1104, 2, 8, 16
        gen = torch.Generator().manual_seed(5)
        w = (torch.randn(M, K, generator=gen) * 0.05).bfloat16().to(dev)
        x = torch.randn(tokens, K, generator=gen).bfloat16().to(dev)
        results = {}
        for exchange, rounds in (("peer", 1), ("peer", 2), ("gather", 2)):
            layer = RowShardedNMMatmul.from_full_weight(w, n, m, g, rounds=rounds, exchange=exchange)
            for _ in range(2):  # the peer buffers are reused by the second call
                c = layer(x)
            torch.cuda.synchronize()
            results[(exchange, rounds)] = c.clone()
        full = sten.GroupedNMTensor.from_dense(w, n, m, sparse_dim=0, group_size=g, group_dim=1).to_dense()
        ref = full.double() @ x.double().t()
        errs = {k: float((v.double() - ref).norm() / ref.norm()) for k, v in results.items()}
        def close(a, b):  # variants differ in fp32 summation order (fused kernel with a split reduction axis vs two passes)
            return float((a.double() - b.double()).norm() / b.double().norm()) <= 2e-3

        same = torch.equal(results[("peer", 1)], results[("peer", 2)]) and close(results[("gather", 2)], results[("peer", 1)])
        # Consecutive calls with DIFFERENT activations and a consumer kernel in between, never synchronising the host:
        # a rank that runs ahead must not overwrite a result a slower rank is still reading (the layer alternates two
        # peer buffers for that).  Rank 1 is made slow by extra work queued before each of its consumers.  Both store
        # paths are covered: through the NVSwitch multicast address (when the allocation has one) and one store per peer.
        how = {}
        for multicast in (True, False):
            layer = RowShardedNMMatmul.from_full_weight(w, n, m, g, rounds=1, exchange="peer")
            layer.multicast = multicast
            xs = [torch.randn(tokens, K, generator=gen).bfloat16().to(dev) for _ in range(4)]
            ballast = torch.randn(4096, 4096, device=dev)
            consumed = []
            for xi in xs:
                ci = layer(xi)
                if rank == 1:
                    for _ in range(3):
                        ballast = (ballast @ ballast).clamp_(-1, 1)
                consumed.append(ci.double())  # the consumer: reads the peer buffer on the layer's stream
            torch.cuda.synchronize()
            how[multicast] = layer.last_exchange
            for xi, got in zip(xs, consumed):
                want = full.double() @ xi.double().t()
                errs[("consecutive", multicast, len(errs))] = float((got - want).norm() / want.norm())
        errs["store paths"] = 0.0 if ("one st.global per peer" in how[False]) else 1.0
        print(f"rank {rank}: peer exchange ran as {how}", flush=True)
        # host operands: every rank uploads half of X, downloads the rows it computed
        layer = RowShardedNMMatmul.from_full_weight(w, n, m, g, rounds=1, exchange="peer")
        x_host = x.cpu().pin_memory()
        out_host = torch.zeros(M, tokens, dtype=torch.bfloat16).pin_memory()
        layer.forward_host(x_host, out_host)
        torch.cuda.synchronize()
        rp = M // world
        same = same and close(out_host[rank * rp:(rank + 1) * rp], results[("peer", 1)][rank * rp:(rank + 1) * rp].cpu())
        same = same and float(out_host[(1 - rank) * rp:(2 - rank) * rp].abs().max()) == 0
        result_q.put((rank, errs, same, None))
    except Exception as exc:  # noqa: BLE001 - reported to the parent, which fails the test
        result_q.put((rank, None, False, repr(exc)))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_store_exchange_matches_all_gather_and_dense():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, errs, same, exc in got:
        assert exc is None, f"rank {rank}: {exc}"
        assert same, f"rank {rank}: exchange variants disagree"
        assert all(e <= 1e-2 for e in errs.values()), (rank, errs)


def test_host_operand_pipeline_on_one_gpu():
    """forward_host on a single rank: chunked upload / matmul / pitched download on three streams."""
    import sten_b200 as sten
    from sten_b200.sharded import RowShardedNMMatmul
    dev = torch.device("cuda", 0)
    M, K, tokens, n, m, g = 512, 520, 3000, 2, 8, 16
    gen = torch.Generator().manual_seed(9)
    w = (torch.randn(M, K, generator=gen) * 0.05).bfloat16().to(dev)
    x_host = torch.randn(tokens, K, generator=gen).bfloat16().pin_memory()
    layer = RowShardedNMMatmul.from_full_weight(w, n, m, g, rounds=2)
    out_host = torch.zeros(M, tokens, dtype=torch.bfloat16).pin_memory()
    for _ in range(2):  # second call reuses the staging buffers and streams
        layer.forward_host(x_host, out_host, chunk_tokens=1024)
    torch.cuda.synchronize()
    direct = layer(x_host.to(dev))
    # chunks of 1024 tokens and the whole batch may take different kernel variants: same numbers up to fp32 summation order
    assert float((out_host.double() - direct.cpu().double()).norm() / direct.double().norm()) <= 2e-3
    full = sten.GroupedNMTensor.from_dense(w, n, m, sparse_dim=0, group_size=g, group_dim=1).to_dense()
    ref = full.double() @ x_host.to(dev).double().t()
    assert float((direct.double() - ref).norm() / ref.norm()) <= 1e-2
