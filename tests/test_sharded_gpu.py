"""Row-sharded GEMM on real GPUs: NCCL all-gather pipeline against the single-GPU product (needs >= 2 GPUs;
the single-GPU form of the same operator is covered in test_gemm_gpu.py)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, chunks, exchange, q):
    import torch.distributed as dist

    import symplex_b200 as sx
    from symplex_b200.sharding import RowShardedGemm
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator(device=dev).manual_seed(99)  # same A and B on every rank
        A = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        B = torch.randn(K, N, device=dev, generator=g).to(torch.bfloat16)
        op = RowShardedGemm(M, N, K, chunks=chunks, exchange=exchange)
        idx = op.local_row_index().to(dev)
        ref = sx.gemm(A, B)  # the whole product on this GPU
        same = True
        for _ in range(2):  # twice: the second call overwrites a buffer the peers have already filled once
            C = op(A[idx].contiguous(), B)
            torch.cuda.synchronize()
            sx.sync_status()
            same = same and bool(torch.equal(C, ref))
        q.put((rank, op.chunks, op.exchange, same, float((C.float() - ref.float()).abs().max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange,chunks", [("peer_store", 1), ("nccl", 1), ("nccl", 4)])
def test_row_sharded_gemm_matches_single_gpu(exchange, chunks):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp
    M, N, K = 1024 * world, 1024, 512
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, chunks, exchange, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, used, used_exchange, same, maxdiff in sorted(results):
        assert used == chunks and used_exchange == exchange
        assert same, f"rank {rank}: gathered C differs from the single-GPU product (max |diff| {maxdiff})"
