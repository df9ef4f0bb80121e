"""Host logic of the row-sharded GEMM on CPU: the plan, the row ownership map, and the chunked in-place
all-gather pipeline run as two gloo ranks. The per-chunk product is injected (torch on CPU) - these
tests exercise the distribution logic, not the GPU kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from symplex_b200 import sharding
from symplex_b200.sharding import ShardingStrategy


def test_plan_matches_row_sharded_config():
    # the row-sharded workload: A [65536, 8192] split by rows, B replicated, bf16 C all-gathered
    plan = sharding.analyze_matmul(65536, 8192, 8192, 8)
    a, b, c = plan.tensor_shards
    assert (a.strategy, a.local_shape) == (ShardingStrategy.SHARD_DIM_0, [8192, 8192])
    assert (b.strategy, b.local_shape) == (ShardingStrategy.REPLICATE, [8192, 8192])
    assert (c.strategy, c.original_shape, c.local_shape) == (ShardingStrategy.SHARD_DIM_0, [65536, 8192], [8192, 8192])
    assert plan.all_gather_ops == ["all_gather(C, dim=0)"] and plan.all_reduce_ops == []
    # every rank receives 7/8 of C in bf16
    assert plan.total_communication_bytes == 8 * 7 * 8192 * 8192 * 2
    assert "SHARD_DIM_0" in plan.to_string() and "comm_bytes=" in plan.to_string()


def test_plan_like_reference_test():
    # tests/test_distributed.cpp:27-33 of the reference: analyze_matmul(4096^3) gives a non-empty plan
    # with communication; a single device needs none.
    plan = sharding.analyze_matmul(4096, 4096, 4096, 4)
    assert plan.tensor_shards and plan.total_communication_bytes > 0
    solo = sharding.analyze_matmul(4096, 4096, 4096, 1)
    assert solo.total_communication_bytes == 0 and solo.all_gather_ops == []
    with pytest.raises(ValueError):
        sharding.analyze_matmul(1000, 8, 8, 3)


@pytest.mark.parametrize("M,world,chunks", [(1024, 2, 4), (65536, 8, 4), (512, 4, 1), (768, 3, 2)])
def test_row_ownership_is_a_partition(M, world, chunks):
    seen = np.zeros(M, np.int32)
    for r in range(world):
        blocks = sharding.owned_row_blocks(M, world, r, chunks)
        assert len(blocks) == chunks
        for c, (start, n) in enumerate(blocks):
            assert n == M // (world * chunks)
            # chunk c of every rank lies inside one contiguous block of C, in rank order
            assert c * (M // chunks) <= start and start + n <= (c + 1) * (M // chunks)
            assert start == c * (M // chunks) + r * n
            seen[start:start + n] += 1
    assert np.all(seen == 1)


def test_pick_chunks():
    assert sharding.pick_chunks(65536, 1) == 1
    assert sharding.pick_chunks(65536, 8) == 4
    assert sharding.pick_chunks(65536, 8, 16) == 16
    assert sharding.pick_chunks(1024, 8) == 1      # 128 rows per rank: one tile, no split
    assert sharding.pick_chunks(3 * 256, 2, 4) == 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_gemm(A_blk, B, bias, out_blk):
    r = A_blk.float() @ B.float()
    if bias is not None:
        r = r + bias
    out_blk.copy_(r.to(out_blk.dtype))


def _worker(rank, world, port, M, N, K, chunks, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1234)
        A = torch.randn(M, K, generator=g)
        B = torch.randn(K, N, generator=g)
        bias = torch.randn(N, generator=g)
        op = sharding.RowShardedGemm(M, N, K, chunks=chunks, local_gemm=_cpu_gemm)
        idx = op.local_row_index()
        C = op(A[idx].contiguous(), B, bias=bias, out_dtype=torch.float32)
        ref = A @ B + bias
        q.put((rank, op.chunks, bool(torch.equal(C, ref)), idx.tolist()[:3]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 2), (8, 2)])
def test_gloo_pipeline(world, chunks):
    """The host side of the row-sharded product (row ownership, chunked all-gather, gathered C) on CPU ranks: two
    ranks, and eight - the largest world the one-box exchange is built for."""
    M, N, K = 256 * world, 48, 40
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, chunks, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, used_chunks, ok, first_rows in sorted(results):
        assert used_chunks == chunks
        assert ok, f"rank {rank}: gathered C differs from the full product"
    starts = {r: rows[0] for r, _, _, rows in results}
    assert starts[0] == 0 and starts[1] == M // (world * chunks)


def test_single_process_without_process_group():
    op = sharding.RowShardedGemm(256, 32, 16, local_gemm=_cpu_gemm)
    assert (op.world, op.rank, op.chunks) == (1, 0, 1)
    A = torch.randn(256, 16)
    B = torch.randn(16, 32)
    torch.testing.assert_close(op(A, B, out_dtype=torch.float32), A @ B)
    with pytest.raises(ValueError):
        op(torch.randn(100, 16), B)


def _absent_rank_worker(rank, world, port, q):
    """Rank 1 completes step 1 and then never enters step 2 (it just waits for the others to notice, on the host).
    Rank 0 must get a ShardedStepTimeout after its deadline instead of blocking inside the collective."""
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 256, 16, 8
        g = torch.Generator().manual_seed(5)
        A, B = torch.randn(M, K, generator=g), torch.randn(K, N, generator=g)
        op = sharding.RowShardedGemm(M, N, K, chunks=1, local_gemm=_cpu_gemm, step_deadline_s=1.0)
        idx = op.local_row_index()
        C = op(A[idx].contiguous(), B, out_dtype=torch.float32)  # step 1: everybody is there
        ok1 = bool(torch.equal(C, A @ B))
        outcome = "absent"
        if rank == 0:
            t0 = time.monotonic()
            try:
                op(A[idx].contiguous(), B, out_dtype=torch.float32)  # step 2: rank 1 never comes
                outcome = "returned"
            except sharding.ShardedStepTimeout as e:
                outcome = f"timeout after {time.monotonic() - t0:.2f} s: {e}"
        else:
            time.sleep(2.5)  # stays alive (its store connection too) while rank 0 runs into its deadline
        q.put((rank, ok1, outcome))
    finally:
        dist.destroy_process_group()


def test_a_rank_that_never_enters_the_step_is_noticed_on_the_host():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_absent_rank_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict((r, (ok, out)) for r, ok, out in [q.get(timeout=120) for _ in range(world)])
    for p in procs:
        p.join(timeout=60)
    assert results[0][0] and results[1][0], "step 1 (all ranks present) must succeed"
    assert results[0][1].startswith("timeout after"), results[0][1]
    assert "1 of 2 ranks entered step 2" in results[0][1]
    assert 0.9 <= float(results[0][1].split()[2]) <= 2.4


def test_fp32_inputs_move_a_defaulted_instance_to_the_nccl_exchange():
    op = sharding.RowShardedGemm(256, 32, 16, local_gemm=_cpu_gemm)
    assert op.exchange == "nccl"
    with pytest.raises(ValueError):
        sharding.RowShardedGemm(256, 32, 16, exchange="carrier_pigeon")
