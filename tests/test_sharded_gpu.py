"""Row-sharded GEMM on real GPUs (needs >= 2 GPUs): every exchange - the in-kernel forwarders (unicast stores and
NVSwitch multicast), the epilogue-TMA forwarding and the NCCL all-gather pipeline - must leave, on every rank, the
product one GPU computes (bit for bit: the same kernel computes every row either way), and that product is checked
against the CPU oracle on sampled rows. The forwarders themselves are also exercised on one GPU in
tests/test_exchange_gpu.py."""
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
    import sys

    import numpy as np
    import torch.distributed as dist

    import symplex_b200 as sx
    from symplex_b200.sharding import RowShardedGemm
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    result = (rank, None, exchange, False, float("nan"), float("nan"), "did not finish")
    op = None
    try:
        g = torch.Generator(device=dev).manual_seed(99)  # same A and B on every rank
        A = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        B = torch.randn(K, N, device=dev, generator=g).to(torch.bfloat16)
        op = RowShardedGemm(M, N, K, chunks=chunks, exchange=exchange)
        idx = op.local_row_index().to(dev)
        ref = sx.gemm(A, B)  # the whole product on this GPU
        same = True
        for _ in range(3):  # repeatedly: later calls overwrite a buffer the peers have already filled
            C = op(A[idx].contiguous(), B)
            torch.cuda.synchronize()
            sx.sync_status()
            same = same and bool(torch.equal(C, ref))
        err = 0.0
        if rank == 0:  # the product itself against the CPU oracle, on rows from every rank's share
            sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
            from oracle_loader import load_oracle, rel_frobenius
            oracle = load_oracle()
            rows = np.sort(np.random.default_rng(0).choice(M, 64, replace=False))
            want = oracle.bf16_round(oracle.matmul_rows(A.float().cpu().numpy(), B.float().cpu().numpy(), rows))
            err = rel_frobenius(C[torch.from_numpy(rows).to(dev)].float().cpu().numpy(), want)
        result = (rank, op.chunks, op.exchange, same, float((C.float() - ref.float()).abs().max()), err, "")
    except Exception as e:  # reported through the queue; the rank still leaves in step with the others (below)
        result = result[:6] + (repr(e),)
    finally:
        # Every rank reaches this point with no kernel in flight, and leaves together: no rank's memory disappears
        # while a peer still has it mapped (or bound to a multicast object).
        try:
            torch.cuda.synchronize()
            dist.barrier()
        except Exception:
            pass
        q.put(result)
        del op
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange,chunks", [("peer_store", 1), ("peer_store", 2), ("multicast", 1), ("epilogue_tma", 1),
                                             ("nccl", 1), ("nccl", 4)])
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
    if exchange == "multicast" and any("gave none" in r[6] for r in results):
        pytest.skip("this box offers no NVLink multicast mapping")
    for rank, used, used_exchange, same, maxdiff, err, problem in sorted(results):
        assert not problem, f"rank {rank}: {problem}"
        assert used == chunks and used_exchange == exchange
        assert same, f"rank {rank}: gathered C differs from the single-GPU product (max |diff| {maxdiff})"
        assert err <= 1e-2, f"rank {rank}: rel. Frobenius error {err:.3e} against the oracle"
