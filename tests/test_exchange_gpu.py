"""The in-kernel exchange of the row-sharded GEMM (symplex_b200_sharded_gemm), driven over the C ABI on ONE GPU.

Two ranks are emulated one after the other: every "rank" gets its own full C buffer and flag block on the same GPU,
and the flags a real peer would write (READY / DONE of the current call) are set by the test before the launch, so
the single kernel never waits for another kernel. That exercises everything the forwarder warps do - waiting for
the flags, copying each finished tile from the local C to the peer's C, the completion counter, and the flags they
write for the peer - without a second GPU. (Two GPUs and the multicast mode: tests/test_sharded_gpu.py.)

Also here: a peer that never shows up (a flag nothing sets) makes the bounded wait run out, the kernel unwinds and
reports SYMPLEX_ERR_TIMEOUT, and the next call works; the library's unwinding self-test; and the serialisation of
the pooled scratch between streams and host threads.
"""
import ctypes
import threading

import numpy as np
import pytest
import torch

import symplex_b200 as sx
from oracle_loader import rel_frobenius
from symplex_b200 import _capi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
READY, DONE = 0, 8  # word offsets inside a flag block


def _comm(rank, c_bufs, flag_bufs, wait_limit_ms=0):
    comm = _capi.Comm()
    comm.rank, comm.world = rank, len(c_bufs)
    for r, (c, f) in enumerate(zip(c_bufs, flag_bufs)):
        comm.c_base[r] = c.data_ptr()
        comm.flags[r] = f.data_ptr()
    comm.c_multicast = None
    comm.epoch = 0
    comm.wait_limit_ms = wait_limit_ms
    return comm


def _sharded(lib, desc, A_local, B, bias, comm, mode=_capi.XCHG_UNICAST):
    s = torch.cuda.current_stream().cuda_stream
    return lib.symplex_b200_sharded_gemm(ctypes.byref(desc), A_local.data_ptr(), B.data_ptr(),
                                         bias.data_ptr() if bias is not None else None, ctypes.byref(comm), mode, s)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(2048, 1024, 512), (1024, 520, 136), (8192, 2048, 256), (600, 264, 72),
                                   (4096, 1024, 512, 1), (4096, 1024, 512, 2)])
def test_forwarders_copy_every_tile_to_the_peer(lib, oracle, set_option, shape, out_dtype):
    if len(shape) == 4:  # both tile shapes of the CTA-pair kernel carry the forwarder warps
        set_option("pair_mode", shape[3])
    M, N, K = shape[:3]
    world, m_loc = 2, M // 2
    g = torch.Generator(device=DEV).manual_seed(5)
    A = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(K, N, device=DEV, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV, generator=g)
    want = sx.gemm(A, B, bias=bias, activation="relu", out_dtype=out_dtype)
    d = sx.make_desc(M, N, K, sx.DT_BF16, sx.DT_BF16 if out_dtype == torch.bfloat16 else sx.DT_F32, activation="relu")
    C = [torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype) for _ in range(world)]
    F = [torch.zeros(64, device=DEV, dtype=torch.int32) for _ in range(world)]
    comms = [_comm(r, C, F) for r in range(world)]
    for epoch in (1, 2):  # twice: the second call overwrites what the first one delivered
        for r in range(world):
            peer = 1 - r
            # what the peer's kernel would have written into this rank's flag block by now
            F[r][READY + peer] = epoch
            F[r][DONE + peer] = epoch
            before = sx.launch_count()
            assert _sharded(lib, d, A[r * m_loc:(r + 1) * m_loc], B, bias, comms[r]) == 0, _capi.last_error()
            assert sx.launch_count() - before == 1, "GEMM and exchange must be one kernel"
            assert lib.symplex_b200_sync_status(None) == 0, _capi.last_error()
            assert comms[r].epoch == epoch
            # this rank told its peer that it entered the call and that its tiles have landed
            assert int(F[peer][READY + r]) == epoch and int(F[peer][DONE + r]) == epoch
        for r in range(world):
            assert torch.equal(C[r], want), f"epoch {epoch}: rank {r}'s gathered C differs from the one-GPU product"
        if epoch == 1:
            for c in C:
                c.fill_(float("nan"))
    # and the one-GPU product itself against the oracle on sampled rows
    rows = np.sort(np.random.default_rng(1).choice(M, min(M, 48), replace=False))
    Af, Bf = A.float().cpu().numpy(), B.float().cpu().numpy()
    ref = oracle.epilogue(oracle.matmul_rows(Af, Bf, rows), bias=bias.cpu().numpy(), act=_capi.ACT_RELU)
    if out_dtype == torch.bfloat16:
        ref = oracle.bf16_round(ref)
    assert rel_frobenius(C[0][torch.from_numpy(rows).to(DEV)].float().cpu().numpy(), ref) <= 1e-2


def test_a_peer_that_never_shows_up_times_out_and_the_next_call_works(lib):
    """READY of the peer is never written: the forwarders' bounded wait (5 ms here) runs out, every role of every
    CTA unwinds, the kernel returns and the status word says SYMPLEX_ERR_TIMEOUT. Nothing traps or spins on."""
    M, N, K = 1024, 512, 256
    g = torch.Generator(device=DEV).manual_seed(6)
    A = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(K, N, device=DEV, generator=g).to(torch.bfloat16)
    d = sx.make_desc(M, N, K, sx.DT_BF16, sx.DT_BF16)
    C = [torch.zeros(M, N, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    F = [torch.zeros(64, device=DEV, dtype=torch.int32) for _ in range(2)]
    comm = _comm(0, C, F, wait_limit_ms=5)
    assert _sharded(lib, d, A[:M // 2], B, None, comm) == 0
    assert lib.symplex_b200_sync_status(None) == _capi.ERR_TIMEOUT
    assert "timed out" in _capi.last_error()
    assert int(F[1][DONE + 0]) == 0, "a rank that gave up must not tell its peer that its tiles have landed"
    assert lib.symplex_b200_sync_status(None) == 0  # the word was cleared
    # the same communicator, now with the peer's flags in place: works
    F[0][READY + 1] = 2
    F[0][DONE + 1] = 2
    assert _sharded(lib, d, A[:M // 2], B, None, comm) == 0
    assert lib.symplex_b200_sync_status(None) == 0, _capi.last_error()
    assert torch.equal(C[1][:M // 2], sx.gemm(A[:M // 2], B))
    # an ordinary product still works on this device
    assert torch.equal(sx.gemm(A, B), sx.gemm(A, B))
    assert lib.symplex_b200_sync_status(None) == 0


def test_unwinding_self_test(lib, oracle):
    """symplex_b200_selftest_wait_timeout: the TMA producer leaves out the last k-block, the MMA thread's 2 ms wait
    runs out, the CTA unwinds (copies drained, tensor memory freed) and the kernel returns with its status set."""
    g = torch.Generator(device=DEV).manual_seed(7)
    A = torch.randn(128, 128, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(128, 64, device=DEV, generator=g).to(torch.bfloat16)
    C = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        rc = lib.symplex_b200_selftest_wait_timeout(A.data_ptr(), B.data_ptr(), C.data_ptr(), 2, None)
        assert rc == _capi.ERR_TIMEOUT, _capi.last_error()
        assert lib.symplex_b200_sync_status(None) == 0
    # tensor memory was released and the device is healthy: the same shape through the same kernel, for real
    with _capi.option("pair_mode", 0):
        got = sx.gemm(A, B)
    sx.sync_status()
    ref = oracle.bf16_round(oracle.jit_parallel_matmul(A.float().cpu().numpy(), B.float().cpu().numpy()))
    assert rel_frobenius(got.float().cpu().numpy(), ref) <= 1e-2
    assert lib.symplex_b200_selftest_wait_timeout(A.data_ptr(), B.data_ptr(), C.data_ptr(), 0, None) == _capi.ERR_INVALID


def test_pooled_scratch_is_serialised_between_streams(lib):
    """Two streams run fp32 products that both need the pooled {hi, lo} planes: the second user must wait for the
    first one's kernels on the GPU (an event), and growing the pool must not free a block in use."""
    g = torch.Generator(device=DEV).manual_seed(8)
    probs = []
    for (M, N, K) in [(2048, 1536, 640), (1536, 2048, 1024), (3072, 1280, 768)]:  # growing scratch: 3 pool growths
        A = torch.rand(M, K, device=DEV, generator=g) * 2 - 1
        B = torch.rand(K, N, device=DEV, generator=g) * 2 - 1
        probs.append((A, B, sx.gemm(A, B)))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(device=DEV) for _ in range(2)]
    outs = []
    for rep in range(4):
        for i, (A, B, want) in enumerate(probs):
            s = streams[(rep + i) % 2]
            with torch.cuda.stream(s):
                outs.append((sx.gemm(A, B, stream=s.cuda_stream), want))
    torch.cuda.synchronize()
    sx.sync_status()
    for got, want in outs:
        assert torch.equal(got, want)


def test_host_paths_keep_their_scratch_per_thread(lib, oracle):
    """Two host threads call the host-pointer drop-in with fp32 problems that need scratch, at the same time."""
    rng = np.random.default_rng(9)
    jobs = []
    for (M, N, K) in [(1500, 1100, 300), (1100, 1500, 520)]:
        A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        jobs.append((A, B, sx.matmul_jit(A, B)))
    results = {}

    def work(i):
        A, B, _ = jobs[i]
        results[i] = [sx.matmul_jit(A, B) for _ in range(6)]

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for i, (A, B, serial) in enumerate(jobs):
        for got in results[i]:
            np.testing.assert_array_equal(got, serial)
        rows = np.arange(0, A.shape[0], 97)
        assert rel_frobenius(serial[rows], oracle.matmul_rows(A, B, rows)) <= 1e-5
