"""The allocation-free fp32 GEMM entry point (symplex_b200_sgemm_noalloc) and its status reader.

Some users of this library may not allocate GPU memory when they call it: their own allocator already owns
the device, or their service forbids allocation (and the device-wide stall it causes) after start-up. For
them the library carries a fixed 16 MiB scratch array and this one entry point that uses it. The test calls
it through the C ABI twice in a row - the second time with a smaller problem, so stale scratch contents of
the first would show - and compares each result with the regular pooled entry point on the same inputs and
with the CPU oracle. It also checks what the entry point is for: a warm call leaves the amount of free device
memory exactly as it found it, and its failures are reported by symplex_b200_noalloc_status (which does not
allocate either), not by the pooled entry points' status call.
"""
import ctypes

import pytest
import torch

from oracle_loader import rel_frobenius
from symplex_b200 import _capi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _pooled(lib, A, B):
    M, K = A.shape
    N = B.shape[1]
    d = _capi.GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), M, N, K, _capi.DT_F32, _capi.DT_F32)
    C = torch.full((M, N), float("nan"), device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    assert lib.symplex_b200_gemm(ctypes.byref(d), A.data_ptr(), B.data_ptr(), C.data_ptr(), None, None, s) == 0
    return C


def _noalloc(lib, A, B, C=None):
    M, K = A.shape
    N = B.shape[1]
    if C is None:
        C = torch.full((M, N), float("nan"), device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    rc = lib.symplex_b200_sgemm_noalloc(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, s)
    assert rc == 0, _capi.last_error()
    return C


def test_noalloc_matches_pooled_entry_point_and_oracle_twice_in_a_row(lib, oracle):
    assert lib.symplex_cuda_available() == 1
    g = torch.Generator(device=DEV).manual_seed(77)
    for (M, N, K) in [(768, 640, 900), (130, 257, 63)]:  # second call: smaller and ragged
        A = torch.rand(M, K, device=DEV, generator=g) * 2 - 1
        B = torch.rand(K, N, device=DEV, generator=g) * 2 - 1
        want = _pooled(lib, A, B)
        got = _noalloc(lib, A, B)
        assert lib.symplex_b200_noalloc_status(torch.cuda.current_stream().cuda_stream) == 0, _capi.last_error()
        assert lib.symplex_b200_sync_status(None) == 0
        assert not torch.isnan(got).any()
        err = ((got.double() - want.double()).norm() / want.double().norm()).item()
        assert err <= 1e-5, f"{M}x{N}x{K}: rel. Frobenius error {err:.3e} vs the pooled entry point"
        ref = oracle.jit_parallel_matmul(A.cpu().numpy(), B.cpu().numpy())
        assert rel_frobenius(got.cpu().numpy(), ref) <= 1e-5


def test_a_warm_noalloc_call_leaves_free_device_memory_unchanged(lib):
    g = torch.Generator(device=DEV).manual_seed(78)
    A = torch.rand(512, 700, device=DEV, generator=g)
    B = torch.rand(700, 384, device=DEV, generator=g)
    C = torch.empty(512, 384, device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    _noalloc(lib, A, B, C)  # first call on the device: symbol lookup, module load
    assert lib.symplex_b200_noalloc_status(s) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        _noalloc(lib, A, B, C)
        assert lib.symplex_b200_noalloc_status(s) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the allocation-free entry point (or its status call) allocated device memory"


def test_noalloc_rejects_problems_beyond_its_scratch(lib):
    buf = torch.zeros(16, device=DEV)
    rc = lib.symplex_b200_sgemm_noalloc(buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 1024, 1024, 1024, None)
    assert rc == _capi.ERR_INVALID
    assert "16 MiB" in _capi.last_error()
    assert lib.symplex_b200_sgemm_noalloc(buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 0, 8, 8, None) == 0
