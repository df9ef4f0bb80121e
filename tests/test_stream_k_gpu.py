"""Stream-K of the 512 x 256 CTA-pair kernel: the pairs share the k-blocks of all tiles evenly; a pair whose range ends
inside a tile leaves raw partial sums in a workspace, the pair holding the tile's last k-block adds them (fixed order).

It is an option (`stream_k` = 1): on B200 it measured within a few percent of whole tiles either way, so the library
does not choose it by itself. Checked here: the result against the CPU oracle on sampled rows and against the whole-tile kernel on every element
(same products, another fp32 summation grouping: a few ulps before the output rounding), bit-identical repeats, one
kernel launch, every epilogue and both layouts of B, ragged edges, tiles split across many pairs (forced on small
problems), operands that need the repack pre-pass (the workspace then sits behind the repacked copies), batches, and
two streams sharing the pooled workspace.
"""
import numpy as np
import pytest
import torch

import symplex_b200 as sx
from oracle_loader import rel_frobenius
from symplex_b200 import _capi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sk_count(lib):
    return lib.symplex_b200_get_option(b"stream_k_launches")


def _operands(M, N, K, seed, b_layout=sx.ROW_MAJOR, batch=None):
    g = torch.Generator(device=DEV).manual_seed(seed)
    lead = () if batch is None else (batch,)
    A = torch.randn(*lead, M, K, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(*lead, *((K, N) if b_layout == sx.ROW_MAJOR else (N, K)), device=DEV, generator=g).to(torch.bfloat16)
    return A, B


def _oracle_rows(oracle, A, B, rows, b_layout, bias=None, act=_capi.ACT_NONE, bf16=True):
    Af = A.float().cpu().numpy()
    Bf = B.float().cpu().numpy()
    if b_layout == sx.COL_MAJOR:
        Bf = np.ascontiguousarray(Bf.T)
    ref = oracle.epilogue(oracle.matmul_rows(Af, Bf, rows), bias=None if bias is None else bias.cpu().numpy(), act=act)
    return oracle.bf16_round(ref) if bf16 else ref


def test_stream_k_on_a_mostly_idle_last_wave(lib, oracle, set_option):
    """4608 x 4608: 162 tiles of 512 x 256 on 74 pairs are 2.19 waves - the third wave keeps 14 pairs busy and 60 idle.
    Stream-K is an option (it measured no faster than whole tiles on this GPU), so by default it does not run."""
    M = N = 4608
    K = 4096
    A, B = _operands(M, N, K, 21)
    before = _sk_count(lib)
    whole = sx.gemm(A, B)
    assert _sk_count(lib) == before, "stream-K must not run unless the option asks for it"
    set_option("stream_k", 1)
    launches = sx.launch_count()
    got = sx.gemm(A, B)
    assert sx.launch_count() - launches == 1, "stream-K is one kernel launch"
    assert _sk_count(lib) == before + 1
    again = sx.gemm(A, B)
    sx.sync_status()
    assert torch.equal(got, again), "stream-K must repeat bit for bit"
    # the same products summed in another grouping: equal up to the rounding of the bf16 output
    diff = (got.float() - whole.float()).abs()
    assert float(diff.max()) <= 2.0 ** -7 * float(whole.float().abs().max())
    assert float((diff > 0).float().mean()) < 0.05
    rows = np.sort(np.random.default_rng(2).choice(M, 48, replace=False))
    ref = _oracle_rows(oracle, A, B, rows, sx.ROW_MAJOR)
    assert rel_frobenius(got[torch.from_numpy(rows).to(DEV)].float().cpu().numpy(), ref) <= 1e-2


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b_layout", [sx.ROW_MAJOR, sx.COL_MAJOR])
@pytest.mark.parametrize("shape", [(1024, 1024, 9600),    # 8 tiles: every tile is shared by nine or ten pairs
                                   (1500, 1000, 9608),    # ragged rows, columns and last k-block
                                   (2048, 2560, 2048),    # 40 tiles, two or three pairs per tile
                                   (4096, 4864, 1024)])   # 152 tiles: two whole tiles per pair plus a share
def test_forced_stream_k_matches_the_oracle_and_the_whole_tile_kernel(lib, oracle, set_option, shape, b_layout, out_dtype):
    M, N, K = shape
    A, B = _operands(M, N, K, 22, b_layout)
    bias = torch.randn(N, device=DEV, generator=torch.Generator(device=DEV).manual_seed(3))
    kw = dict(bias=bias, activation="gelu", out_dtype=out_dtype, b_layout=b_layout)
    set_option("pair_mode", 2)
    set_option("stream_k", 0)
    whole = sx.gemm(A, B, **kw)
    set_option("stream_k", 1)
    before = _sk_count(lib)
    got = sx.gemm(A, B, **kw)
    sx.sync_status()
    assert _sk_count(lib) == before + 1
    assert torch.equal(got, sx.gemm(A, B, **kw))
    tol = 2.0 ** -7 if out_dtype == torch.bfloat16 else 2e-5
    scale = float(whole.float().abs().max())
    assert float((got.float() - whole.float()).abs().max()) <= tol * scale
    rows = np.sort(np.random.default_rng(4).choice(M, 40, replace=False))
    ref = _oracle_rows(oracle, A, B, rows, b_layout, bias=bias, act=_capi.ACT_GELU, bf16=out_dtype == torch.bfloat16)
    assert rel_frobenius(got[torch.from_numpy(rows).to(DEV)].float().cpu().numpy(), ref) <= 1e-2


def test_stream_k_with_residual_alpha_beta_and_plain_stores(lib, oracle, set_option):
    """beta * residual + alpha * AB through the register-store epilogue (tma_store off) and the staged one."""
    M, N, K = 1536, 1280, 6400
    A, B = _operands(M, N, K, 23)
    R = torch.randn(M, N, device=DEV, generator=torch.Generator(device=DEV).manual_seed(5)).to(torch.bfloat16)
    set_option("pair_mode", 2)
    outs = []
    for tma_store in (1, 0):
        set_option("tma_store", tma_store)
        set_option("stream_k", 1)
        before = _sk_count(lib)
        outs.append(sx.gemm(A, B, residual=R, alpha=0.5, beta=-1.5, activation="relu"))
        assert _sk_count(lib) == before + 1
    sx.sync_status()
    assert torch.equal(outs[0], outs[1]), "both store paths write the same values"
    rows = np.arange(0, M, 37)
    acc = oracle.matmul_rows(A.float().cpu().numpy(), B.float().cpu().numpy(), rows)
    ref = np.maximum(0.5 * acc - 1.5 * R.float().cpu().numpy()[rows], 0.0)
    assert rel_frobenius(outs[0][torch.from_numpy(rows).to(DEV)].float().cpu().numpy(), oracle.bf16_round(ref)) <= 1e-2


def test_stream_k_behind_the_repack_prepass_and_over_a_batch(lib, oracle, set_option):
    """K = 8204 breaks the 16-byte row alignment TMA needs: A and B are repacked into the pooled scratch and the
    stream-K workspace lies behind them. Then a batch of three: tiles of all problems form one line of k-blocks."""
    set_option("pair_mode", 2)
    set_option("stream_k", 1)
    M, N, K = 2048, 1024, 8204
    A, B = _operands(M, N, K, 24, sx.COL_MAJOR)
    before = _sk_count(lib)
    got = sx.gemm(A, B, b_layout=sx.COL_MAJOR)
    sx.sync_status()
    assert _sk_count(lib) == before + 1
    rows = np.arange(0, M, 41)
    ref = _oracle_rows(oracle, A, B, rows, sx.COL_MAJOR)
    assert rel_frobenius(got[torch.from_numpy(rows).to(DEV)].float().cpu().numpy(), ref) <= 1e-2

    A3, B3 = _operands(1024, 1024, 4096, 25, batch=3)
    before = _sk_count(lib)
    got3 = sx.gemm(A3, B3)
    sx.sync_status()
    assert _sk_count(lib) == before + 1
    set_option("stream_k", 0)
    whole3 = sx.gemm(A3, B3)
    assert float((got3.float() - whole3.float()).abs().max()) <= 2.0 ** -7 * float(whole3.float().abs().max())
    rows = np.arange(0, 1024, 53)
    for z in range(3):
        ref = _oracle_rows(oracle, A3[z], B3[z], rows, sx.ROW_MAJOR)
        assert rel_frobenius(got3[z][torch.from_numpy(rows).to(DEV)].float().cpu().numpy(), ref) <= 1e-2


def test_two_streams_share_the_stream_k_workspace(lib, set_option):
    """The workspace and the flag words belong to the device's scratch pool: launches from two streams are ordered on
    the GPU by the pool's event, so neither overwrites partial sums the other still has to add."""
    set_option("pair_mode", 2)
    set_option("stream_k", 1)
    probs = []
    for i, (M, N, K) in enumerate([(2048, 2560, 2048), (1024, 1024, 9600), (4096, 4096, 1024)]):
        A, B = _operands(M, N, K, 30 + i)
        probs.append((A, B, sx.gemm(A, B)))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(device=DEV) for _ in range(2)]
    outs = []
    for rep in range(6):
        for i, (A, B, want) in enumerate(probs):
            s = streams[(rep + i) % 2]
            with torch.cuda.stream(s):
                outs.append((sx.gemm(A, B, stream=s.cuda_stream), want))
    torch.cuda.synchronize()
    sx.sync_status()
    for got, want in outs:
        assert torch.equal(got, want)


def test_stream_k_is_not_taken_where_it_cannot_run(lib, set_option):
    """Forced on, but the range per pair would be shorter than 16 k-blocks: the whole-tile kernel runs."""
    set_option("pair_mode", 2)
    set_option("stream_k", 1)
    A, B = _operands(1024, 512, 256, 40)  # 4 tiles x 4 k-blocks: far fewer than 16 k-blocks per pair
    before = _sk_count(lib)
    got = sx.gemm(A, B)
    sx.sync_status()
    assert _sk_count(lib) == before
    set_option("stream_k", 0)
    assert torch.equal(got, sx.gemm(A, B))
