"""Row-sharded GEMM across the GPUs of one box, and the ShardPlan vocabulary that describes it.

Mirrors the planning types of the reference (``include/symplex/distributed/sharding.h:18-95``:
``ShardingStrategy``, ``ShardingSpec``, ``ShardPlan``; ``nccl_bridge.h:19-26``: ``CollectiveOp``) and
turns the plan into an executed computation: one process per GPU, the tcgen05 GEMM library for the math,
``torch.distributed`` for the plumbing (process group, symmetric-memory rendezvous, barriers).

Ways to exchange C:

``exchange="peer_store"`` (default on GPUs with bf16 inputs)
    C lives in symmetric memory (every rank can address every rank's copy). ONE kernel per rank
    (``symplex_b200_sharded_gemm``) computes the local rows and gathers C: the epilogue writes each finished
    tile to the local C, and dedicated forwarder warps of the same kernel copy it from there (an L2 hit) to
    the same place in every peer's C with 16-byte stores over NVLink, so link back-pressure never reaches the
    warps that feed the tensor cores. The ranks order themselves with flags in each other's memory (a rank's
    C is not overwritten before that rank has entered the call; the kernel ends when every peer's tiles have
    landed) - no host barrier, no collective kernel competing for SMs.
``exchange="multicast"``
    Same kernel, but the forwarders store each tile ONCE to a multicast mapping of C (``multimem.st``) and the
    NVSwitch delivers it to every GPU: 1/(world-1) of the egress of ``peer_store``.
``exchange="epilogue_tma"``
    The first fused design, kept for comparison: the epilogue warps forward their own blocks with TMA stores
    (``symplex_b200_gemm_peers``), bracketed by two one-element all-reduces.
``exchange="nccl"``
    The local rows are computed in ``chunks`` pieces and each piece is gathered in place by an asynchronous
    ``all_gather_into_tensor`` while the next piece computes (also the path the CPU/gloo tests drive).

Partition (the reference parallelises the same way over CPU threads,
``rust-engine/src/x86_emitter.rs:1857-1874``): rows of A and C are split evenly over the ranks, B is
replicated, and C is all-gathered so every rank ends with the full product. To overlap the exchange
with compute the local rows are processed in ``chunks`` pieces; the piece of every rank for chunk c
forms one contiguous block of C, so each chunk is gathered in place by a single all-gather while the
next chunk's GEMM runs. Rank g therefore owns, for each chunk c, rows
``c*M/chunks + g*M/(chunks*world) + [0, M/(chunks*world))`` — with ``chunks == 1`` the usual
contiguous split.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple


class ShardingStrategy(enum.Enum):
    """``sharding.h:18-24``."""
    REPLICATE = 0
    SHARD_DIM_0 = 1
    SHARD_DIM_1 = 2
    SHARD_2D = 3
    PIPELINE = 4


class CollectiveOp(enum.Enum):
    """``nccl_bridge.h:19-26``."""
    ALL_REDUCE = 0
    ALL_GATHER = 1
    REDUCE_SCATTER = 2
    ALL_TO_ALL = 3
    BROADCAST = 4
    SEND_RECV = 5


@dataclass
class ShardingSpec:
    """``sharding.h:27-62``."""
    tensor_name: str
    strategy: ShardingStrategy = ShardingStrategy.REPLICATE
    shard_dims: List[int] = field(default_factory=list)
    original_shape: List[int] = field(default_factory=list)
    local_shape: List[int] = field(default_factory=list)

    def to_string(self) -> str:
        return (f"ShardingSpec{{name='{self.tensor_name}', strategy={self.strategy.name}, "
                f"shard_dims=[{', '.join(map(str, self.shard_dims))}], "
                f"original=[{'x'.join(map(str, self.original_shape))}], "
                f"local=[{'x'.join(map(str, self.local_shape))}]}}")


@dataclass
class ShardPlan:
    """``sharding.h:65-95`` plus ``all_gather_ops`` (the reference's plan only names all-reduce and
    all-to-all; the row-sharded GEMM needs an all-gather)."""
    tensor_shards: List[ShardingSpec] = field(default_factory=list)
    all_reduce_ops: List[str] = field(default_factory=list)
    all_to_all_ops: List[str] = field(default_factory=list)
    all_gather_ops: List[str] = field(default_factory=list)
    total_communication_bytes: int = 0
    peak_memory_per_device: int = 0

    def to_string(self) -> str:
        return (f"ShardPlan{{tensors=[{', '.join(s.to_string() for s in self.tensor_shards)}], "
                f"all_reduce_ops=[{', '.join(self.all_reduce_ops)}], "
                f"all_to_all_ops=[{', '.join(self.all_to_all_ops)}], "
                f"all_gather_ops=[{', '.join(self.all_gather_ops)}], "
                f"comm_bytes={self.total_communication_bytes}, peak_mem={self.peak_memory_per_device}}}")


def analyze_matmul(M: int, N: int, K: int, world_size: int, tensor_a: str = "A", tensor_b: str = "B",
                   tensor_c: str = "C", bytes_per_element: int = 2) -> ShardPlan:
    """Plan C = A.B over ``world_size`` devices: A ``SHARD_DIM_0``, B ``REPLICATE``, C computed
    ``SHARD_DIM_0`` and all-gathered (``ShardingAnalyzer::analyze_matmul``, ``sharding.h:107-112``, with
    the row split this path uses instead of the K split the reference's comment describes).

    ``total_communication_bytes`` counts what every device receives: (world-1)/world of C.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    if M % world_size != 0:
        raise ValueError(f"M={M} rows do not split evenly over {world_size} devices")
    m_loc = M // world_size
    bpe = bytes_per_element
    plan = ShardPlan()
    plan.tensor_shards = [
        ShardingSpec(tensor_a, ShardingStrategy.SHARD_DIM_0, [0], [M, K], [m_loc, K]),
        ShardingSpec(tensor_b, ShardingStrategy.REPLICATE, [], [K, N], [K, N]),
        ShardingSpec(tensor_c, ShardingStrategy.SHARD_DIM_0, [0], [M, N], [m_loc, N]),
    ]
    if world_size > 1:
        plan.all_gather_ops = [f"all_gather({tensor_c}, dim=0)"]
        plan.total_communication_bytes = world_size * (world_size - 1) * m_loc * N * bpe
    plan.peak_memory_per_device = (m_loc * K + K * N + M * N) * bpe
    return plan


def owned_row_blocks(M: int, world_size: int, rank: int, chunks: int) -> List[Tuple[int, int]]:
    """``(first_row, row_count)`` of the block of C (and A) that ``rank`` owns in each chunk."""
    if M % (world_size * chunks) != 0:
        raise ValueError(f"M={M} must be a multiple of world_size*chunks={world_size * chunks}")
    blk = M // (world_size * chunks)
    return [(c * (M // chunks) + rank * blk, blk) for c in range(chunks)]


def pick_chunks(M: int, world_size: int, requested: Optional[int] = None) -> int:
    """Largest chunk count <= requested (default 4) that splits the rows evenly into blocks of whole
    128-row tiles; 1 on a single device (nothing to overlap)."""
    if world_size == 1:
        return 1
    want = requested if requested is not None else 4
    for c in range(max(1, want), 0, -1):
        if M % (world_size * c) == 0 and (M // (world_size * c)) % 128 == 0:
            return c
    return 1


class ShardedStepTimeout(RuntimeError):
    """A rank of the group did not enter a sharded step before the deadline."""


def _group_store(group):
    """The key-value store behind a process group (the default group's store for ``None``)."""
    import torch.distributed as dist
    from torch.distributed import distributed_c10d as c10d
    pg = group if group is not None else dist.group.WORLD
    return c10d._get_process_group_store(pg)


class RowShardedGemm:
    """C = act(alpha * A.B + bias) with A row-sharded, B replicated, C all-gathered (bf16; fp32 through the NCCL
    exchange).

    One instance per process; ``__call__`` takes this rank's rows of A (``[M/world, K]``, ordered as
    ``local_row_index()`` says), the full B, and returns the full C on every rank. The all-gather of
    chunk c is issued asynchronously right after chunk c's GEMM and runs on NCCL's stream while chunk
    c+1 computes; the call returns after all chunks have been gathered (stream-ordered, no host sync).
    """

    EXCHANGES = ("peer_store", "multicast", "epilogue_tma", "nccl")
    FUSED = ("peer_store", "multicast", "epilogue_tma")

    def __init__(self, M: int, N: int, K: int, *, group=None, chunks: Optional[int] = None, activation=None,
                 b_layout: int = 0, local_gemm: Optional[Callable] = None, exchange: Optional[str] = None,
                 wait_limit_ms: int = 0, step_deadline_s: Optional[float] = None):
        import torch.distributed as dist
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        if M % self.world != 0:
            raise ValueError(f"M={M} rows do not split evenly over {self.world} ranks")
        self.M, self.N, self.K = M, N, K
        # Default: the fused exchange; a first call with float32 inputs (which the fused kernels do not take)
        # moves a defaulted instance to the NCCL pipeline.
        self._exchange_defaulted = exchange is None
        if exchange is None:
            exchange = "nccl" if (local_gemm is not None or self.world == 1) else "peer_store"
        if exchange not in self.EXCHANGES:
            raise ValueError(f"exchange must be one of {self.EXCHANGES}")
        self.exchange = exchange
        self._requested_chunks = chunks
        if exchange in self.FUSED and chunks is None:
            chunks = 1  # one GEMM launch over all local rows; the exchange rides on the same kernel
        if exchange == "epilogue_tma":
            chunks = 1
        self._symm_out = None
        self._peer_ptrs = None
        self._flag = None
        self._comm = None
        self.wait_limit_ms = wait_limit_ms
        self.step_deadline_s = step_deadline_s
        self._steps = 0
        self.chunks = pick_chunks(M, self.world, chunks)
        self.blocks = owned_row_blocks(M, self.world, self.rank, self.chunks)
        self.activation = activation
        self.b_layout = b_layout
        self.plan = analyze_matmul(M, N, K, self.world)
        # Host-logic tests (gloo, CPU tensors) inject the per-chunk product; the default is the CUDA library.
        self._local_gemm = local_gemm

    def local_row_index(self):
        """Global row numbers of this rank's rows of A / C, in local storage order."""
        import torch
        return torch.cat([torch.arange(s, s + n) for s, n in self.blocks])

    def output_buffer(self, dtype, device):
        """The [M, N] result buffer of the peer-store exchange: symmetric memory, allocated and exchanged
        among the ranks on first use (a collective call), then reused by every ``__call__``."""
        import os

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if self._symm_out is not None and self._symm_out.dtype == dtype:
            return self._symm_out
        # plain peer mappings are all the unicast exchanges need; NVLink multicast objects are created only
        # for exchange="multicast"
        if self.exchange != "multicast":
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        elif os.environ.get("TORCH_SYMM_MEM_DISABLE_MULTICAST") == "1":
            # an earlier unicast instance of this process switched multicast objects off; torch may have latched
            # that at its first symmetric allocation, in which case the check below reports it
            os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "0"
        buf = symm_mem.empty((self.M, self.N), dtype=dtype, device=device)
        flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
        flags.zero_()
        grp = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(buf, grp)
        fhdl = symm_mem.rendezvous(flags, grp)
        self._symm_out = buf
        self._symm_flags = flags
        self._peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._hdl, self._fhdl = hdl, fhdl
        self._flag = torch.zeros(1, device=device, dtype=torch.int32)
        from . import _capi
        comm = _capi.Comm()
        comm.rank, comm.world = self.rank, self.world
        for r in range(self.world):
            comm.c_base[r] = int(hdl.buffer_ptrs[r])
            comm.flags[r] = int(fhdl.buffer_ptrs[r])
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        if self.exchange == "multicast" and mc == 0:
            raise RuntimeError("exchange='multicast' needs an NVLink multicast mapping of C; this box gave none")
        comm.c_multicast = mc if self.exchange == "multicast" else None
        comm.epoch = 0
        comm.wait_limit_ms = int(self.wait_limit_ms)
        self._comm = comm
        # One communicator per row chunk: the same ranks and flags, C (and its multicast mapping) advanced to the
        # chunk's block of rows. The call counter is shared (see _call_fused).
        self._chunk_comms = []
        blk_bytes = (self.M // self.chunks) * self.N * buf.element_size()
        for c in range(self.chunks):
            cc = _capi.Comm()
            cc.rank, cc.world = self.rank, self.world
            for r in range(self.world):
                cc.c_base[r] = int(hdl.buffer_ptrs[r]) + c * blk_bytes
                cc.flags[r] = int(fhdl.buffer_ptrs[r])
            cc.c_multicast = (mc + c * blk_bytes) if self.exchange == "multicast" else None
            cc.wait_limit_ms = int(self.wait_limit_ms)
            self._chunk_comms.append(cc)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anybody's kernel writes one
        return buf

    def _barrier(self):
        """Stream-ordered barrier over the group (a one-element all-reduce)."""
        import torch.distributed as dist
        dist.all_reduce(self._flag, group=self.group)

    def _call_fused(self, A_local, B, bias, out_dtype):
        """One kernel per rank (and row chunk) computes and gathers (``symplex_b200_sharded_gemm``)."""
        from . import gemm
        out = self.output_buffer(out_dtype, A_local.device)
        if self.exchange == "epilogue_tma":
            row0, nrows = self.blocks[0]
            elt = out.element_size()
            mine = out[row0:row0 + nrows]
            peers = [p + row0 * self.N * elt for r, p in enumerate(self._peer_ptrs) if r != self.rank]
            self._barrier()  # every rank has finished with the previous contents of C
            gemm(A_local, B, bias=bias, activation=self.activation, out=mine, b_layout=self.b_layout,
                 peer_outputs=peers)
            self._barrier()  # every rank's tiles have been written everywhere
            return out
        A_local = A_local.contiguous()
        B = B.contiguous()
        blk = (self.M // self.world) // self.chunks
        for c in range(self.chunks):
            self.run_chunk(c, A_local[c * blk:(c + 1) * blk], B, bias, out_dtype)
        return out

    def run_chunk(self, c, A_blk, B, bias=None, out_dtype=None, stream=None):
        """Chunk ``c`` of a fused step: one ``symplex_b200_sharded_gemm`` call (GEMM + exchange in one kernel) over
        this rank's ``M / (world * chunks)`` rows of the chunk, whose result lands, on every rank, in rows
        ``c * M / chunks + rank * M / (world * chunks) + ...`` of ``output_buffer()``. Collective: every rank runs
        the chunks in the same order. A caller that stages A chunk by chunk (host buffers) calls this directly."""
        import ctypes

        import torch

        from . import _capi, make_desc
        if self.exchange not in ("peer_store", "multicast") or self.world == 1:
            raise ValueError("run_chunk() belongs to the exchanges that run inside the GEMM kernel")
        if out_dtype is None:
            out_dtype = self._symm_out.dtype if self._symm_out is not None else A_blk.dtype
        self.output_buffer(out_dtype, A_blk.device)
        if A_blk.dtype != torch.bfloat16 or B.dtype != torch.bfloat16:
            raise ValueError("the fused exchanges take bfloat16 inputs; use exchange='nccl' for float32")
        key = (out_dtype, self.activation, self.b_layout)
        if getattr(self, "_desc_key", None) != key:
            self._desc = make_desc(self.M // self.chunks, self.N, self.K, _capi.DT_BF16,
                                   _capi.DT_F32 if out_dtype == torch.float32 else _capi.DT_BF16,
                                   b_layout=self.b_layout, activation=self.activation)
            self._desc_key = key
        mode = _capi.XCHG_MULTICAST if self.exchange == "multicast" else _capi.XCHG_UNICAST
        s = stream if stream is not None else torch.cuda.current_stream(A_blk.device).cuda_stream
        cc = self._chunk_comms[c]
        cc.epoch = self._comm.epoch  # one call counter for all chunks: the flags are shared
        rc = _capi.load().symplex_b200_sharded_gemm(
            ctypes.byref(self._desc), A_blk.data_ptr(), B.data_ptr(), bias.data_ptr() if bias is not None else None,
            ctypes.byref(cc), mode, s)
        self._comm.epoch = cc.epoch
        _capi.check(rc)

    def _host_handshake(self):
        """Before a step is launched, every rank posts its step number in the process group's store and waits,
        with a deadline, until all ranks have posted it. A rank that never enters the step (it raised, hung on
        the host, or exited) is noticed HERE, on the host, as a ``ShardedStepTimeout`` - not as a collective
        that blocks for ever. Enabled by ``step_deadline_s``."""
        import time

        import torch.distributed as dist
        self._steps += 1
        if self.step_deadline_s is None or self.world == 1:
            return
        store = _group_store(self.group)
        key = f"symplex_b200/row_sharded_gemm/{id(self.group) if self.group is not None else 0}/step{self._steps}"
        store.add(key, 1)
        deadline = time.monotonic() + float(self.step_deadline_s)
        while True:
            if store.add(key, 0) >= self.world:
                return
            if time.monotonic() > deadline:
                raise ShardedStepTimeout(
                    f"rank {self.rank}: only {store.add(key, 0)} of {self.world} ranks entered step {self._steps} "
                    f"within {self.step_deadline_s} s")
            time.sleep(0.002)

    def _gemm_chunk(self, A_blk, B, bias, out_blk):
        if self._local_gemm is not None:
            self._local_gemm(A_blk, B, bias, out_blk)
            return
        from . import gemm
        gemm(A_blk, B, bias=bias, activation=self.activation, out=out_blk, b_layout=self.b_layout)

    def __call__(self, A_local, B, *, bias=None, out=None, out_dtype=None):
        import torch
        import torch.distributed as dist
        m_loc = self.M // self.world
        if tuple(A_local.shape) != (m_loc, self.K):
            raise ValueError(f"A_local must be [{m_loc}, {self.K}], got {tuple(A_local.shape)}")
        if (self._exchange_defaulted and self.exchange in self.FUSED and self.world > 1
                and A_local.dtype != torch.bfloat16):
            self.exchange = "nccl"
            self.chunks = pick_chunks(self.M, self.world, self._requested_chunks)
            self.blocks = owned_row_blocks(self.M, self.world, self.rank, self.chunks)
        self._host_handshake()
        if self.exchange in self.FUSED and self.world > 1:
            dt = out.dtype if out is not None else (out_dtype if out_dtype is not None else A_local.dtype)
            if out is not None and (self._symm_out is None or out.data_ptr() != self._symm_out.data_ptr()):
                raise ValueError("with a fused exchange the result lives in output_buffer(); pass out=None "
                                 "or that buffer")
            return self._call_fused(A_local, B, bias, dt)
        if out is None:
            dt = out_dtype if out_dtype is not None else A_local.dtype
            out = torch.empty((self.M, self.N), device=A_local.device, dtype=dt)
        elif tuple(out.shape) != (self.M, self.N) or not out.is_contiguous():
            raise ValueError(f"out must be a contiguous [{self.M}, {self.N}] tensor")
        blk = m_loc // self.chunks
        chunk_rows = self.M // self.chunks
        works = []
        for c, (row0, nrows) in enumerate(self.blocks):
            mine = out[row0:row0 + nrows]
            self._gemm_chunk(A_local[c * blk:(c + 1) * blk], B, bias, mine)
            if self.world > 1:
                whole = out[c * chunk_rows:(c + 1) * chunk_rows]
                # in place: this rank's block already sits at its slot of the gathered chunk
                works.append(dist.all_gather_into_tensor(whole, mine, group=self.group, async_op=True))
        for w in works:
            w.wait()  # makes the current stream wait for the collective; does not block the host on NCCL
        return out
