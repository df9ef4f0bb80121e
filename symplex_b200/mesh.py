"""Device mesh and communication schedule vocabulary of the reference's distributed headers, for the one plan
this library executes (rows of A and C sharded over the GPUs of one NVLink domain, C all-gathered).

* ``MeshDimension`` / ``DeviceDescriptor`` / ``ClusterMesh`` — ``include/symplex/distributed/mesh.h:17-160``
  (row-major linearisation of mesh coordinates, submeshes, device health; ``create_2d_mesh`` lays the mesh out as
  ``[dp, pp, tp]`` with 8 GPUs per node)
* ``CommOp`` / ``CommunicationSchedule`` / ``NCCLBridge`` — ``include/symplex/distributed/nccl_bridge.h:19-119``
  (the reference declares these without an implementation; the latency model here uses the figures measured for
  this library's exchange instead of the header's 600 / 100 GB/s constants)

Pure host code: nothing here touches a GPU. The executed counterpart is ``sharding.RowShardedGemm``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

from .sharding import CollectiveOp, ShardPlan

GPUS_PER_NODE = 8


@dataclass
class MeshDimension:
    name: str = ""
    size: int = 0

    def to_string(self) -> str:
        return f"{self.name}={self.size}"


@dataclass
class DeviceDescriptor:
    global_id: int = -1
    local_id: int = -1   # within its node
    node_id: int = -1
    mesh_coord: List[int] = field(default_factory=list)
    hostname: str = ""
    gpu_id: int = -1
    alive: bool = True

    def to_string(self) -> str:
        coord = "(" + ", ".join(map(str, self.mesh_coord)) + ")"
        return (f"Device{{gid={self.global_id}, lid={self.local_id}, node={self.node_id}, gpu={self.gpu_id}, "
                f"coord={coord}, alive={'yes' if self.alive else 'no'}}}")


class ClusterMesh:
    """An n-dimensional grid of devices; the last dimension varies fastest."""

    def __init__(self, dims: Sequence[MeshDimension] = (), devices: Sequence[DeviceDescriptor] = ()):
        self._dims = list(dims)
        self._devices = list(devices)
        total = 1
        for d in self._dims:
            if d.size <= 0:
                raise ValueError(f"mesh dimension {d.name!r} has size {d.size}")
            total *= d.size
        if self._dims and len(self._devices) != total:
            raise ValueError(f"mesh of {total} slots got {len(self._devices)} devices")

    # -- accessors
    def ndim(self) -> int:
        return len(self._dims)

    def size(self, dim: int) -> int:
        return self._dims[dim].size

    def total_devices(self) -> int:
        return len(self._devices)

    def dimensions(self) -> List[MeshDimension]:
        return list(self._dims)

    def devices(self) -> List[DeviceDescriptor]:
        return list(self._devices)

    # -- coordinates
    def coord_to_linear(self, coord: Sequence[int]) -> int:
        if len(coord) != len(self._dims):
            raise ValueError("coordinate rank does not match the mesh")
        idx = 0
        for c, d in zip(coord, self._dims):
            if not 0 <= c < d.size:
                raise IndexError(f"coordinate {tuple(coord)} outside the mesh")
            idx = idx * d.size + c
        return idx

    def linear_to_coord(self, linear_id: int) -> List[int]:
        if not 0 <= linear_id < len(self._devices):
            raise IndexError(f"device {linear_id} outside the mesh")
        coord = []
        for d in reversed(self._dims):
            coord.append(linear_id % d.size)
            linear_id //= d.size
        return coord[::-1]

    def device_at(self, coord: Sequence[int]) -> DeviceDescriptor:
        return self._devices[self.coord_to_linear(coord)]

    def devices_along(self, dim: int, fixed: Sequence[int]) -> List[DeviceDescriptor]:
        out = []
        for i in range(self._dims[dim].size):
            c = list(fixed)
            c[dim] = i
            out.append(self.device_at(c))
        return out

    def submesh(self, dim: int, start: int, end: int) -> "ClusterMesh":
        if not 0 <= start < end <= self._dims[dim].size:
            raise ValueError("bad submesh range")
        dims = [MeshDimension(d.name, d.size) for d in self._dims]
        dims[dim].size = end - start
        devices = []
        for dev in self._devices:
            if start <= dev.mesh_coord[dim] < end:
                coord = list(dev.mesh_coord)
                coord[dim] -= start
                devices.append(DeviceDescriptor(dev.global_id, dev.local_id, dev.node_id, coord, dev.hostname,
                                                dev.gpu_id, dev.alive))
        return ClusterMesh(dims, devices)

    # -- health
    def mark_device_dead(self, global_id: int) -> None:
        for d in self._devices:
            if d.global_id == global_id:
                d.alive = False

    def mark_device_alive(self, global_id: int) -> None:
        for d in self._devices:
            if d.global_id == global_id:
                d.alive = True

    def num_alive_devices(self) -> int:
        return sum(1 for d in self._devices if d.alive)

    def dead_device_ids(self) -> List[int]:
        return [d.global_id for d in self._devices if not d.alive]

    def to_string(self) -> str:
        return ("ClusterMesh{dims=[" + ", ".join(d.to_string() for d in self._dims) +
                f"], devices={len(self._devices)}, alive={self.num_alive_devices()}}}")

    # -- factories
    @staticmethod
    def create_2d_mesh(tp_size: int, pp_size: int, dp_size: int) -> "ClusterMesh":
        """``[dp, pp, tp]`` mesh (``mesh.h:150-156``): tensor-parallel neighbours are consecutive GPUs of a node."""
        dims = [MeshDimension("data_parallel", dp_size), MeshDimension("pipeline_parallel", pp_size),
                MeshDimension("tensor_parallel", tp_size)]
        devices = []
        gid = 0
        for d in range(dp_size):
            for p in range(pp_size):
                for t in range(tp_size):
                    devices.append(DeviceDescriptor(gid, gid % GPUS_PER_NODE, gid // GPUS_PER_NODE, [d, p, t],
                                                    f"node{gid // GPUS_PER_NODE}", gid % GPUS_PER_NODE))
                    gid += 1
        return ClusterMesh(dims, devices)

    @staticmethod
    def single_node(world_size: int) -> "ClusterMesh":
        """The mesh this library runs on: ``world_size`` GPUs of one NVSwitch domain, one process each."""
        return ClusterMesh.create_2d_mesh(world_size, 1, 1)


@dataclass
class CommOp:
    op: CollectiveOp
    bytes: int
    src_devices: List[int]
    dst_devices: List[int]
    tensor_name: str
    asynchronous: bool   # can it overlap with computation? (`async` in the reference)

    def to_string(self) -> str:
        return (f"CommOp{{op={self.op.name}, bytes={self.bytes}, tensor='{self.tensor_name}', "
                f"src=[{','.join(map(str, self.src_devices))}], dst=[{','.join(map(str, self.dst_devices))}], "
                f"async={'yes' if self.asynchronous else 'no'}}}")


@dataclass
class CommunicationSchedule:
    operations: List[CommOp] = field(default_factory=list)
    total_sync_bytes: int = 0
    total_async_bytes: int = 0

    def to_string(self) -> str:
        return ("CommunicationSchedule{ops=[" + ", ".join(o.to_string() for o in self.operations) +
                f"], sync_bytes={self.total_sync_bytes}, async_bytes={self.total_async_bytes}}}")


class NCCLBridge:
    """Turns a ``ShardPlan`` into the collectives it needs and estimates their cost on this library's hardware.

    Bandwidths per GPU and direction, measured on B200 / NVLink 5 through NVSwitch: 650 GB/s for the peer stores the
    fused GEMM epilogue issues, 296 GB/s for NCCL's all-gather at these sizes; 50 GB/s assumed between nodes (not
    measured: this library runs inside one node)."""

    PEER_STORE_GBPS = 650.0
    NCCL_ALL_GATHER_GBPS = 296.0
    INTER_NODE_GBPS = 50.0
    INTRA_NODE_LATENCY_NS = 2000.0    # two stream-ordered one-element all-reduces bracket the fused exchange
    INTER_NODE_LATENCY_NS = 10000.0

    def __init__(self, mesh: ClusterMesh, exchange: str = "peer_store"):
        if exchange not in ("peer_store", "nccl"):
            raise ValueError("exchange must be 'peer_store' or 'nccl'")
        self.mesh = mesh
        self.exchange = exchange

    def is_available(self) -> bool:
        try:
            import torch.distributed as dist
            return bool(dist.is_available() and dist.is_nccl_available())
        except Exception:
            return False

    def _same_node(self, devices: Sequence[int]) -> bool:
        nodes = {self.mesh.devices()[d].node_id for d in devices}
        return len(nodes) <= 1

    def generate_schedule(self, plan: ShardPlan) -> CommunicationSchedule:
        """One ``CommOp`` per collective the plan names. ``bytes`` is what ONE device sends (= receives) for it.
        The all-gather of the row-sharded GEMM overlaps the GEMM (it is issued from the kernel's epilogue, or per
        chunk behind the next chunk's GEMM), so it counts as asynchronous; all-reduces and all-to-alls would not."""
        ids = [d.global_id for d in self.mesh.devices() if d.alive]
        world = max(1, len(ids))
        sched = CommunicationSchedule()
        per_device = plan.total_communication_bytes // world if world > 1 else 0
        named = ([(CollectiveOp.ALL_GATHER, s, True) for s in plan.all_gather_ops] +
                 [(CollectiveOp.ALL_REDUCE, s, False) for s in plan.all_reduce_ops] +
                 [(CollectiveOp.ALL_TO_ALL, s, False) for s in plan.all_to_all_ops])
        for op, label, overlaps in named:
            nbytes = per_device // max(1, len(named))
            tensor = label[label.find("(") + 1:].split(",")[0].rstrip(")") if "(" in label else label
            sched.operations.append(CommOp(op, nbytes, list(ids), list(ids), tensor, overlaps))
            if overlaps:
                sched.total_async_bytes += nbytes
            else:
                sched.total_sync_bytes += nbytes
        return sched

    @staticmethod
    def nccl_op_name(op: CollectiveOp) -> str:
        return {CollectiveOp.ALL_REDUCE: "ncclAllReduce", CollectiveOp.ALL_GATHER: "ncclAllGather",
                CollectiveOp.REDUCE_SCATTER: "ncclReduceScatter", CollectiveOp.ALL_TO_ALL: "ncclAllToAll",
                CollectiveOp.BROADCAST: "ncclBroadcast", CollectiveOp.SEND_RECV: "ncclSend/ncclRecv"}[op]

    def emit_nccl_ops(self, schedule: CommunicationSchedule) -> str:
        """The calls a plain NCCL implementation of the schedule would make, one per line (text, like the
        reference's; this library's default exchange does not call NCCL for the all-gather at all)."""
        lines = []
        for o in schedule.operations:
            lines.append(f"{self.nccl_op_name(o.op)}({o.tensor_name}, bytes={o.bytes}, ranks={len(o.dst_devices)}, "
                         f"{'async' if o.asynchronous else 'sync'});")
        return "\n".join(lines)

    def estimate_communication_latency_ns(self, schedule: CommunicationSchedule) -> float:
        total = 0.0
        for o in schedule.operations:
            if len(o.dst_devices) <= 1 or o.bytes == 0:
                continue
            if self._same_node(o.dst_devices):
                gbps = self.PEER_STORE_GBPS if (self.exchange == "peer_store" and o.op == CollectiveOp.ALL_GATHER) \
                    else self.NCCL_ALL_GATHER_GBPS
                total += self.INTRA_NODE_LATENCY_NS + o.bytes / gbps
            else:
                total += self.INTER_NODE_LATENCY_NS + o.bytes / self.INTER_NODE_GBPS
        return total
