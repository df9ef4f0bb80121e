"""Mesh and communication-schedule vocabulary (host only). Known answers from the reference's own test
(tests/test_distributed.cpp:19-57): create_2d_mesh(4, 2, 8) has 64 devices in 3 dimensions; a 2 x 2 x 2 mesh has 8
alive devices, 7 after mark_device_dead(3), and one dead id; analyze_matmul(4096^3) has shards and traffic."""
import pytest

from symplex_b200 import mesh as M
from symplex_b200.sharding import CollectiveOp, analyze_matmul


def test_reference_known_answers():
    m = M.ClusterMesh.create_2d_mesh(4, 2, 8)
    assert m.total_devices() == 64 and m.ndim() == 3
    assert [d.size for d in m.dimensions()] == [8, 2, 4]
    h = M.ClusterMesh.create_2d_mesh(2, 2, 2)
    assert h.num_alive_devices() == 8
    h.mark_device_dead(3)
    assert h.num_alive_devices() == 7 and h.dead_device_ids() == [3]
    h.mark_device_alive(3)
    assert h.num_alive_devices() == 8
    plan = analyze_matmul(4096, 4096, 4096, world_size=8)
    assert plan.tensor_shards and plan.total_communication_bytes > 0


def test_coordinates_and_submesh():
    m = M.ClusterMesh.create_2d_mesh(4, 2, 3)   # dims [dp 3, pp 2, tp 4]
    for gid in range(m.total_devices()):
        c = m.linear_to_coord(gid)
        assert m.coord_to_linear(c) == gid and m.device_at(c).global_id == gid
    assert m.linear_to_coord(23) == [2, 1, 3] and m.coord_to_linear([1, 0, 2]) == 10
    tp = m.devices_along(2, [1, 1, 0])
    assert [d.global_id for d in tp] == [12, 13, 14, 15]            # tensor-parallel neighbours are consecutive
    assert m.device_at([1, 1, 0]).node_id == 1 and m.device_at([1, 1, 0]).local_id == 4
    sub = m.submesh(0, 1, 3)
    assert sub.total_devices() == 16 and sub.size(0) == 2 and sub.device_at([0, 0, 0]).global_id == 8
    with pytest.raises(IndexError):
        m.coord_to_linear([3, 0, 0])
    with pytest.raises(ValueError):
        M.ClusterMesh([M.MeshDimension("x", 2)], [])
    assert "alive=24" in m.to_string()


def test_schedule_for_the_row_sharded_gemm():
    world, Mrows, N, K = 8, 65536, 8192, 8192
    mesh = M.ClusterMesh.single_node(world)
    plan = analyze_matmul(Mrows, N, K, world_size=world, bytes_per_element=2)
    bridge = M.NCCLBridge(mesh)
    sched = bridge.generate_schedule(plan)
    assert len(sched.operations) == 1
    op = sched.operations[0]
    assert op.op == CollectiveOp.ALL_GATHER and op.tensor_name == "C" and op.asynchronous
    assert op.bytes == (world - 1) * (Mrows // world) * N * 2           # 0.94 GB per GPU
    assert sched.total_async_bytes == op.bytes and sched.total_sync_bytes == 0
    assert op.src_devices == list(range(8)) == op.dst_devices
    assert bridge.emit_nccl_ops(sched).startswith("ncclAllGather(C, bytes=939524096, ranks=8, async);")
    t_peer = bridge.estimate_communication_latency_ns(sched)
    t_nccl = M.NCCLBridge(mesh, "nccl").estimate_communication_latency_ns(sched)
    assert 1.40e6 < t_peer < 1.50e6 and t_nccl > 2 * t_peer              # 0.94 GB at 650 GB/s = 1.45 ms
    # one GPU: nothing to exchange
    solo = M.NCCLBridge(M.ClusterMesh.single_node(1)).generate_schedule(analyze_matmul(1024, 64, 64, world_size=1))
    assert solo.operations == [] and M.NCCLBridge(mesh).estimate_communication_latency_ns(solo) == 0.0
    # a dead device drops out of the schedule's rank list
    mesh.mark_device_dead(5)
    assert 5 not in M.NCCLBridge(mesh).generate_schedule(plan).operations[0].dst_devices
    with pytest.raises(ValueError):
        M.NCCLBridge(mesh, "carrier pigeon")


def test_commop_strings():
    op = M.CommOp(CollectiveOp.ALL_GATHER, 128, [0, 1], [0, 1], "C", True)
    assert op.to_string() == "CommOp{op=ALL_GATHER, bytes=128, tensor='C', src=[0,1], dst=[0,1], async=yes}"
    s = M.CommunicationSchedule([op], 0, 128)
    assert s.to_string().endswith("sync_bytes=0, async_bytes=128}")
    assert M.NCCLBridge.nccl_op_name(CollectiveOp.REDUCE_SCATTER) == "ncclReduceScatter"
