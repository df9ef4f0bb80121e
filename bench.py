#!/usr/bin/env python
"""Benchmark of the GEMM hot path: `python bench.py --gpus N --steps K --warmup W [--impl reference]`.

Default workload: the row-sharded bf16 GEMM A[65536,8192] x B[8192,8192] -> bf16 C, rows of A split evenly
over the N GPUs, C all-gathered over NVLink inside the GEMM kernel (N = 1: the same GEMM on one GPU, no
exchange). Total work is fixed as N grows ("scaling": "strong"). One step = one full product.

Prints ONE JSON line (rank 0). `value` is device-resident throughput (inputs in HBM, CUDA events, max over
ranks); `e2e` is the same product through the host-buffer entry points with the pinned-host -> device and
device -> host copies inside the timed region. `roofline` describes the GEMM kernel alone (plus an `nvlink`
block for the exchange at N > 1), `cpu_baseline` the reference's CPU path timed on this box's host cores on a
bounded row sample (`cpu_baseline.all`: the x86-JIT order, the BLIS order, the reference's C kernel and np.matmul).
`parity_check` is a float64 check of the finished product on every rank; the exit code is 3 if it fails.
On one GPU the default run appends `secondary`: short runs of the other GEMM workloads under the same timing rules.
`config` names the workload (the same keys in both arms); how this arm ran it is in `detail`.

`--impl reference` times the reference's own CPU implementation of the path instead (its C kernel compiled
unchanged when available, else the oracle port), on a bounded row sample of the same workload per step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, N, K, batch, in, out, b_layout, activation, bias, description)
    "cfg5_row_sharded_bf16_65536x8192x8192": dict(M=65536, N=8192, K=8192, batch=1, dt="bf16", out="bf16", b_col=False,
                                                  act=None, bias=False, sharded=True),
    "headline_bf16_8192_cube_bias_gelu": dict(M=8192, N=8192, K=8192, batch=1, dt="bf16", out="bf16", b_col=False,
                                              act="gelu", bias=True, sharded=False),
    "cfg1_fp32_512_cube": dict(M=512, N=512, K=512, batch=1, dt="f32", out="f32", b_col=False, act=None, bias=False,
                               sharded=False),
    "cfg2_bf16_4096_cube_colmajor_b": dict(M=4096, N=4096, K=4096, batch=1, dt="bf16", out="f32", b_col=True, act=None,
                                           bias=False, sharded=False),
    "cfg2_fp32_4096_cube_colmajor_b": dict(M=4096, N=4096, K=4096, batch=1, dt="f32", out="f32", b_col=True, act=None,
                                           bias=False, sharded=False),
    "cfg3_fused_gelu_mlp_8192x4096x16384": dict(M=8192, N=16384, K=4096, batch=1, dt="bf16", out="bf16", b_col=False,
                                                act="gelu", bias=True, sharded=False),
    "cfg4_batched_fp32_2048x64_cube": dict(M=64, N=64, K=64, batch=2048, dt="f32", out="f32", b_col=False, act=None,
                                           bias=False, sharded=False),
    # Workloads that reach the kernels the ones above do not (for profiling and for the record; not in `secondary`):
    # the single-CTA bf16 kernel (what small and narrow problems run), the 256 x 256 CTA-pair tile, the fp32
    # pre-pass with a transposing split (row-major B), bf16 operands whose rows are not 16-byte multiples (padded
    # copies first), and the f64 product behind blas_dgemm.
    "aux_bf16_2048_cube_single_cta_tiles": dict(M=2048, N=2048, K=2048, batch=1, dt="bf16", out="bf16", b_col=False,
                                                act=None, bias=False, sharded=False, options={"pair_mode": 0}),
    "aux_bf16_2048_cube_pair_256x256_tiles": dict(M=2048, N=2048, K=2048, batch=1, dt="bf16", out="bf16", b_col=False,
                                                  act=None, bias=False, sharded=False, options={"pair_mode": 1}),
    "aux_fp32_4096_cube_rowmajor_b": dict(M=4096, N=4096, K=4096, batch=1, dt="f32", out="f32", b_col=False, act=None,
                                          bias=False, sharded=False),
    "aux_bf16_4096x4096x4100_unaligned_rows": dict(M=4096, N=4096, K=4100, batch=1, dt="bf16", out="bf16", b_col=True,
                                                   act=None, bias=False, sharded=False),
    # 304 tiles of 512 x 256 on 74 CTA pairs are 4.11 waves. First entry: stream-K (the pairs share the k-blocks of
    # all tiles evenly; an option, off by default); second: the same tiles whole, five waves, what the option replaces.
    "aux_bf16_8192x4864x8192_stream_k": dict(M=8192, N=4864, K=8192, batch=1, dt="bf16", out="bf16", b_col=False,
                                             act=None, bias=False, sharded=False,
                                             options={"stream_k": 1, "pair_mode": 2}),
    "aux_bf16_8192x4864x8192_whole_512x256_tiles": dict(M=8192, N=4864, K=8192, batch=1, dt="bf16", out="bf16",
                                                        b_col=False, act=None, bias=False, sharded=False,
                                                        options={"stream_k": 0, "pair_mode": 2}),
    # The smallest shape of that kind, used for the ncu capture: 162 tiles = 2.19 waves.
    "aux_bf16_4608x4608x4096_stream_k": dict(M=4608, N=4608, K=4096, batch=1, dt="bf16", out="bf16", b_col=False,
                                             act=None, bias=False, sharded=False,
                                             options={"stream_k": 1, "pair_mode": 2}),
    "aux_f64_2048_cube": dict(M=2048, N=2048, K=2048, batch=1, dt="f64", out="f64", b_col=False, act=None, bias=False,
                              sharded=False),
    # The kernel of the row-sharded product (GEMM + forwarder warps) on ONE GPU: rank 0 of 4, whose three "peers" are
    # buffers in this GPU's own memory and whose flags are preset, so the one kernel never waits for another. Same
    # tiles, same forwarder traffic (3 x 256 MiB of stores per step) as one rank of a 4-GPU run, without NVLink.
    "aux_bf16_sharded_kernel_rank0_of_4_local_peers": dict(M=16384, N=8192, K=8192, batch=1, dt="bf16", out="bf16",
                                                           b_col=False, act=None, bias=False, sharded=False,
                                                           emulate_ranks=4),
    # One rank of 8: 8192 local rows, seven destinations - the link-bound case, which takes the 256 x 256 tiles.
    "aux_bf16_sharded_kernel_rank0_of_8_local_peers": dict(M=8192, N=8192, K=8192, batch=1, dt="bf16", out="bf16",
                                                           b_col=False, act=None, bias=False, sharded=False,
                                                           emulate_ranks=8),
}
SECONDARY = ["headline_bf16_8192_cube_bias_gelu", "cfg1_fp32_512_cube", "cfg2_bf16_4096_cube_colmajor_b",
             "cfg2_fp32_4096_cube_colmajor_b", "cfg3_fused_gelu_mlp_8192x4096x16384", "cfg4_batched_fp32_2048x64_cube"]
DEFAULT_WORKLOAD = "cfg5_row_sharded_bf16_65536x8192x8192"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (absent where no capture of that workload exists).
#   bf16 pair kernel, 8192 x 8192 x 8192: 882.17 MB read + 119.91 MB written (profiles/gemm_pair_kernel_bf16_8192_cube_bias_gelu.md).
#   Its traffic is proportional to the rows of A per launch (B is re-streamed once per band of 2048 rows, A and C
#   are touched once), so the row-sharded workload scales that capture by rows / 8192.
#   fp32 3xTF32 kernel, 4096^3: 1103.19 MB + 62.13 MB (profiles/gemm_tf32x3_kernel_fp32_4096_cube.md).
NCU_TRAFFIC_PER_8192_ROWS_BF16_N8192_K8192 = 882.17e6 + 119.91e6
NCU_TRAFFIC_BYTES = {
    "headline_bf16_8192_cube_bias_gelu": NCU_TRAFFIC_PER_8192_ROWS_BF16_N8192_K8192,
    "cfg2_fp32_4096_cube_colmajor_b": 1103.19e6 + 62.13e6,
    # small-row fp32 kernel, 2048 x 64^3: 67.21 MB read + 6.10 MB written (most of C is still in L2 at the end)
    "cfg4_batched_fp32_2048x64_cube": 67.21e6 + 6.10e6,
    # fused fp32 kernel, 512^3 with split-K: 2.18 MB read (A and B once), C stays in L2
    "cfg1_fp32_512_cube": 2.18e6,
    # fused elementwise ring kernel: 800.09 MB read (+ 4.09 MB of earlier dirty lines written back);
    # 805.38 MB read + 240.92 MB written (the last 27 MB of dst are still in L2 when the kernel ends)
    "f3_fused_axpb_sum_200M": 800.09e6 + 4.09e6,
    "f3_fused_mul_add_relu_64M": 805.38e6 + 240.92e6,
}

# Fused elementwise chains (single HBM pass; not GEMMs): (op, lhs_src, lhs_idx, rhs_src, rhs_idx) programs of the
# reference's FusedOpDesc form. "axpb_sum" is the chain the reference's own comment uses as its example
# (x * 2.0 + 1.0 -> sum over an 800 MB array).
ELEMENTWISE_WORKLOADS = {
    "f3_fused_axpb_sum_200M": dict(n=200_000_000, n_inputs=1, ops=[(2, 0, 0, 1, 0), (0, 2, 0, 1, 1)],
                                   consts=[2.0, 1.0], reduce_op=0, desc="sum(x * 2.0 + 1.0)"),
    "f3_fused_mul_add_relu_64M": dict(n=64 << 20, n_inputs=3, ops=[(2, 0, 0, 0, 1), (0, 2, 0, 0, 2), (15, 2, 1, 0, 0)],
                                      consts=[], reduce_op=255, desc="dst = relu(a * b + c)"),
    "f3_fused_axpb_store_128M": dict(n=128 << 20, n_inputs=1, ops=[(2, 0, 0, 1, 0), (0, 2, 0, 1, 1)], consts=[2.0, 1.0],
                                     reduce_op=255, desc="dst = x * 2.0 + 1.0"),
    # the f64 twin (what the reference's Python layer calls for float64 NumPy arrays)
    "f3_fused_axpb_f64_64M": dict(n=64 << 20, n_inputs=1, ops=[(2, 0, 0, 1, 0), (0, 2, 0, 1, 1)], consts=[2.0, 1.0],
                                  reduce_op=255, desc="dst = x * 2.0 + 1.0 (float64)", f64=True),
    # arrays that all start 4 bytes off a 16-byte boundary (x[1:] of aligned arrays): the bulk-copy ring from the next
    # boundary on, the element in front of it by the ring kernel's scalar path
    "f3_fused_axpb_store_unaligned_64M": dict(n=64 << 20, n_inputs=1, ops=[(2, 0, 0, 1, 0), (0, 2, 0, 1, 1)],
                                              consts=[2.0, 1.0], reduce_op=255, desc="dst = x * 2.0 + 1.0, unaligned arrays",
                                              misalign=1),
    # source 4 bytes and destination 8 bytes off: no common boundary, the plain-load kernel
    "f3_fused_axpb_store_mixed_offsets_64M": dict(n=64 << 20, n_inputs=1, ops=[(2, 0, 0, 1, 0), (0, 2, 0, 1, 1)],
                                                  consts=[2.0, 1.0], reduce_op=255,
                                                  desc="dst = x * 2.0 + 1.0, source and destination misaligned differently",
                                                  misalign=1, misalign_out=2),
}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "of measured"
    return dict(FALLBACK_PEAKS), "of fallback"


def flops_of(w):
    return 2.0 * w["M"] * w["N"] * w["K"] * w["batch"]


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # "under load" = samples in the upper half of the observed power range
        lo, hi = min(power), max(power)
        loaded = [s for s, p in zip(sm, power) if p >= lo + 0.5 * (hi - lo)] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": hi}


# ----------------------------------------------------------------------------- CPU reference timing
def _host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def _parts(cores, M, N, K):
    """Row blocks a CPU matmul is split into: one per thread, but none smaller than ~20 MFLOP (a hand-off to a
    thread costs more than a 64^3 product)."""
    return int(max(1, min(cores, M, 2.0 * M * N * K // 2e7)))


def _load_cpu_reference():
    """(callable(A, B, C, M, N, K), kind, cores, name): the reference's CPU matmul for this path.

    Rows of A are split into one contiguous block per host thread and every block runs the reference's kernel
    on its own rows of C, which is how the reference's rayon entry points spread a matmul over the cores
    (rust-engine/src/x86_emitter.rs:1877-1897 `parallel_matmul`, :1845-1875 `parallel_cache_blocked_matmul`);
    the per-element arithmetic of a row does not depend on the split.
    """
    from concurrent.futures import ThreadPoolExecutor
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle_loader import load_oracle, load_ref_kernels
    cores = _host_threads()
    ref = load_ref_kernels()
    if ref is not None:
        pool = ThreadPoolExecutor(max_workers=cores) if cores > 1 else None

        def rows(A, B, C, r0, r1, N, K):
            ref.symplex_matmul_f32(A.ctypes.data + r0 * K * 4, B.ctypes.data, C.ctypes.data + r0 * N * 4, r1 - r0, N, K)

        def run(A, B, C, M, N, K):
            parts = _parts(cores, M, N, K)
            if pool is None or parts <= 1:
                return rows(A, B, C, 0, M, N, K)
            cuts = [M * i // parts for i in range(parts + 1)]
            for f in [pool.submit(rows, A, B, C, cuts[i], cuts[i + 1], N, K) for i in range(parts)]:
                f.result()
        return run, "reference", cores, (f"kernels/matmul.c:symplex_matmul_f32 compiled unchanged, one row block per "
                                         f"thread on up to {cores} threads (the reference's rayon row split)")
    orc = load_oracle()

    def run(A, B, C, M, N, K):
        orc.lib.oracle_jit_parallel_matmul(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, N, K,
                                           _parts(cores, M, N, K))
    return run, "port", cores, f"oracle port of jit_parallel_matmul, row blocks on up to {cores} threads"


def cpu_step_seconds(args):
    """Seconds of CPU work one step of the CPU arm is sized for: a row sample of up to ~3 s, shrunk so that all of the
    arm's steps end within about a minute. Both arms size their sample with this, so they time the same rows."""
    return max(0.25, min(3.0, 60.0 / (args.steps + max(1, args.warmup))))


def cpu_sample(w, rows):
    """Seeded operands of a `rows`-row slice of the workload (fp32; bf16 workloads use bf16-rounded values)."""
    import numpy as np
    rng = np.random.default_rng(0)
    M = min(rows, w["M"])
    A = rng.standard_normal((M, w["K"])).astype(np.float32)
    B = rng.standard_normal((w["K"], w["N"])).astype(np.float32)
    if w["dt"] == "bf16":
        import torch
        A = torch.from_numpy(A).to(torch.bfloat16).float().numpy()
        B = torch.from_numpy(B).to(torch.bfloat16).float().numpy()
    return A, B, np.zeros((M, w["N"]), np.float32)


def time_cpu_reference(w, seconds, steps, warmup):
    """Time the reference's CPU matmul on a row sample of workload `w` sized so that one step takes about `seconds`.

    The sample is sized from a calibration pass (two rows per thread) run on this host: the kernel streams all of B
    for every row of A, so its rate with every core busy depends on the box's memory system, not on a per-core guess.
    """
    import numpy as np
    run, kind, cores, name = _load_cpu_reference()
    N, K = w["N"], w["K"]
    rows0 = min(w["M"], max(2 * cores, 8))
    A, B, C = cpu_sample(w, w["M"] if w["M"] * K <= (1 << 24) else max(rows0, min(w["M"], 64 * cores)))
    run(A, B, C, rows0, N, K)  # pages in B and the code
    t0 = time.perf_counter()
    run(A, B, C, rows0, N, K)
    rate = rows0 / max(time.perf_counter() - t0, 1e-6)  # rows per second
    M = int(max(min(cores, w["M"]), min(w["M"], rate * seconds)))
    if M > A.shape[0]:  # more rows than were drawn: repeat them (the kernel's speed does not depend on the values)
        reps = (M + A.shape[0] - 1) // A.shape[0]
        A = np.ascontiguousarray(np.tile(A, (reps, 1))[:M])
        C = np.zeros((M, N), np.float32)
    for _ in range(warmup):
        run(A, B, C, M, N, K)
    t0 = time.perf_counter()
    for _ in range(steps):
        run(A, B, C, M, N, K)
    dt = (time.perf_counter() - t0) / max(1, steps)
    tflops = 2.0 * M * N * K / dt / 1e12
    sample = f"{M} of {w['M']} rows of A (all of B), one problem of {w['batch']}; {name}"
    return tflops, dt, kind, _parts(cores, M, N, K), sample


# ----------------------------------------------------------------------------- main
# ----------------------------------------------------------------------------- fused elementwise workloads
def _elementwise_cpu(w, n_sample, steps, warmup):
    """GB/s of the CPU restatement of the reference's interpreter (oracle port, 1 thread) on n_sample elements."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle_loader import load_oracle
    orc = load_oracle()
    rng = np.random.default_rng(0)
    ndt = np.float64 if w.get("f64") else np.float32
    arrays = [rng.uniform(-1, 1, n_sample).astype(ndt) for _ in range(w["n_inputs"])]
    for _ in range(max(1, warmup)):
        orc.fused_elementwise(w["ops"], arrays, w["consts"], reduce_op=w["reduce_op"], dtype=ndt)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.fused_elementwise(w["ops"], arrays, w["consts"], reduce_op=w["reduce_op"], dtype=ndt)
    dt = (time.perf_counter() - t0) / steps
    streams = w["n_inputs"] + (0 if w["reduce_op"] != 255 else 1)
    sample = (f"{n_sample} of {w['n']} elements, C restatement of the reference's fused_elem_f32_avx2_core "
              "(scalar code, 1 thread; the reference runs the same chain 8 lanes wide on 1 thread)")
    return (8.0 if w.get("f64") else 4.0) * streams * n_sample / dt / 1e9, dt, sample


def main_elementwise(args):
    w = ELEMENTWISE_WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n, reduce = w["n"], w["reduce_op"] != 255
    f64 = bool(w.get("f64"))
    eb = 8 if f64 else 4
    streams = w["n_inputs"] + (0 if reduce else 1)
    algo_bytes = float(eb) * streams * n
    config = {"workload": args.workload, "chain": w["desc"], "elements": n, "inputs": w["n_inputs"],
              "output": "scalar (f64)" if reduce else ("f64 array" if f64 else "f32 array"), "partition": "replicas only",
              "l2": f"arrays of {eb * n / 1e6:.0f} MB each, larger than L2"}
    if args.impl == "reference":
        if rank != 0:
            return 0
        gbs, dt, sample = _elementwise_cpu(w, 16 << 20, args.steps, args.warmup)
        line = {"impl": "reference", "metric": "fused_elementwise_gbps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f64" if f64 else "f32", "data": "synthetic",
                "config": config,
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return 0

    import numpy as np
    import torch
    import torch.distributed as dist

    import symplex_b200 as sx
    from symplex_b200 import _capi, _symplex_core
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks, peak_note = load_peaks()
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    tdt = torch.float64 if f64 else torch.float32
    mis = int(w.get("misalign", 0))  # elements by which every array is shifted off its 16-byte boundary
    arrays = [(torch.rand(n + mis, device=dev, generator=g, dtype=tdt) * 2 - 1)[mis:] for _ in range(w["n_inputs"])]
    mis_out = int(w.get("misalign_out", mis))
    out = None if reduce else torch.empty(n + mis_out, device=dev, dtype=tdt)[mis_out:]

    # Arguments of the C-ABI call are packed once: a step is then one library call = one kernel launch, with
    # a few microseconds of host work (the kernels run 0.1-0.2 ms, so per-step Python work would show).
    lib = _capi.load()
    c_ops = _capi.pack_fused_ops(w["ops"])
    c_ptrs = (ctypes.c_void_p * len(arrays))(*[a.data_ptr() for a in arrays])
    c_consts = ((ctypes.c_double if f64 else ctypes.c_float) * max(len(w["consts"]), 1))(*w["consts"])
    c_fn = lib.symplex_b200_fused_elementwise_f64 if f64 else lib.symplex_b200_fused_elementwise_f32
    res = torch.zeros((), device=dev, dtype=torch.float64) if reduce else out
    stream = torch.cuda.current_stream(dev).cuda_stream

    def step():
        rc = c_fn(c_ops, len(w["ops"]), c_ptrs, len(arrays), c_consts, len(w["consts"]), n, w["reduce_op"],
                  None if reduce else out.data_ptr(), res.data_ptr() if reduce else None, stream)
        if rc != 0:
            raise SystemExit(f"fused elementwise failed: {_capi.last_error()}")
        return res

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = sx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sx.sync_status()
    elapsed_ms = e0.elapsed_time(e1)
    launches = sx.launch_count() - launches0
    if sampler and elapsed_ms < 1500:  # keep the kernel running long enough for nvidia-smi to sample it under load
        t_end = time.perf_counter() + 1.5
        while time.perf_counter() < t_end:
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([elapsed_ms, float(launches)], device=dev, dtype=torch.float64)
    if world > 1:
        tmax, tsum = t.clone(), t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        elapsed_ms, launches = tmax[0].item(), int(tsum[1].item())
    ms_per_step = elapsed_ms / args.steps
    value = algo_bytes * world / (ms_per_step * 1e-3) / 1e9

    # End to end through the reference-shaped host entry point: pinned host arrays in, host array / scalar out.
    e2e = None
    if not args.no_e2e:
        host = [torch.empty(n, dtype=tdt).pin_memory() for _ in range(w["n_inputs"])]
        for h, a in zip(host, arrays):
            h.copy_(a)
        hout = None if reduce else torch.empty(n, dtype=tdt).pin_memory()
        ptrs = [h.data_ptr() for h in host]
        host_fn = _symplex_core.simd_fused_elementwise_f64 if f64 else _symplex_core.simd_fused_elementwise_f32

        def host_step():
            return host_fn(w["ops"], ptrs, w["consts"], n, w["reduce_op"], 0 if reduce else hout.data_ptr())
        host_step()
        reps = max(2, min(args.steps, 5))
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            hv = host_step()
        dt = (time.perf_counter() - t0) / reps
        tt = torch.tensor([dt], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = tt.item()
        e2e = {"value": algo_bytes * world / dt / 1e9, "unit": "GB/s", "ms_per_step": dt * 1e3,
               "h2d_bytes_per_step": eb * n * w["n_inputs"], "d2h_bytes_per_step": 8 if reduce else eb * n,
               "api": f"symplex_simd_fused_elementwise_{'f64' if f64 else 'f32'} (pinned host arrays, chunked "
                      "copy/compute/copy pipeline)"}
        if reduce:
            e2e["result"] = hv
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0
    ach = algo_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": ach, "peak": float(peaks["hbm_gbs"]), "unit": "GB/s",
                "frac": ach / float(peaks["hbm_gbs"]), "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                "kernel_ms": ms_per_step, "peak_kind": f"HBM copy, {peak_note}", "bytes_per_launch": algo_bytes,
                "note": "one step = one launch of " + ("fused_elementwise_plain_kernel" if mis else
                                                         "fused_elementwise_ring_kernel")}
    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        gbs, dt, sample = _elementwise_cpu(w, 16 << 20, steps=3, warmup=1)
        cpu_baseline = {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample}
    line = {"metric": "fused_elementwise_gbps", "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64" if f64 else "f32", "data": "synthetic", "config": config,
            "roofline": roofline,
            "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks}
    if reduce:
        line["result"] = float(res.item())
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def base_config(name, w, gpus):
    """The workload as both arms of the benchmark name it (identical keys and values in either arm)."""
    return {"workload": name, "M": w["M"], "N": w["N"], "K": w["K"], "batch": w["batch"],
            "inputs": w["dt"], "output": w["out"], "b_layout": "col_major" if w["b_col"] else "row_major",
            "epilogue": ("bias+" if w["bias"] else "") + (w["act"] or "none"),
            "partition": f"rows of A over {gpus} GPU(s), B replicated, C all-gathered" if w["sharded"]
            else "replicas only"}


def cpu_baselines(w, seconds_each):
    """The CPU comparators of this path, each timed on its own bounded row sample of workload `w`:
    the x86-JIT order (AVX-512 twin of the size-baked kernel, 1 thread, as the reference runs it), the BLIS order on
    min(ceil(M / 128), cores) threads, the reference's C kernel compiled unchanged (one row block per thread) and
    np.matmul (OpenBLAS, all cores - the comparator the reference's own benchmark uses)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle_loader import load_oracle
    orc = load_oracle()
    cores = _host_threads()
    N, K = w["N"], w["K"]
    out = []

    def timed(fn, rows0, label, kind, threads, par=1):
        """Calibrate on rows0 rows, then time one run sized for ~seconds_each (par: threads the sized run will use
        beyond those of the calibration run)."""
        A, B, C = cpu_sample(w, max(rows0, 8))
        rows0 = min(rows0, A.shape[0])
        fn(A[:rows0], B, C[:rows0], 1 if par > 1 else threads)  # warm: pages, code
        t0 = time.perf_counter()
        fn(A[:rows0], B, C[:rows0], 1 if par > 1 else threads)
        rate = par * rows0 / max(time.perf_counter() - t0, 1e-6)
        M = int(max(rows0, min(w["M"], rate * seconds_each)))
        if M > A.shape[0]:
            reps = (M + A.shape[0] - 1) // A.shape[0]
            A = np.ascontiguousarray(np.tile(A, (reps, 1))[:M])
            C = np.zeros((M, N), np.float32)
        t0 = time.perf_counter()
        fn(A[:M], B, C[:M], threads)
        dt = time.perf_counter() - t0
        out.append({"kind": kind, "name": label, "cores": threads, "value": 2.0 * M * N * K / dt / 1e12,
                    "unit": "TFLOP/s", "sample": f"{M} of {w['M']} rows of A (all of B)"})

    def avx512(A, B, C, threads):
        if orc.lib.oracle_matmul_jit_avx512(A.ctypes.data, B.ctypes.data, C.ctypes.data, A.shape[0], N, K) != 0:
            orc.lib.oracle_matmul_jit_order(A.ctypes.data, B.ctypes.data, C.ctypes.data, A.shape[0], N, K, 1)
    timed(avx512, 2, "x86-JIT order: AVX-512 twin of compile_matmul_avx512 (oracle), single thread as in the reference",
          "port", 1)
    blis_threads = int(max(1, min(cores, (w["M"] + 127) // 128)))

    def blis(A, B, C, threads):
        orc.lib.oracle_matmul_blis_order(A.ctypes.data, B.ctypes.data, C.ctypes.data, A.shape[0], N, K, int(threads))
    timed(blis, 8, "BLIS order (oracle restatement), rows split over min(ceil(M / 128), cores) threads as the "
          "reference's rayon row blocks", "port", blis_threads, par=blis_threads)
    run, kind, rcores, name = _load_cpu_reference()

    def ref(A, B, C, threads):
        run(A, B, C, A.shape[0], N, K)
    timed(ref, 2 * cores, name, kind, rcores)

    def npmm(A, B, C, threads):
        np.matmul(A, B, out=C)
    timed(npmm, min(w["M"], 64 * cores), "np.matmul (OpenBLAS, all cores)", "numpy", cores)
    return out


class Ctx:
    """Process-wide state of one benchmark run (one rank)."""


def _capi_check(rc):
    if rc != 0:
        from symplex_b200 import _capi
        raise SystemExit(f"symplex_b200 call failed ({rc}): {_capi.last_error()}")


def parity_check(ctx, w, A_of_rows, B, bias, C, row_base, n_rows_total):
    """Check a finished product on the device, in fp64: (i) where the epilogue is linear, the whole-output identity
    C.1 = A.(B.1) + N-sum of the bias over this rank's rows of A against the gathered C; (ii) 64 sampled rows of the
    WHOLE C (also rows computed by other ranks) against a float64 evaluation of the same formula.
    `A_of_rows(rows)` returns the A rows for global row numbers (gathered from their owners when sharded)."""
    torch = ctx.torch
    M, N, K = n_rows_total, w["N"], w["K"]
    dev = C.device
    Bm = B.transpose(-1, -2) if w["b_col"] else B  # [K, N] view
    res = {"rows": 64, "ok": True}
    g = torch.Generator(device="cpu").manual_seed(4242)
    rows = torch.sort(torch.randperm(M, generator=g)[:64]).values.to(dev)
    Ar = A_of_rows(rows).double()
    want = Ar @ Bm.double()
    if bias is not None:
        want = want + bias.double()
    if w["act"] == "gelu":
        want = 0.5 * want * (1.0 + torch.tanh(0.7978845608028654 * (want + 0.044715 * want ** 3)))
    elif w["act"] == "relu":
        want = torch.clamp(want, min=0)
    got = C[rows].double()
    rel = float((got - want).norm() / want.norm().clamp_min(1e-300))
    tol = 1e-2 if (w["dt"] == "bf16" or w["out"] == "bf16") else (1e-13 if w["dt"] == "f64" else 1e-5)
    res["max_rel"] = rel
    res["tolerance"] = tol
    res["ok"] = bool(rel <= tol)
    if w["act"] is None:
        # whole output: row sums, evaluated in chunks so the float64 copies stay small
        bsum = Bm.double().sum(dim=1)
        lhs = torch.cat([C[i:i + 4096].double().sum(dim=1) for i in range(0, M, 4096)])
        mine = ctx.local_A.double() @ bsum
        scale = ctx.local_A.double().abs() @ Bm.double().abs().sum(dim=1)
        if ctx.world > 1 and w["sharded"]:
            # every rank contributes the sums of the rows it owns, at their global row numbers
            rhs = torch.zeros(M, device=dev, dtype=torch.float64)
            sc = torch.zeros(M, device=dev, dtype=torch.float64)
            rhs[ctx.local_rows] = mine
            sc[ctx.local_rows] = scale
            ctx.dist.all_reduce(rhs)
            ctx.dist.all_reduce(sc)
        else:
            rhs, sc = mine, scale
        if bias is not None:
            rhs = rhs + bias.double().sum()
        ident = float((lhs - rhs).norm() / sc.norm())
        res["checksum_rel"] = ident
        res["ok"] = bool(res["ok"] and ident <= (1e-3 if w["out"] == "bf16" else 1e-5))

    return res


def run_gemm_workload(ctx, args, name, primary):
    """Measure one GEMM workload on this rank (and its peers); returns the JSON line as a dict (rank 0) or None.
    `primary`: the workload the line is about (full protocol: K timed steps, e2e, CPU baselines, spread of single
    steps). Secondary workloads get a short device-timed run with the same timing rules and a parity check."""
    torch, dist, sx, lib = ctx.torch, ctx.dist, ctx.sx, ctx.lib
    from symplex_b200.sharding import RowShardedGemm
    w = WORKLOADS[name]
    rank, local_rank, world, dev = ctx.rank, ctx.local_rank, ctx.world, ctx.dev
    peaks, peak_note = ctx.peaks, ctx.peak_note
    config = base_config(name, w, args.gpus)
    detail = {}

    f64 = w["dt"] == "f64"
    tdt = torch.bfloat16 if w["dt"] == "bf16" else (torch.float64 if f64 else torch.float32)
    odt = torch.bfloat16 if w["out"] == "bf16" else (torch.float64 if f64 else torch.float32)
    M, N, K, batch = w["M"], w["N"], w["K"], w["batch"]
    saved_options = []
    for oname, oval in (w.get("options") or {}).items():  # tuning overrides that select the kernel under test
        saved_options.append((oname.encode(), lib.symplex_b200_get_option(oname.encode())))
        _capi_check(lib.symplex_b200_set_option(oname.encode(), int(oval)))
        detail.setdefault("options", {})[oname] = oval
    g = torch.Generator(device=dev).manual_seed(1234)  # same B on every rank
    b_shape = (N, K) if w["b_col"] else (K, N)
    scale = 0.02 if w["act"] == "gelu" else 1.0
    if batch > 1:
        Bm = (torch.randn((batch,) + b_shape, device=dev, generator=g) * scale).to(tdt)
    else:
        Bm = (torch.randn(b_shape, device=dev, generator=g) * scale).to(tdt)
    bias = (torch.randn(N, device=dev, generator=g) * scale) if w["bias"] else None
    b_layout = sx.COL_MAJOR if w["b_col"] else sx.ROW_MAJOR

    sharded = w["sharded"]
    op = None
    if sharded:
        op = RowShardedGemm(M, N, K, chunks=args.chunks, activation=w["act"], b_layout=b_layout,
                            exchange=args.exchange)
        m_loc = M // op.world
        ga = torch.Generator(device=dev).manual_seed(100 + rank)
        A = (torch.randn(m_loc, K, device=dev, generator=ga) * scale).to(tdt)
        fused = op.exchange in op.FUSED and op.world > 1
        C = op.output_buffer(odt, dev) if fused else torch.empty(M, N, device=dev, dtype=odt)
        detail["chunks"] = op.chunks
        detail["exchange"] = {
            "peer_store": "in the GEMM kernel: forwarder warps copy each finished tile to every peer's C (16-byte "
                          "stores over NVLink), ranks ordered by flags in peer memory",
            "multicast": "in the GEMM kernel: forwarder warps store each finished tile once to a multicast mapping "
                         "(multimem.st), the NVSwitch delivers it to every GPU",
            "epilogue_tma": "in the GEMM kernel: epilogue warps forward their blocks to every peer by TMA stores",
            "nccl": "NCCL all_gather_into_tensor per row chunk, overlapped with the next chunk's GEMM",
        }[op.exchange] if op.world > 1 else "none (1 GPU)"
        detail["exchange_mode"] = op.exchange if op.world > 1 else "none"
        ctx.local_A = A

        def step():
            op(A, Bm, bias=bias, out=C)
        launches_per_step_flops = flops_of(w) / max(1, op.world) / op.chunks
    else:
        ga = torch.Generator(device=dev).manual_seed(100 + rank)
        a_shape = (batch, M, K) if batch > 1 else (M, K)
        # small problems: rotate over several operand sets so each step reads cold data (larger than L2 in total)
        esz = {"bf16": 2, "f32": 4, "f64": 8}
        bytes_per_set = (M * K + K * N) * batch * esz[w["dt"]] + M * N * batch * esz[w["out"]]
        nsets = 1 if bytes_per_set > 256e6 else int(min(64, 512e6 // bytes_per_set + 1))
        As = [(torch.randn(a_shape, device=dev, generator=ga) * scale).to(tdt) for _ in range(nsets)]
        Bs = [Bm] + [(torch.randn_like(Bm.float()) * scale).to(tdt) for _ in range(nsets - 1)]
        Cs = [torch.empty((batch, M, N) if batch > 1 else (M, N), device=dev, dtype=odt) for _ in range(nsets)]
        counter = [0]
        detail["l2"] = ("inputs larger than L2" if nsets == 1 else f"rotating over {nsets} operand sets "
                        f"({nsets * bytes_per_set / 1e6:.0f} MB > L2) so every step reads cold data")
        ctx.local_A = As[0] if batch == 1 else None

        stream = torch.cuda.current_stream(dev).cuda_stream
        emu = int(w.get("emulate_ranks", 0))
        if emu:
            import ctypes as _ct
            from symplex_b200 import _capi as _c
            peers_c = [torch.empty(emu * M, N, device=dev, dtype=odt) for _ in range(emu - 1)]
            flags_ = [torch.full((64,), 1 << 30, device=dev, dtype=torch.int32) for _ in range(emu)]
            emu_desc = sx.make_desc(emu * M, N, K, sx.DT_BF16, sx.DT_BF16 if w["out"] == "bf16" else sx.DT_F32)
            emu_full = {}
            detail["exchange"] = (f"rank 0 of {emu}: forwarder warps copy every tile to {emu - 1} buffers in local memory; "
                                  "flags preset (no other kernel is waited for)")

        def gemm_into(A_, B_, C_):
            if emu:  # C_ is rank 0's rows; the communicator wants the full buffer they are the top of
                key = C_.data_ptr()
                if key not in emu_full:
                    comm = _c.Comm()
                    comm.rank, comm.world = 0, emu
                    full = torch.empty(emu * M, N, device=dev, dtype=odt)
                    comm.c_base[0] = full.data_ptr()
                    for r in range(1, emu):
                        comm.c_base[r] = peers_c[r - 1].data_ptr()
                    for r in range(emu):
                        comm.flags[r] = flags_[r].data_ptr()
                    emu_full[key] = (comm, full)
                comm, full = emu_full[key]
                _capi_check(lib.symplex_b200_sharded_gemm(_ct.byref(emu_desc), A_.data_ptr(), B_.data_ptr(), None,
                                                          _ct.byref(comm), _c.XCHG_UNICAST, stream))
                if not emu_timed[0]:
                    C_.copy_(full[:M])
            elif f64:  # the product behind blas_dgemm / cache_tiled_dgemm_thin, on device pointers
                _capi_check(lib.symplex_b200_dgemm(A_.data_ptr(), B_.data_ptr(), C_.data_ptr(), M, N, K, 0, 0, 0, stream))
            else:
                sx.gemm(A_, B_, bias=bias, activation=w["act"], out=C_, b_layout=b_layout)

        emu_timed = [True]  # the timed steps leave the result in the communicator's buffer; the check copies it out

        def step():
            i = counter[0] % nsets
            counter[0] += 1
            gemm_into(As[i], Bs[i], Cs[i])
        launches_per_step_flops = flops_of(w)
    if sharded:
        detail["l2"] = "inputs larger than L2 (per GPU: A %.0f MiB, B %.0f MiB, C %.0f MiB)" % (
            A.numel() * A.element_size() / 2**20, Bm.numel() * Bm.element_size() / 2**20,
            C.numel() * C.element_size() / 2**20)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    steps, warmup = args.steps, args.warmup
    if not primary:
        # a short run: at least 3 warm-up steps, then enough steps for ~0.4 s (so the clock sampler sees the load)
        warmup = 3
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        step()
        torch.cuda.synchronize()
        est = max(time.perf_counter() - t0, 2e-5)
        steps = int(max(10, min(400, 0.4 / est)))
    else:
        for _ in range(warmup):
            step()
    barrier()
    sx.sync_status()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3 if primary else 0.1)
    launches0 = lib.symplex_b200_launch_count()
    stream_k0 = lib.symplex_b200_get_option(b"stream_k_launches")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    launches = lib.symplex_b200_launch_count() - launches0
    if lib.symplex_b200_get_option(b"stream_k_launches") > stream_k0:
        detail["stream_k_launches"] = lib.symplex_b200_get_option(b"stream_k_launches") - stream_k0
    sx.sync_status()

    # Steps of a few tens of microseconds: the Python caller cannot issue launches that fast, so the loop above
    # times the host. The same K steps are then captured into one CUDA graph and the replay is timed - the
    # library's launches are capturable (no allocation or synchronisation on a warm call).
    graph = None
    if not sharded and world == 1 and elapsed_ms / steps < 0.1:
        detail["eager_ms_per_step"] = elapsed_ms / steps
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(steps):
                step()
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        elapsed_ms = e0.elapsed_time(e1)
        detail["launch"] = f"one CUDA graph of {steps} steps (eager launches are host-bound at this size)"
        sx.sync_status()

    # Spread of single steps (outside the timed region above, which stays K back-to-back steps): one event between
    # consecutive steps; for graph-launched workloads one event between consecutive replays of the K-step graph.
    # One GPU only: these steps directly follow the timed ones, so on a power-capped board they show the sustained
    # rate (the clock has settled by then) next to the burst the first K steps may have run at.
    step_spread = None
    if world == 1 and primary:
        nspread = max(3, min(steps, 20))
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(nspread + 1)]
        marks[0].record()
        for i in range(nspread):
            if graph is not None:
                graph.replay()
            else:
                step()
            marks[i + 1].record()
        torch.cuda.synchronize()
        per = [marks[i].elapsed_time(marks[i + 1]) / (steps if graph is not None else 1) for i in range(nspread)]
        step_spread = {"min": min(per), "median": statistics.median(per), "max": max(per), "n": nspread}
        sx.sync_status()

    # per-launch duration of the GEMM kernel alone (no exchange), CUDA events on the launching stream
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sharded:
        blk = (M // op.world) // op.chunks
        Ak = A[:blk]
        Ck = torch.empty(blk, N, device=dev, dtype=odt) if world > 1 else C[:blk]

        def kernel_only():
            sx.gemm(Ak, Bm, bias=bias, activation=w["act"], out=Ck, b_layout=b_layout)
    else:
        kernel_only = step
    if (sharded and op.world == 1) or graph is not None or not sharded:
        kernel_ms = elapsed_ms / steps  # one step is exactly one launch of the GEMM kernel
    else:
        kernel_only()
        torch.cuda.synchronize()
        kreps = max(3, min(steps, 10))
        k0.record()
        for _ in range(kreps):
            kernel_only()
        k1.record()
        torch.cuda.synchronize()
        kernel_ms = k0.elapsed_time(k1) / kreps
    clocks = sampler.stop() if sampler else None

    # ---------------- result check (every rank, every N): sampled rows in float64 + whole-output row sums
    if sharded:
        step()
        barrier()
        # global row -> (owner, position in the owner's local A): chunk-major blocks (sharding.owned_row_blocks)
        blk_rows = (M // world) // op.chunks
        chunk_rows = M // op.chunks
        ctx.local_rows = op.local_row_index().to(dev)

        def A_of_rows(rows):
            if world == 1:
                return A[rows]
            c, within = rows // chunk_rows, rows % chunk_rows
            mine = (within // blk_rows) == rank
            local = c * blk_rows + within % blk_rows
            buf = torch.zeros(rows.numel(), K, device=dev, dtype=torch.float32)
            buf[mine] = A[local[mine]].float()
            dist.all_reduce(buf)
            return buf
        check = parity_check(ctx, w, A_of_rows, Bm, bias, C, 0, M)
    elif batch == 1:
        emu_timed[0] = False
        gemm_into(As[0], Bs[0], Cs[0])
        torch.cuda.synchronize()
        check = parity_check(ctx, w, lambda rows: As[0][rows], Bs[0], bias, Cs[0], 0, M)
        if emu:  # every "peer" buffer received rank 0's rows as well
            check["peers_identical"] = bool(all(torch.equal(pc[:M], Cs[0]) for pc in peers_c))
            check["ok"] = bool(check["ok"] and check["peers_identical"])
    else:
        gemm_into(As[0], Bs[0], Cs[0])
        torch.cuda.synchronize()
        want = torch.bmm(As[0].double(), (Bs[0].transpose(-1, -2) if w["b_col"] else Bs[0]).double())
        rel = float((Cs[0].double() - want).norm() / want.norm())
        check = {"rows": int(batch * M), "max_rel": rel, "tolerance": 1e-5, "ok": bool(rel <= 1e-5)}
    sx.sync_status()
    okt = torch.tensor([1.0 if check["ok"] else 0.0, check["max_rel"]], device=dev, dtype=torch.float64)
    if world > 1:
        okmin = okt.clone()
        dist.all_reduce(okmin, op=dist.ReduceOp.MIN)
        okmax = okt.clone()
        dist.all_reduce(okmax, op=dist.ReduceOp.MAX)
        check["ok"] = bool(okmin[0].item() > 0.5)
        check["max_rel"] = float(okmax[1].item())
        check["ranks"] = world
    ctx.parity_ok = ctx.parity_ok and check["ok"]

    t = torch.tensor([elapsed_ms, float(launches)], device=dev, dtype=torch.float64)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        elapsed_ms = tmax[0].item()
        launches = int(tsum[1].item())
    ms_per_step = elapsed_ms / steps
    replicas = 1 if sharded else world
    value = flops_of(w) * replicas / (ms_per_step * 1e-3) / 1e12

    # ---------------- end to end through the host-buffer entry points (pinned host memory)
    e2e = None
    if primary and not args.no_e2e:
        e2e = run_e2e(args, w, sx, lib, torch, dist, dev, rank, world, Bm, bias, b_layout, tdt, odt,
                      op if sharded else None, scale)
    ctx.local_A = None
    for oname, old in saved_options:
        lib.symplex_b200_set_option(oname, old)
    if rank != 0:
        return None

    achieved = launches_per_step_flops / (kernel_ms * 1e-3) / 1e12
    traffic = NCU_TRAFFIC_BYTES.get(name)
    if sharded:  # rows of A per launch, scaled from the 8192-row capture of the same kernel
        traffic = NCU_TRAFFIC_PER_8192_ROWS_BF16_N8192_K8192 * (M / args.gpus / detail["chunks"]) / 8192.0
    tensor_bound = w["dt"] in ("bf16", "f64") or w["K"] >= 1024
    if w["dt"] == "bf16":
        peak = float(peaks["bf16_tflops"])
        peak_desc = f"bf16 dense burst, {peak_note}"
    elif f64:
        # No measured fp64 figure exists for these boards; NVIDIA quotes 40 TFLOP/s (fp64, vector and tensor alike) for
        # the part. The kernel also rounds every product and sum separately, as the reference does: 2 instructions per
        # multiply-add, so half of that figure is its own ceiling.
        peak = 40.0
        peak_desc = "nominal fp64 rate of the part (no measured figure); unfused multiply + add halves it"
    else:
        peak = float(peaks["bf16_tflops"]) / 6.0
        peak_desc = f"derived 3xTF32 ceiling = bf16 burst / 2 / 3, {peak_note}"
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "kernel_ms": kernel_ms, "peak_kind": peak_desc,
                "flops_per_launch": launches_per_step_flops}
    if w["dt"] == "bf16" and "bf16_tflops_sustained" in peaks:
        roofline["frac_of_sustained"] = achieved / float(peaks["bf16_tflops_sustained"])
    if not tensor_bound:
        algo_bytes = ((M * K + K * N) * 4 + M * N * 4) * batch
        ach = algo_bytes / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": ach, "peak": float(peaks["hbm_gbs"]), "unit": "GB/s",
                    "frac": ach / float(peaks["hbm_gbs"]), "traffic": traffic,
                    "kernel_ms": kernel_ms, "peak_kind": f"HBM copy, {peak_note}", "bytes_per_launch": algo_bytes,
                    "note": "one step = one launch of the in-kernel-split fp32 GEMM kernel (no pre-pass)"}
    if sharded and world > 1:
        # The exchange: every GPU must receive the other ranks' rows of C; with unicast stores it also sends its own
        # rows world - 1 times, with the multicast mapping once. Time = the step (exchange and GEMM are one kernel).
        c_bytes = float(M) * N * (2 if w["out"] == "bf16" else 4)
        recv = c_bytes * (world - 1) / world
        send = c_bytes / world * (1 if op.exchange == "multicast" else (world - 1))
        link_ms = recv / 900e9 * 1e3
        roofline["nvlink"] = {
            "bytes_in_per_gpu": recv, "bytes_out_per_gpu": send,
            "achieved_in_gbs": recv / (ms_per_step * 1e-3) / 1e9, "achieved_out_gbs": send / (ms_per_step * 1e-3) / 1e9,
            "frac_of_900_in": recv / (ms_per_step * 1e-3) / 900e9, "nominal_link_ms": link_ms,
            "compute_ms": kernel_ms, "step_ms": ms_per_step,
            "achieved_over_bound": max(link_ms, kernel_ms) / ms_per_step,
            "note": "bound = the slower of the GEMM alone and the inbound bytes at the nominal 900 GB/s per direction"}

    line = {"metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if sharded else "weak", "vs_baseline": None,
            "dtype": {"bf16": "bf16", "f32": "f32 (3xTF32 on tensor cores)", "f64": "f64"}[w["dt"]], "data": "synthetic",
            "config": config, "detail": detail,
            "frac_of_bf16_peak": value / (args.gpus * float(peaks["bf16_tflops"])),
            "roofline": roofline, "parity_check": check, "gpu_launches": launches, "clocks": clocks}
    if primary:
        cpu_baseline = None
        if not args.no_cpu_baseline and world == 1:
            # the same row sample as the `--impl reference` arm takes for these --steps / --warmup, timed 3 times
            tfl, dt, kind, cores, sample = time_cpu_reference(w, cpu_step_seconds(args), steps=3, warmup=1)
            cpu_baseline = {"value": tfl, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample}
            try:
                cpu_baseline["all"] = cpu_baselines(w, 3.0)
            except Exception as e:  # the headline baseline above stands on its own
                cpu_baseline["all_error"] = repr(e)
        line.update({"cpu_baseline": cpu_baseline, "e2e": e2e, "step_ms": step_spread})
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="symplex_b200", choices=["symplex_b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(ELEMENTWISE_WORKLOADS))
    ap.add_argument("--chunks", type=int, default=None, help="row chunks per rank for the NCCL all-gather pipeline")
    ap.add_argument("--exchange", default=None, choices=["peer_store", "multicast", "epilogue_tma", "nccl"],
                    help="how C is all-gathered at N > 1 (default: forwarder warps inside the GEMM kernel)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="default workload on one GPU: skip the short runs of the other workloads")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl != "reference":
        args.warmup = 3  # timing rule: at least 3 warm-up steps
    if args.workload in ELEMENTWISE_WORKLOADS:
        return main_elementwise(args)

    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank != 0:
            return 0
        config = base_config(args.workload, w, args.gpus)
        tflops, dt, kind, cores, sample = time_cpu_reference(w, cpu_step_seconds(args), args.steps, max(1, args.warmup))
        line = {"impl": "reference", "metric": "gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                "scaling": "strong" if w["sharded"] else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config,
                "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
                "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return 0

    import torch
    import torch.distributed as dist

    import symplex_b200 as sx
    from symplex_b200 import _capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    ctx = Ctx()
    ctx.torch, ctx.dist, ctx.sx = torch, dist, sx
    ctx.rank, ctx.local_rank, ctx.world = rank, local_rank, world
    ctx.dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=ctx.dev)
    ctx.lib = _capi.load()
    ctx.peaks, ctx.peak_note = load_peaks()
    ctx.parity_ok = True
    ctx.local_A = None
    rc = 0
    try:
        line = run_gemm_workload(ctx, args, args.workload, primary=True)
        if world == 1 and args.workload == DEFAULT_WORKLOAD and not args.no_secondary:
            secondary = []
            for name in SECONDARY:
                torch.cuda.empty_cache()
                sec = run_gemm_workload(ctx, args, name, primary=False)
                secondary.append({k: sec[k] for k in ("config", "detail", "value", "unit", "steps", "warmup", "ms_per_step",
                                                      "dtype", "roofline", "parity_check", "gpu_launches", "clocks")})
            line["secondary"] = secondary
        if rank == 0:
            print(json.dumps(line), flush=True)
        if not ctx.parity_ok:
            if rank == 0:
                print("bench.py: a result check failed (parity_check.ok is false)", file=sys.stderr, flush=True)
            rc = 3
    finally:
        # every rank leaves in step: no rank's memory disappears while a peer still has it mapped
        if world > 1:
            try:
                torch.cuda.synchronize()
                dist.barrier()
            except Exception:
                pass
            dist.destroy_process_group()
    return rc


def run_e2e(args, w, sx, lib, torch, dist, dev, rank, world, Bm, bias, b_layout, tdt, odt, op, scale):
    """Same product with host buffers: pinned host -> device copies, compute, device -> host read, every step."""
    M, N, K, batch = w["M"], w["N"], w["K"], w["batch"]
    steps = max(2, min(args.steps, 5))
    in_b = 2 if w["dt"] == "bf16" else 4
    out_b = 2 if w["out"] == "bf16" else 4
    m_loc = M // world if op is not None else M
    hA = torch.empty((batch, m_loc, K) if batch > 1 else (m_loc, K), dtype=tdt).pin_memory()
    hA.copy_((torch.randn(hA.shape, device=dev) * scale).to(tdt))
    hB = Bm.cpu().pin_memory()
    hbias = bias.cpu().pin_memory() if bias is not None else None
    hC = torch.empty((batch, m_loc, N) if batch > 1 else (m_loc, N), dtype=odt).pin_memory()
    h2d = hA.numel() * in_b + hB.numel() * in_b + (N * 4 if bias is not None else 0)
    d2h = hC.numel() * out_b

    if op is None or world == 1:
        d = sx.make_desc(M, N, K, sx.DT_BF16 if w["dt"] == "bf16" else sx.DT_F32,
                         sx.DT_BF16 if w["out"] == "bf16" else sx.DT_F32, batch=batch, b_layout=b_layout,
                         activation=w["act"])

        def host_step():
            sx.gemm_host(d, hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), hbias.data_ptr() if hbias is not None else None)
        api = "symplex_b200_gemm_host (C ABI, pinned host buffers)"
    elif op.exchange in ("peer_store", "multicast"):
        # Per rank: the local rows go through in row chunks. Chunk c's rows of A are copied in on one stream, its
        # GEMM + exchange (one kernel) runs on a second as soon as they have landed, and this rank's rows of the
        # chunk's result go back to the host on a third - so copy-in, compute and copy-out of neighbouring chunks
        # overlap, as the one-GPU host entry point does it. B and the bias travel first, every step.
        from symplex_b200.sharding import RowShardedGemm
        nch = 4 if (m_loc % 4 == 0 and (m_loc // 4) % 256 == 0) else 1
        pipe = RowShardedGemm(M, N, K, chunks=nch, activation=w["act"], b_layout=b_layout, exchange=op.exchange)
        nch = pipe.chunks
        dC = pipe.output_buffer(odt, dev)
        dA = torch.empty(hA.shape, device=dev, dtype=tdt)
        dB = torch.empty(hB.shape, device=dev, dtype=tdt)
        dbias = torch.empty_like(bias) if bias is not None else None
        blk = m_loc // nch
        s_in, s_mm, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        ev_in = [torch.cuda.Event() for _ in range(nch)]
        ev_mm = [torch.cuda.Event() for _ in range(nch)]

        def host_step():
            with torch.cuda.stream(s_in):
                dB.copy_(hB, non_blocking=True)
                if dbias is not None:
                    dbias.copy_(hbias, non_blocking=True)
                for c in range(nch):
                    dA[c * blk:(c + 1) * blk].copy_(hA[c * blk:(c + 1) * blk], non_blocking=True)
                    ev_in[c].record(s_in)
            for c, (row0, nrows) in enumerate(pipe.blocks):
                s_mm.wait_event(ev_in[c])
                pipe.run_chunk(c, dA[c * blk:(c + 1) * blk], dB, dbias, odt, stream=s_mm.cuda_stream)
                ev_mm[c].record(s_mm)
                s_out.wait_event(ev_mm[c])
                with torch.cuda.stream(s_out):
                    hC[c * nrows:(c + 1) * nrows].copy_(dC[row0:row0 + nrows], non_blocking=True)
            torch.cuda.synchronize()
        api = (f"RowShardedGemm.run_chunk per row chunk ({nch} per rank) with pinned host shards: copy-in, "
               "GEMM + exchange and copy-out of neighbouring chunks overlap on three streams")
    else:
        dA = torch.empty(hA.shape, device=dev, dtype=tdt)
        dB = torch.empty(hB.shape, device=dev, dtype=tdt)
        dC = op.output_buffer(odt, dev) if op.exchange in op.FUSED else torch.empty(M, N, device=dev, dtype=odt)

        def host_step():
            dA.copy_(hA, non_blocking=True)
            dB.copy_(hB, non_blocking=True)
            op(dA, dB, bias=bias, out=dC)
            for c, (row0, nrows) in enumerate(op.blocks):  # this rank's rows of C go back to its host buffer
                hC[c * nrows:(c + 1) * nrows].copy_(dC[row0:row0 + nrows], non_blocking=True)
            torch.cuda.synchronize()
        api = "RowShardedGemm with pinned host shards per rank (copy-in, step, copy-out back to back)"

    host_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        host_step()
    torch.cuda.synchronize()
    dt = torch.tensor([(time.perf_counter() - t0) / steps], device=dev, dtype=torch.float64)
    tot = torch.tensor([float(h2d), float(d2h)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    sx.sync_status()
    replicas = 1 if op is not None else world
    return {"value": flops_of(w) * replicas / dt.item() / 1e12, "unit": "TFLOP/s", "ms_per_step": dt.item() * 1e3,
            "h2d_bytes_per_step": int(tot[0].item()), "d2h_bytes_per_step": int(tot[1].item()), "steps": steps,
            "api": api}


if __name__ == "__main__":
    sys.exit(main())
