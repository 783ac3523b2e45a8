#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `c2_m1`: the Q4_K 14336x4096 decode GEMV with one bf16 activation row (the shape
the headline metric "weight-GB/s at M=1" is quoted on).  One STEP is four passes over a stack of 32
distinct weight matrices of that shape (1.06 GB, far larger than the 126 MB L2, so every launch
streams its weights from HBM); the 128 launches of a step are replayed from one CUDA graph.

Printed JSON (one line, rank 0):
  value      whole-job weight-GB/s with everything resident in HBM (CUDA events, max over ranks)
  e2e        the same metric through the public GcuDevice API: activations copied from host memory
             and the result copied back and synchronised inside every step
  roofline   algorithmic weight+activation+output bytes of one launch / average launch duration
             inside the timed region, against the measured HBM copy bandwidth
  cpu_baseline   the CPU restatement of the same dequant-dot on this box's host cores (bounded sample)

`--impl reference` times that CPU path alone (the reference's own kernels need the vendor toolchain
and device, so the CPU restatement is the only reference arm that can run).

Other workloads (c1, c2_m4, c2_m16, c3, c4, c5_m1, c5_m512; q6k_m1 for the Q6_K decode kernel) print the same
line for the other configurations.  The linear workloads run one replica per GPU (weak scaling); c4 (MoE layer) and c5
(70B-shaped linear stack) shard over the ranks (expert / tensor parallel, strong scaling) with NCCL
all-reduces through the eccl entry points.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read + dram__bytes_write of ONE launch of the workload's dominant kernel, from the ncu
# captures summarised under profiles/ (null where no capture has been taken yet)
NCU_TRAFFIC_BYTES = {"c1": 17896448, "c2_m1": 33104128, "c3": 66714368}

Q4K_ROW_BYTES = lambda K: K // 256 * 144  # noqa: E731
Q8_ROW_BYTES = lambda K: K // 32 * 34  # noqa: E731
Q6K_ROW_BYTES = lambda K: K // 256 * 210  # noqa: E731


def wl_format(wl) -> str:
    """"Q8_0", "Q4_K" or "Q6_K" (key ``fmt`` overrides the is_q4k flag)."""
    return wl.get("fmt", "Q4_K" if wl["is_q4k"] else "Q8_0")


def wl_row_bytes(wl) -> int:
    return {"Q8_0": Q8_ROW_BYTES, "Q4_K": Q4K_ROW_BYTES, "Q6_K": Q6K_ROW_BYTES}[wl_format(wl)](wl["K"])


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------- rank rendezvous
class Control:
    """Host-side rendezvous of the ranks over a CPU (gloo) group: barriers, max-over-ranks of timings and
    the hand-over of the collective library's unique id.  The data path's collectives are NCCL, through
    the eccl entry points; keeping the control plane off the GPU means no second NCCL communicator shares
    the device with them."""

    def __init__(self, torch, dist, world: int):
        self.torch, self.dist, self.world = torch, dist, world
        self.group = dist.new_group(backend="gloo") if world > 1 else None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier(group=self.group)

    def max(self, value: float) -> float:
        if self.world == 1:
            return value
        t = self.torch.tensor([value], dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def all_gather(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj, group=self.group)
        return out

    def broadcast(self, obj):
        box = [obj]
        if self.world > 1:
            self.dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]


CTL = None  # set by main()


# ----------------------------------------------------------------------------- CPU arm
class CpuArm:
    """The CPU restatement (oracle/ub_oracle.c, OpenMP over weight rows) on this workload's matrix:
    the same block-wise dequantise-and-dot, f32 accumulation, all host threads."""

    def __init__(self, workload: dict):
        from oracle import oracle as o

        self.o, self.wl = o, workload
        N, K, M, is_q4k = workload["N"], workload["K"], workload["M"], workload["is_q4k"]
        rng = np.random.default_rng(workload["seed"])
        fmt = wl_format(workload)
        self.w = {"Q8_0": o.gen_q8_0_weight, "Q4_K": o.gen_q4k_weight, "Q6_K": o.gen_q6k_weight}[fmt](rng, N, K)
        self.fmt_code = {"Q8_0": o.FMT_Q8_0, "Q4_K": o.FMT_Q4K, "Q6_K": o.FMT_Q6K}[fmt]
        self.Ms = min(M, workload.get("cpu_rows", M))
        self.x = o.gen_activation(rng, self.Ms, K, workload["x_bf16"])
        self.y = np.empty((self.Ms, N), dtype=np.float32)
        self.fn = o.clib().ub_oracle_qmatmul_f32
        self.cores = os.cpu_count()
        self.call()  # warm-up: page-in and thread pool

    def call(self):
        o, wl = self.o, self.wl
        self.fn(o._p(self.x), o._p(self.w), o._p(self.y), self.Ms, wl["N"], wl["K"], self.fmt_code)

    def run(self, budget_s: float):
        """Repeats the matmul for about budget_s seconds; returns (value in the metric's unit, sample text)."""
        wl = self.wl
        reps, t0 = 0, time.perf_counter()
        while True:
            self.call()
            reps += 1
            el = time.perf_counter() - t0
            if el >= budget_s:
                break
        per_call = el / reps
        if wl["unit"] == "GB/s":
            value = self.w.nbytes / per_call / 1e9
        elif wl["unit"] == "tok/s":
            # expert GEMM rate of the sample, converted with the layer's flop per token
            value = 2.0 * self.Ms * wl["N"] * wl["K"] / per_call / wl["flop_per_token"]
        else:
            value = 2.0 * self.Ms * wl["N"] * wl["K"] / per_call / 1e12
        sample = "%d x [%dx%d %s] . x[%d rows] in %.2f s" % (reps, wl["N"], wl["K"], wl_format(wl),
                                                          self.Ms, el)
        return value, sample


# ----------------------------------------------------------------------------- workloads
WORKLOADS = {
    # name: N, K, M, format, activation type, metric unit, seed, number of distinct weight copies per step
    "c1": dict(N=4096, K=4096, M=1, is_q4k=False, x_bf16=False, unit="GB/s", seed=1001, copies=64,
               desc="Q8_0 4096x4096 decode GEMV, f32 activations"),
    "c2_m1": dict(N=14336, K=4096, M=1, is_q4k=True, x_bf16=True, unit="GB/s", seed=1002, copies=32, passes=4,
                  desc="Q4_K 14336x4096 decode GEMV, bf16 activations, M=1"),
    "c2_m4": dict(N=14336, K=4096, M=4, is_q4k=True, x_bf16=True, unit="GB/s", seed=1002, copies=32,
                  desc="Q4_K 14336x4096 small-batch decode, M=4"),
    "c2_m16": dict(N=14336, K=4096, M=16, is_q4k=True, x_bf16=True, unit="GB/s", seed=1002, copies=32,
                   desc="Q4_K 14336x4096 small-batch decode, M=16"),
    "q6k_m1": dict(N=14336, K=4096, M=1, is_q4k=False, fmt="Q6_K", x_bf16=True, unit="GB/s", seed=1006, copies=16,
                   passes=4, desc="Q6_K 14336x4096 decode GEMV, bf16 activations, M=1"),
    "c3": dict(N=14336, K=4096, M=2048, is_q4k=True, x_bf16=True, unit="TFLOP/s", seed=1002, copies=2, cpu_rows=64,
               desc="Q4_K 14336x4096 prefill GEMM, M=2048"),
    "c3_m1024": dict(N=14336, K=4096, M=1024, is_q4k=True, x_bf16=True, unit="TFLOP/s", seed=1002, copies=2,
                     cpu_rows=64, desc="Q4_K 14336x4096 prefill GEMM, M=1024 (the small case profiled under ncu)"),
    # sharded workloads.  N, K, M, cpu_rows describe the matrix the CPU arm samples (one expert's gate
    # projection; a quarter of the gate projection of the 70B-shaped MLP).
    "c4": dict(kind="ep", T=256, H=4096, I=14336, E=8, top_k=2, block=64, unit="tok/s", seed=1004, is_q4k=True,
               x_bf16=True, N=14336, K=4096, M=256, cpu_rows=64, flop_per_token=2 * 3 * 2.0 * 4096 * 14336,
               desc="Mixtral-shaped fused MoE layer, 8 experts top-2, 256 tokens, Q4_K experts, expert parallel"),
    "c5_m1": dict(kind="tp", hidden=8192, inter=28672, q_heads=64, kv_heads=8, head_dim=128, unit="GB/s", seed=1005,
                  is_q4k=True, x_bf16=True, N=7168, K=8192, M=1,
                  desc="Llama-3-70B-shaped QKV/O + MLP linear stack, Q4_K, tensor parallel, M=1"),
    "c5_m512": dict(kind="tp", hidden=8192, inter=28672, q_heads=64, kv_heads=8, head_dim=128, unit="TFLOP/s",
                    seed=1005, is_q4k=True, x_bf16=True, N=7168, K=8192, M=512, cpu_rows=32,
                    desc="Llama-3-70B-shaped QKV/O + MLP linear stack, Q4_K, tensor parallel, M=512"),
}


def run_linear(args, wl, rank, world, torch, dist):
    """Replicated (data-parallel, weak scaling) linear workloads: every rank streams its own copies."""
    import ubridge_b200 as ub
    from ubridge_b200 import synth as o  # seeded synthetic inputs
    from ubridge_b200 import ops

    dev_index = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev_index)
    N, K, M, is_q4k = wl["N"], wl["K"], wl["M"], wl["is_q4k"]
    rng = np.random.default_rng(wl["seed"] + rank)
    fmt = wl_format(wl)
    w_host = {"Q8_0": o.gen_q8_0_weight, "Q4_K": o.gen_q4k_weight, "Q6_K": o.gen_q6k_weight}[fmt](rng, N, K).reshape(-1)
    w_bytes = w_host.nbytes
    copies = wl["copies"]
    x_dtype = ub.DTYPE_BF16 if wl["x_bf16"] else ub.DTYPE_F32
    y_dtype = ub.DTYPE_BF16 if wl["x_bf16"] else ub.DTYPE_F32
    xs = o.gen_activation(rng, M, K, wl["x_bf16"])
    x_host = o.f32_to_bf16_bits(xs).reshape(M, K) if wl["x_bf16"] else xs
    esz = 2 if wl["x_bf16"] else 4

    # distinct weight buffers resident in HBM (same bytes at different addresses: what matters is that
    # their total size exceeds L2, so every launch streams from DRAM)
    w_dev = torch.empty((copies, w_bytes), dtype=torch.uint8, device="cuda")
    base = torch.from_numpy(w_host).cuda()
    for c in range(copies):
        w_dev[c].copy_(base)
    del base
    x_dev = torch.from_numpy(x_host.view(np.uint8).reshape(-1).copy()).cuda()
    y_dev = torch.empty((M * N * esz,), dtype=torch.uint8, device="cuda")
    ws_bytes = 0 if fmt == "Q6_K" else ops.qmatmul_workspace_bytes(M, N, K, is_q4k)

    def matmul(y, x, w, workspace, stream):
        if fmt == "Q6_K":
            ops.qmatmul_q6k(y, x, w, M, N, K, x_dtype=x_dtype, out_dtype=y_dtype, stream=stream)
        else:
            ops.qmatmul(y, x, w, M, N, K, is_q4k=is_q4k, x_dtype=x_dtype, out_dtype=y_dtype, workspace=workspace,
                        ws_bytes=ws_bytes, stream=stream)
    ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device="cuda")

    stream = torch.cuda.Stream()
    sp = ctypes.c_void_p(stream.cuda_stream)

    passes = wl.get("passes", 1)

    def one_step():
        for _p in range(passes):
            for c in range(copies):
                matmul(y_dev.data_ptr(), x_dev.data_ptr(), w_dev[c].data_ptr(), ws.data_ptr(), sp)

    with torch.cuda.stream(stream):
        one_step()  # first call resolves symbols and attributes outside any capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_step()
        for _ in range(args.warmup):
            graph.replay()
        stream.synchronize()
        CTL.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(dev_index)
        if rank == 0:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        ev1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    ms_total = CTL.max(ms_total)
    ms_step = ms_total / args.steps

    # Q8_0 decode kernel: M rows are processed 4/2/1 at a time, one launch each
    def decode_launches(m):
        n = 0
        while m > 0:
            t_ = 4 if m >= 4 else (2 if m >= 2 else 1)
            m -= t_
            n += 1
        return n
    if is_q4k:
        # decode kernel: up to eight rows per pass; bf16 in and out from nine rows on: one tensor-core launch
        launches_per_call = 1 if M > 16 or (M > 8 and wl["x_bf16"]) else (M + 7) // 8
    else:  # Q8_0 and Q6_K
        launches_per_call = decode_launches(M)
    launches = args.steps * copies * passes * launches_per_call

    calls = copies * passes * world
    if wl["unit"] == "GB/s":
        value = calls * w_bytes / (ms_step * 1e-3) / 1e9
    else:
        value = calls * 2.0 * M * N * K / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public device API: host activations in, host result out, every step
    e2e = None
    if rank == 0 or world > 1:
        dev = ub.GcuDevice(dev_index)
        w_e2e = [dev.alloc(w_bytes) for _ in range(copies)]
        for c in range(copies):
            ub.lib().ub_memcpy_dtod(dev._handle, ctypes.c_void_p(w_e2e[c].ptr), ctypes.c_void_p(w_dev[c].data_ptr()),
                                    w_bytes)
        dev.synchronize()
        del w_dev
        torch.cuda.empty_cache()
        host_x = torch.from_numpy(x_host.view(np.uint8).reshape(-1).copy()).pin_memory()
        host_y = torch.empty((M * N * esz,), dtype=torch.uint8).pin_memory()
        d_x, d_y = dev.alloc(host_x.numel()), dev.alloc(host_y.numel())
        d_ws = dev.alloc(max(ws_bytes, 256))
        lib = ub.lib()

        def e2e_step():
            lib.ub_memcpy_htod(dev._handle, ctypes.c_void_p(d_x.ptr), ctypes.c_void_p(host_x.data_ptr()), host_x.numel())
            for _p in range(passes):
                for c in range(copies):
                    matmul(d_y, d_x, w_e2e[c], d_ws, dev.stream)
            lib.ub_memcpy_dtoh(dev._handle, ctypes.c_void_p(host_y.data_ptr()), ctypes.c_void_p(d_y.ptr), host_y.numel())
            dev.synchronize()

        for _ in range(max(3, args.warmup)):
            e2e_step()
        CTL.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        el = time.perf_counter() - t0
        el = CTL.max(el)
        s_step = el / args.steps
        ev = calls * w_bytes / s_step / 1e9 if wl["unit"] == "GB/s" else calls * 2.0 * M * N * K / s_step / 1e12
        e2e = {"value": ev, "unit": wl["unit"], "h2d_bytes_per_step": int(host_x.numel()),
               "d2h_bytes_per_step": int(host_y.numel())}

    peaks = measured_peaks()
    algo_bytes = w_bytes + M * K * esz + M * N * esz
    avg_launch_s = ms_total * 1e-3 / (args.steps * copies * passes)  # per matmul call (all of its launches)
    if wl["unit"] == "GB/s":
        achieved = algo_bytes / avg_launch_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": algo_bytes, "avg_launch_us": avg_launch_s * 1e6}
    else:
        achieved = 2.0 * M * N * K / avg_launch_s / 1e12
        # a timed region shorter than a second is a burst (the clocks have not settled under the power cap):
        # compare it with the burst GEMM peak; longer regions with the sustained one
        burst = ms_total < 1000.0
        peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": None, "peak_source": peaks["source"],
                "peak_kind": "burst" if burst else "sustained",
                "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
                "algorithmic_flops_per_launch": 2.0 * M * N * K, "avg_launch_us": avg_launch_s * 1e6}
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload)
    return dict(value=value, ms_per_step=ms_step, launches=launches, e2e=e2e, roofline=roof, clocks=clocks,
                dtype={"Q4_K": "u4+f16 scales -> f32 accumulate", "Q8_0": "i8+f16 scales -> f32 accumulate",
                       "Q6_K": "u6+i8 scales+f16 -> f32 accumulate"}[fmt])


def run_sharded(args, wl, rank, world, torch, dist):
    """Tensor-parallel (c5) and expert-parallel (c4) workloads: the matrices are split over the ranks, every
    rank streams its shard and the partial outputs meet in NCCL all-reduces (strong scaling)."""
    import ubridge_b200 as ub
    from ubridge_b200 import synth as o  # seeded synthetic inputs
    from ubridge_b200 import eccl, parallel

    dev_index = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev_index)
    dev = ub.GcuDevice(dev_index)
    dev.bind_to_thread()
    ext = torch.cuda.ExternalStream(dev.stream.value)
    comm, all_reduce = None, None

    def note(msg):
        if os.environ.get("UB_BENCH_VERBOSE"):
            print("[rank %d] %s" % (rank, msg), file=sys.stderr, flush=True)

    if world > 1:
        # the 128-byte unique id travels out of band (the CPU group), as it does in the reference
        uid = CTL.broadcast(eccl.Id().internal() if rank == 0 else None)
        note("unique id exchanged")
        comm = eccl.Comm.from_rank(rank, world, eccl.Id(uid))
        note("communicator ready")

        # messages of a few KB (the decode path) go through the one-shot peer-memory kernel, larger ones
        # through NCCL; UB_BENCH_ALLREDUCE=nccl forces NCCL for comparison
        oneshot_limit = 0 if os.environ.get("UB_BENCH_ALLREDUCE") == "nccl" else 65536
        oneshot = eccl.OneShotAllReduce(dev, rank, world, oneshot_limit, CTL.all_gather) if oneshot_limit else None
        CTL.barrier()
        note("peer staging buffers open")

        def all_reduce(buf, count):
            if oneshot is not None and count * 2 <= oneshot_limit and count % 8 == 0:
                oneshot.all_reduce(buf, count)
            else:
                comm.all_reduce(buf, buf, count, eccl.Bfloat16, eccl.ReduceOp.Sum, stream=dev.stream)

    rng = np.random.default_rng(wl["seed"] + 17 * rank)
    q4 = lambda n, k: o.gen_q4k_weight(rng, n, k).reshape(-1)  # noqa: E731
    kind = wl["kind"]
    if kind == "tp":
        H, I, M = wl["hidden"], wl["inter"], wl["M"]
        ql, kvl, il = wl["q_heads"] * wl["head_dim"] // world, wl["kv_heads"] * wl["head_dim"] // world, I // world
        shapes = [(ql + 2 * kvl, H), (H, ql), (2 * il, H), (H, il)]  # this rank's shards, generated at shard shape
        shard_bytes = sum(n * Q4K_ROW_BYTES(k) for n, k in shapes)
        total_bytes = shard_bytes * world
        flop = 2.0 * M * sum(n * k for n, k in shapes) * world
        in_elems, out_elems = M * H, M * H
    else:
        T, H, I, E = wl["T"], wl["H"], wl["I"], wl["E"]
        e0, e1 = parallel.expert_range(E, rank, world)
        el = e1 - e0
        shard_bytes = el * (2 * I * Q4K_ROW_BYTES(H) + H * Q4K_ROW_BYTES(I))
        total_bytes = E * (2 * I * Q4K_ROW_BYTES(H) + H * Q4K_ROW_BYTES(I))
        flop = T * wl["flop_per_token"]
        in_elems, out_elems = T * H, T * H
    # distinct copies of the shard so that consecutive steps stream from HBM, not from the 126 MB L2
    ncopies = max(1, -(-300_000_000 // shard_bytes))
    layers = []
    for _c in range(ncopies):
        if kind == "tp":
            ws_ = [q4(n, k) for n, k in shapes]
            layers.append(parallel.TPLinearStack(dev, H, I, wl["q_heads"], wl["kv_heads"], wl["head_dim"], world,
                                                 ws_[0], ws_[1], ws_[2], ws_[3], M, all_reduce))
        else:
            w13 = np.concatenate([q4(2 * I, H) for _e in range(el)])
            w2 = np.concatenate([q4(H, I) for _e in range(el)])
            layers.append(parallel.EPMoELayer(dev, T, H, I, E, wl["top_k"], wl["block"], rank, world, w13, w2,
                                              all_reduce))
    xr = np.random.default_rng(wl["seed"])  # activations are replicated: same seed on every rank
    x_host = o.f32_to_bf16_bits(o.gen_activation(xr, in_elems // H, H, True)).reshape(-1)
    d_x = dev.htod_sync_copy(x_host)
    d_logits = None
    if kind == "ep":
        lg_host = o.f32_to_bf16_bits(o.gen_activation(xr, wl["T"], wl["E"], True)).reshape(-1)
        d_logits = dev.htod_sync_copy(lg_host)

    def forward(layer):
        return layer.forward(d_x, wl["M"]) if kind == "tp" else layer.forward(d_x, d_logits)

    # one eager pass per copy (resolves symbols, sets attributes), then one CUDA graph per copy; with several
    # GPUs the graphs contain the NCCL all-reduces
    note("weights resident, %d copies" % ncopies)
    for layer in layers:
        forward(layer)
    dev.synchronize()
    note("eager pass done")
    use_graph = True
    graphs = []
    with torch.cuda.stream(ext):
        if use_graph:
            for layer in layers:
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=ext, capture_error_mode="thread_local"):
                    forward(layer)
                graphs.append(g_)
            note("graphs captured")

        def step(i):
            if use_graph:
                graphs[i % ncopies].replay()
            else:
                forward(layers[i % ncopies])

        for i in range(args.warmup):
            step(i)
        ext.synchronize()
        note("warm-up done")
        CTL.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(dev_index)
        if rank == 0:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(ext)
        for i in range(args.steps):
            step(i)
        ev1.record(ext)
        ext.synchronize()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    note("timed region done: %.3f ms" % ms_total)
    ms_total = CTL.max(ms_total)
    ms_step = ms_total / args.steps
    s_step = ms_step * 1e-3

    def metric_value(sec):
        if wl["unit"] == "GB/s":
            return total_bytes / sec / 1e9
        if wl["unit"] == "TFLOP/s":
            return flop / sec / 1e12
        return wl["T"] / sec

    value = metric_value(s_step)
    # ---- end to end: host activations in, host result out, every step (eager launches through the API)
    host_x = torch.from_numpy(x_host.view(np.uint8).reshape(-1).copy()).pin_memory()
    host_y = torch.empty((out_elems * 2,), dtype=torch.uint8).pin_memory()
    lib = ub.lib()

    # A single GPU launches the layer eagerly through the API.  With several GPUs the step replays the
    # captured graph between the two copies, so that host launch cost does not hide the collectives.
    e2e_graph = world > 1

    def e2e_step(i):
        lib.ub_memcpy_htod(dev._handle, ctypes.c_void_p(d_x.ptr), ctypes.c_void_p(host_x.data_ptr()), host_x.numel())
        if e2e_graph:
            with torch.cuda.stream(ext):
                graphs[i % ncopies].replay()
            out = layers[i % ncopies].out
        else:
            out = forward(layers[i % ncopies])
        lib.ub_memcpy_dtoh(dev._handle, ctypes.c_void_p(host_y.data_ptr()), ctypes.c_void_p(out.ptr), host_y.numel())
        dev.synchronize()

    note("end-to-end loop starts")
    for i in range(max(3, args.warmup)):
        e2e_step(i)
    note("end-to-end warm-up done")
    CTL.barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    el_s = time.perf_counter() - t0
    el_s = CTL.max(el_s)
    note("end-to-end loop done")
    e2e = {"value": metric_value(el_s / args.steps), "unit": wl["unit"], "h2d_bytes_per_step": int(host_x.numel()),
           "d2h_bytes_per_step": int(host_y.numel()), "launch_mode": "cuda graph" if e2e_graph else "eager"}

    peaks = measured_peaks()
    # per-GPU roofline: this rank's shard bytes (or flop) per step against one GPU's measured peak
    hbm = shard_bytes / s_step / 1e9
    tf = flop / world / s_step / 1e12
    tensor_peak = peaks["bf16_tflops"] if ms_total < 1000.0 else peaks["bf16_tflops_sustained"]
    if wl["unit"] == "TFLOP/s":
        roof = {"bound": "tensor", "achieved": tf, "peak": tensor_peak, "unit": "TFLOP/s", "frac": tf / tensor_peak}
    else:
        roof = {"bound": "hbm", "achieved": hbm, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": hbm / peaks["hbm_gbs"],
                "tensor_frac": tf / tensor_peak}
    roof.update({"traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_source": peaks["source"], "per_gpu": True,
                 "algorithmic_bytes_per_step_per_gpu": shard_bytes, "algorithmic_flops_per_step": flop,
                 "step_us": s_step * 1e6})
    # kernels of ours per step: tp = 4 matmuls (+ conversions none: bf16) + copy + SiLU.up; ep = the fused layer
    launches = args.steps * layers[0].launches_per_forward
    if comm is not None:
        # NCCL keeps a communicator alive while a CUDA graph that captured its collectives exists, and
        # ncclCommDestroy waits for those references: release the graphs first
        dev.synchronize()
        graphs.clear()
        g_ = None
        import gc
        gc.collect()
        CTL.barrier()
        note("graphs released")
        if oneshot is not None:
            oneshot.close()
        comm.destroy()
        note("communicator destroyed")
    return dict(value=value, ms_per_step=ms_step, launches=launches, e2e=e2e, roofline=roof, clocks=clocks,
                dtype="u4+f16 scales -> f32 accumulate", ncopies=ncopies,
                launch_mode="cuda graph" if use_graph else "eager",
                allreduce=("one-shot peer-memory kernel up to 64 KB, NCCL above" if world > 1 and oneshot_limit
                           else ("NCCL" if world > 1 else "none")))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_m1", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU baseline sample")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    metric = {"GB/s": "weight_GBps", "TFLOP/s": "TFLOPS", "tok/s": "moe_tokens_per_s"}[wl["unit"]]
    sharded = "kind" in wl
    if sharded:
        config = {"workload": "%s: %s; one step = one pass over the layer; consecutive steps use distinct weight "
                              "copies (>= 300 MB per GPU in total, larger than L2)" % (args.workload, wl["desc"]),
                  "M": wl["M"], "format": "Q4_K", "l2_policy": "inputs larger than L2",
                  "parallelism": "%s%d" % (wl["kind"], args.gpus)}
    else:
        config = {"workload": "%s: %s; one step = %d matmuls over %d distinct weight copies (%.0f MB, larger than "
                              "L2)" % (args.workload, wl["desc"], wl["copies"] * wl.get("passes", 1), wl["copies"],
                                       wl["copies"] * wl["N"] * wl_row_bytes(wl) / 1e6),
                  "N": wl["N"], "K": wl["K"], "M": wl["M"], "format": wl_format(wl),
                  "l2_policy": "inputs larger than L2", "parallelism": "replicas x%d" % args.gpus}

    if args.impl == "reference":
        if rank != 0:
            return
        vals = []
        sample = ""
        arm = CpuArm(wl)
        cores = arm.cores
        per = max(0.25, min(args.cpu_seconds, 60.0 / max(1, args.steps + args.warmup)))
        for i in range(args.warmup + args.steps):
            v, sample = arm.run(per)
            if i >= args.warmup:
                vals.append(v)
        value = statistics.mean(vals)
        line = {"impl": "reference", "metric": metric, "value": value, "unit": wl["unit"], "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True,
                "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config,
                "cpu_baseline": {"value": value, "unit": wl["unit"], "cores": cores, "kind": "port",
                                 "sample": "each step: " + sample},
                "e2e": {"value": value, "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        # torch's own NCCL communicator is created lazily and never used: every collective of the control
        # plane goes through the CPU group of Control
        dist.init_process_group("nccl")
    global CTL
    CTL = Control(torch, dist, world)
    try:
        res = (run_sharded if sharded else run_linear)(args, wl, rank, world, torch, dist)
        if rank == 0:
            cpu = None
            if world == 1:
                arm = CpuArm(wl)
                v, sample = arm.run(args.cpu_seconds)
                cpu = {"value": v, "unit": wl["unit"], "cores": arm.cores, "kind": "port", "sample": sample}
            if "launch_mode" in res:
                config["launch_mode"] = res["launch_mode"]
                config["weight_copies"] = res["ncopies"]
                config["allreduce"] = res["allreduce"]
            line = {"metric": metric, "value": res["value"], "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                    "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": res["dtype"],
                    "data": "synthetic",
                    "config": config, "roofline": res["roofline"], "cpu_baseline": cpu, "e2e": res["e2e"],
                    "gpu_launches": res["launches"], "clocks": res["clocks"]}
            print(json.dumps(line))
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
