#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `c2_m1`: the Q4_K 14336x4096 decode GEMV with one bf16 activation row (the shape
the headline metric "weight-GB/s at M=1" is quoted on).  One CUDA graph holds four passes over a stack of 32
distinct weight matrices of that shape (1.06 GB, far larger than the 126 MB L2, so every launch
streams its weights from HBM); one STEP replays that graph k times, k chosen so that the timed region
(--steps steps) lasts at least two seconds: long enough for the clocks to settle and for the clock sampler
to see them.  k is stated in config.workload.

With the default workload the line also carries
  secondary  (one GPU) the other single-GPU configurations: c1, c2_m4, c2_m8, c2_m16, c3
  sharded    (any number of GPUs) the strong-scaling configurations at this GPU count: c5_m1, c5_m512
             (tensor parallel) and c4 (expert parallel), run in the same process group
(--no-extras leaves both out).

Printed JSON (one line, rank 0):
  value      whole-job weight-GB/s with everything resident in HBM (CUDA events, max over ranks)
  e2e        the same metric through the public GcuDevice API: activations copied from host memory
             and the result copied back and synchronised inside every step
  e2e_per_call   one matmul per round trip: host activations in, one launch, host result out, synchronise
  roofline   algorithmic weight+activation+output bytes of one launch / average launch duration
             inside the timed region, against the measured HBM copy bandwidth
  cpu_baseline   the CPU restatement of the same dequant-dot on this box's host cores (bounded sample)

`--impl reference` times that CPU path alone (the reference's own kernels need the vendor toolchain
and device, so the CPU restatement is the only reference arm that can run).

Other workloads (c1, c2_m4, c2_m8, c2_m16, c3, c4, c5_m1, c5_m512; q6k_m1, q5k_m1, q4_0_m1 for the decode kernels of the other GGUF formats) print the same
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

# ncu summary of the workload's dominant kernel: its line `dram_bytes_per_launch = <n>` (dram__bytes_read +
# dram__bytes_write of ONE launch) is what roofline.traffic reports; null where no capture has been summarised
PROFILE_OF = {"c1": "qgemv_q8_0_m1_kernel__c1.md", "c2_m1": "qgemv_q4k_m1_kernel__c2_m1.md",
              "c2_m4": "qgemv_q4k_mt_kernel__c2_m4.md", "c2_m8": "qgemv_q4k_mc_kernel__c2_m8.md",
              "c2_m16": "qgemm_q4k_tc_kernel__c2_m16.md", "c3": "qgemm_q4k_tc_kernel__c3.md",
              "c4": "qgemm_q4k_tc_kernel__c4.md", "q6k_m1": "qgemv_q6k_m1_kernel__q6k_m1.md"}


def profile_traffic(workload: str):
    import re

    name = PROFILE_OF.get(workload)
    if not name:
        return None
    try:
        with open(os.path.join(ROOT, "profiles", name)) as f:
            m = re.search(r"dram_bytes_per_launch\s*=\s*(\d+)", f.read())
    except OSError:
        return None
    return int(m.group(1)) if m else None

Q4K_ROW_BYTES = lambda K: K // 256 * 144  # noqa: E731
Q8_ROW_BYTES = lambda K: K // 32 * 34  # noqa: E731
Q6K_ROW_BYTES = lambda K: K // 256 * 210  # noqa: E731
Q5K_ROW_BYTES = lambda K: K // 256 * 176  # noqa: E731
Q4_0_ROW_BYTES = lambda K: K // 32 * 18   # noqa: E731


def GEN_WEIGHT(o):
    """Synthetic weight generators by format name (o: the module that holds them)."""
    return {"Q8_0": o.gen_q8_0_weight, "Q4_K": o.gen_q4k_weight, "Q6_K": o.gen_q6k_weight, "Q5_K": o.gen_q5k_weight,
            "Q4_0": o.gen_q4_0_weight}


def wl_format(wl) -> str:
    """"Q8_0", "Q4_K", "Q6_K", "Q5_K" or "Q4_0" (key ``fmt`` overrides the is_q4k flag)."""
    return wl.get("fmt", "Q4_K" if wl["is_q4k"] else "Q8_0")


def wl_row_bytes(wl) -> int:
    return {"Q8_0": Q8_ROW_BYTES, "Q4_K": Q4K_ROW_BYTES, "Q6_K": Q6K_ROW_BYTES, "Q5_K": Q5K_ROW_BYTES,
            "Q4_0": Q4_0_ROW_BYTES}[wl_format(wl)](wl["K"])


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
        self.w = GEN_WEIGHT(o)[fmt](rng, N, K)
        self.fmt_code = {"Q8_0": o.FMT_Q8_0, "Q4_K": o.FMT_Q4K, "Q6_K": o.FMT_Q6K, "Q5_K": o.FMT_Q5K,
                         "Q4_0": o.FMT_Q4_0}[fmt]
        self.Ms = min(M, workload.get("cpu_rows", M))
        self.x = o.gen_activation(rng, self.Ms, K, workload["x_bf16"])
        self.y = np.empty((self.Ms, N), dtype=np.float32)
        self.fn = o.clib().ub_oracle_qmatmul_f32
        # launchers such as torch.distributed.run export OMP_NUM_THREADS=1: ask for every host core and report
        # the thread count OpenMP actually grants
        self.cores = o.set_threads(os.cpu_count() or 1)
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
    "c2_m8": dict(N=14336, K=4096, M=8, is_q4k=True, x_bf16=True, unit="GB/s", seed=1002, copies=32,
                  desc="Q4_K 14336x4096 small-batch decode, M=8"),
    "c2_m16": dict(N=14336, K=4096, M=16, is_q4k=True, x_bf16=True, unit="GB/s", seed=1002, copies=32,
                   desc="Q4_K 14336x4096 small-batch decode, M=16"),
    "q6k_m1": dict(N=14336, K=4096, M=1, is_q4k=False, fmt="Q6_K", x_bf16=True, unit="GB/s", seed=1006, copies=16,
                   passes=4, desc="Q6_K 14336x4096 decode GEMV, bf16 activations, M=1"),
    "q5k_m1": dict(N=14336, K=4096, M=1, is_q4k=False, fmt="Q5_K", x_bf16=True, unit="GB/s", seed=1007, copies=16,
                   passes=4, desc="Q5_K 14336x4096 decode GEMV, bf16 activations, M=1"),
    "q4_0_m1": dict(N=14336, K=4096, M=1, is_q4k=False, fmt="Q4_0", x_bf16=True, unit="GB/s", seed=1008, copies=32,
                    passes=4, desc="Q4_0 14336x4096 decode GEMV, bf16 activations, M=1"),
    "c3": dict(N=14336, K=4096, M=2048, is_q4k=True, x_bf16=True, unit="TFLOP/s", seed=1002, copies=2, cpu_rows=64,
               desc="Q4_K 14336x4096 prefill GEMM, M=2048"),
    "c3_m1024": dict(N=14336, K=4096, M=1024, is_q4k=True, x_bf16=True, unit="TFLOP/s", seed=1002, copies=2,
                     cpu_rows=64, desc="Q4_K 14336x4096 prefill GEMM, M=1024 (the small case profiled under ncu)"),
    "c1_m512": dict(N=4096, K=4096, M=512, is_q4k=False, x_bf16=True, unit="TFLOP/s", seed=1001, copies=8, cpu_rows=64,
                    desc="Q8_0 4096x4096 prefill GEMM, M=512"),
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


def replays_for(min_seconds: float, steps: int, seconds_per_replay: float) -> int:
    """Graph replays per step so that `steps` steps last at least min_seconds."""
    if seconds_per_replay <= 0:
        return 1
    return max(1, int(np.ceil(min_seconds / (steps * seconds_per_replay))))


def run_linear(wl_name, wl, steps, warmup, min_seconds, rank, world, torch, with_e2e=True):
    """Replicated (data-parallel, weak scaling) linear workloads: every rank streams its own copies."""
    import ubridge_b200 as ub
    from ubridge_b200 import synth as o  # seeded synthetic inputs
    from ubridge_b200 import ops

    dev_index = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(dev_index)
    N, K, M, is_q4k = wl["N"], wl["K"], wl["M"], wl["is_q4k"]
    rng = np.random.default_rng(wl["seed"] + rank)
    fmt = wl_format(wl)
    w_host = np.ascontiguousarray(GEN_WEIGHT(o)[fmt](rng, N, K)).reshape(-1)
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
    ws_bytes = 0 if fmt in ("Q6_K", "Q5_K", "Q4_0") else ops.qmatmul_workspace_bytes(M, N, K, is_q4k)
    gguf_tag = {"Q5_K": 13, "Q4_0": 2}.get(fmt)  # GGML type tags of the formats that only the blob entry takes

    def matmul(y, x, w, workspace, stream):
        if gguf_tag is not None:
            ops.qmatmul_gguf(y, x, w, gguf_tag, M, N, K, x_dtype=x_dtype, out_dtype=y_dtype, stream=stream)
        elif fmt == "Q6_K":
            ops.qmatmul_q6k(y, x, w, M, N, K, x_dtype=x_dtype, out_dtype=y_dtype, stream=stream)
        else:
            ops.qmatmul(y, x, w, M, N, K, is_q4k=is_q4k, x_dtype=x_dtype, out_dtype=y_dtype, workspace=workspace,
                        ws_bytes=ws_bytes, stream=stream)
    ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device="cuda")

    stream = torch.cuda.Stream()
    sp = ctypes.c_void_p(stream.cuda_stream)
    passes = wl.get("passes", 1)

    def one_replay_body():
        for _p in range(passes):
            for c in range(copies):
                matmul(y_dev.data_ptr(), x_dev.data_ptr(), w_dev[c].data_ptr(), ws.data_ptr(), sp)

    with torch.cuda.stream(stream):
        one_replay_body()  # first call resolves symbols and attributes outside any capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_replay_body()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            graph.replay()
        ev0.record(stream)
        for _ in range(5):
            graph.replay()
        ev1.record(stream)
        stream.synchronize()
        k = replays_for(min_seconds, steps, CTL.max(ev0.elapsed_time(ev1) * 1e-3 / 5))
        for _ in range(warmup):
            for _r in range(k):
                graph.replay()
        stream.synchronize()
        CTL.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(dev_index)
        if rank == 0:
            sampler.start()
        ev0.record(stream)
        for _ in range(steps):
            for _r in range(k):
                graph.replay()
        ev1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    ms_total = CTL.max(ms_total)
    ms_step = ms_total / steps

    # Q8_0 / Q6_K decode kernels: M rows are processed 4/2/1 at a time, one launch each
    def decode_launches(m):
        n = 0
        while m > 0:
            t_ = 4 if m >= 4 else (2 if m >= 2 else 1)
            m -= t_
            n += 1
        return n
    if fmt == "Q4_K":
        # decode kernel: up to eight rows per pass; bf16 in and out from nine rows on: one tensor-core launch
        launches_per_call = 1 if M > 16 or (M > 8 and wl["x_bf16"]) else (M + 7) // 8
    elif fmt == "Q8_0":
        if M > 16 and K % 256 == 0:
            launches_per_call = 1  # tensor-core kernel (bf16 in and out here: no conversion launches)
        else:
            launches_per_call = (M + 7) // 8 if K % 2048 == 0 else decode_launches(M)
    else:
        launches_per_call = decode_launches(M)
    calls_per_step = k * copies * passes
    launches = steps * calls_per_step * launches_per_call

    if wl["unit"] == "GB/s":
        value = world * calls_per_step * w_bytes / (ms_step * 1e-3) / 1e9
    else:
        value = world * calls_per_step * 2.0 * M * N * K / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public device API: host activations in, host result out
    e2e, e2e_call = None, None
    if with_e2e:
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
        hx, hy = ctypes.c_void_p(host_x.data_ptr()), ctypes.c_void_p(host_y.data_ptr())

        def e2e_step():  # one copy in, one pass over the weight stack, one copy out, one synchronisation
            lib.ub_memcpy_htod(dev._handle, ctypes.c_void_p(d_x.ptr), hx, host_x.numel())
            for _p in range(passes):
                for c in range(copies):
                    matmul(d_y, d_x, w_e2e[c], d_ws, dev.stream)
            lib.ub_memcpy_dtoh(dev._handle, hy, ctypes.c_void_p(d_y.ptr), host_y.numel())
            dev.synchronize()

        def e2e_call_once(c):  # what one plugin call with host buffers costs: copy, launch, copy, synchronise
            lib.ub_memcpy_htod(dev._handle, ctypes.c_void_p(d_x.ptr), hx, host_x.numel())
            matmul(d_y, d_x, w_e2e[c % copies], d_ws, dev.stream)
            lib.ub_memcpy_dtoh(dev._handle, hy, ctypes.c_void_p(d_y.ptr), host_y.numel())
            dev.synchronize()

        for _ in range(3):
            e2e_step()
        t0 = time.perf_counter()
        e2e_step()
        e2e_reps = max(1, int(np.ceil(min(min_seconds, 1.0) / (steps * max(time.perf_counter() - t0, 1e-6)))))
        CTL.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            for _r in range(e2e_reps):
                e2e_step()
        el = CTL.max(time.perf_counter() - t0)
        per_pass = el / (steps * e2e_reps)
        calls = copies * passes * world
        ev = calls * w_bytes / per_pass / 1e9 if wl["unit"] == "GB/s" else calls * 2.0 * M * N * K / per_pass / 1e12
        e2e = {"value": ev, "unit": wl["unit"], "h2d_bytes_per_step": int(host_x.numel()) * e2e_reps,
               "d2h_bytes_per_step": int(host_y.numel()) * e2e_reps,
               "what": "per step %d x (one H2D of x, %d matmuls, one D2H of y, one synchronise)" % (
                   e2e_reps, copies * passes)}
        n_calls = 200 if M <= 16 else 20
        for c in range(10):
            e2e_call_once(c)
        t0 = time.perf_counter()
        for c in range(n_calls):
            e2e_call_once(c)
        per_call = CTL.max(time.perf_counter() - t0) / n_calls
        cv = world * w_bytes / per_call / 1e9 if wl["unit"] == "GB/s" else world * 2.0 * M * N * K / per_call / 1e12
        e2e_call = {"value": cv, "unit": wl["unit"], "us_per_call": per_call * 1e6,
                    "h2d_bytes_per_call": int(host_x.numel()), "d2h_bytes_per_call": int(host_y.numel())}

    peaks = measured_peaks()
    algo_bytes = w_bytes + M * K * esz + M * N * esz
    avg_launch_s = ms_total * 1e-3 / (steps * calls_per_step)  # per matmul call (all of its launches)
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
                "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                "algorithmic_flops_per_launch": 2.0 * M * N * K, "avg_launch_us": avg_launch_s * 1e6}
    roof["traffic"] = profile_traffic(wl_name)
    return dict(value=value, ms_per_step=ms_step, launches=launches, e2e=e2e, e2e_per_call=e2e_call, roofline=roof,
                clocks=clocks, replays_per_step=k, timed_seconds=ms_total * 1e-3,
                dtype={"Q4_K": "u4+f16 scales -> f32 accumulate", "Q8_0": "i8+f16 scales -> f32 accumulate",
                       "Q6_K": "u6+i8 scales+f16 -> f32 accumulate", "Q5_K": "u5+f16 scales -> f32 accumulate",
                       "Q4_0": "u4+f16 scale -> f32 accumulate"}[fmt])


class ShardedContext:
    """What the sharded workloads of one run share: the device, the NCCL communicator behind the eccl entry
    points, the one-shot peer-memory all-reduce and a device-resident pool of random Q4_K super-blocks from
    which every weight shard is filled (any run of whole super-blocks is a valid Q4_K matrix of any shape)."""

    POOL_BLOCKS = 1 << 18  # 37.7 MB of super-blocks

    def __init__(self, rank, world, torch):
        import ubridge_b200 as ub
        from ubridge_b200 import eccl
        from ubridge_b200 import synth as o

        self.rank, self.world, self.torch, self.ub, self.eccl = rank, world, torch, ub, eccl
        self.dev_index = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.dev_index)
        self.dev = ub.GcuDevice(self.dev_index)
        self.dev.bind_to_thread()
        self.ext = torch.cuda.ExternalStream(self.dev.stream.value)
        self.comm, self.oneshot, self.oneshot_limit = None, None, 0
        if world > 1:
            # the 128-byte unique id travels out of band (the CPU group), as it does in the reference
            uid = CTL.broadcast(eccl.Id().internal() if rank == 0 else None)
            self.comm = eccl.Comm.from_rank(rank, world, eccl.Id(uid))
            # messages of a few KB (the decode path) go through the one-shot peer-memory kernel, larger ones
            # through NCCL; UB_BENCH_ALLREDUCE=nccl forces NCCL for comparison
            self.oneshot_limit = 0 if os.environ.get("UB_BENCH_ALLREDUCE") == "nccl" else 65536
            if self.oneshot_limit:
                self.oneshot = eccl.OneShotAllReduce(self.dev, rank, world, self.oneshot_limit, CTL.all_gather)
            CTL.barrier()
        rng = np.random.default_rng(4242 + 17 * rank)
        pool = o.gen_q4k_weight(rng, self.POOL_BLOCKS // 16, 4096).reshape(-1)
        self.pool = self.dev.htod_sync_copy(pool)
        self.pool_bytes = pool.nbytes
        self.cursor = 0

    def nccl_all_reduce(self, buf, count):
        e = self.eccl
        self.comm.all_reduce(buf, buf, count, e.Bfloat16, e.ReduceOp.Sum, stream=self.dev.stream)

    def all_reduce(self, buf, count):
        if self.oneshot is not None and count * 2 <= self.oneshot_limit and count % 8 == 0:
            self.oneshot.all_reduce(buf, count)
        else:
            self.nccl_all_reduce(buf, count)

    def q4k_matrix(self, rows: int, K: int):
        """A device buffer of rows x K/256 super-blocks filled from the pool (wrapping, at a moving offset)."""
        nbytes = rows * Q4K_ROW_BYTES(K)
        buf = self.dev.alloc(nbytes)
        lib, done = self.ub.lib(), 0
        while done < nbytes:
            n = min(nbytes - done, self.pool_bytes - self.cursor)
            lib.ub_memcpy_dtod(self.dev._handle, ctypes.c_void_p(buf.ptr + done), ctypes.c_void_p(self.pool.ptr + self.cursor), n)
            done += n
            self.cursor = (self.cursor + n) % self.pool_bytes
        return buf

    def close(self):
        self.dev.synchronize()
        if self.comm is not None:
            CTL.barrier()
            if self.oneshot is not None:
                self.oneshot.close()
            self.comm.destroy()
            self.comm = None


def run_sharded(ctx, wl_name, wl, steps, warmup, min_seconds, with_e2e=True):
    """Tensor-parallel (c5) and expert-parallel (c4) workloads: the matrices are split over the ranks, every
    rank streams its shard and the partial outputs meet in all-reduces (strong scaling)."""
    from ubridge_b200 import parallel
    from ubridge_b200 import synth as o

    torch, dev, ext, rank, world, ub = ctx.torch, ctx.dev, ctx.ext, ctx.rank, ctx.world, ctx.ub
    all_reduce = ctx.all_reduce if world > 1 else None
    kind = wl["kind"]
    if kind == "tp":
        H, I, M = wl["hidden"], wl["inter"], wl["M"]
        ql, kvl, il = wl["q_heads"] * wl["head_dim"] // world, wl["kv_heads"] * wl["head_dim"] // world, I // world
        shapes = [(ql + 2 * kvl, H), (H, ql), (2 * il, H), (H, il)]  # this rank's shards, filled at shard shape
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
            ws_ = [ctx.q4k_matrix(n, k) for n, k in shapes]
            layers.append(parallel.TPLinearStack(dev, H, I, wl["q_heads"], wl["kv_heads"], wl["head_dim"], world,
                                                 ws_[0], ws_[1], ws_[2], ws_[3], M, all_reduce,
                                                 fused=ctx.oneshot if world > 1 else None))
        else:
            layers.append(parallel.EPMoELayer(dev, T, H, I, E, wl["top_k"], wl["block"], rank, world,
                                              ctx.q4k_matrix(el * 2 * I, H), ctx.q4k_matrix(el * H, I), all_reduce))
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
    # GPUs the graphs contain the all-reduces
    for layer in layers:
        forward(layer)
    dev.synchronize()
    # the exchange checks itself: the layer's output with the one-shot kernel against the same layer with NCCL
    check = None
    if world > 1 and ctx.oneshot is not None and out_elems * 2 <= ctx.oneshot_limit:
        a = dev.dtoh_sync_copy(layers[0].out, np.uint16, (out_elems,)).copy()
        fused_ = getattr(layers[0], "fused", None)
        layers[0].all_reduce = ctx.nccl_all_reduce
        if fused_ is not None:
            layers[0].fused = None
        forward(layers[0])
        b_ = dev.dtoh_sync_copy(layers[0].out, np.uint16, (out_elems,)).copy()
        layers[0].all_reduce = all_reduce
        if fused_ is not None:
            layers[0].fused = fused_
        fa, fb = o.bf16_bits_to_f32(a).astype(np.float64), o.bf16_bits_to_f32(b_).astype(np.float64)
        check = {"one_shot_vs_nccl_rel_l2": float(np.sqrt(((fa - fb) ** 2).sum() / max((fb ** 2).sum(), 1e-30)))}
    graphs = []
    with torch.cuda.stream(ext):
        for layer in layers:
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=ext, capture_error_mode="thread_local"):
                forward(layer)
            graphs.append(g_)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(3):
            graphs[i % ncopies].replay()
        ev0.record(ext)
        for i in range(ncopies):
            graphs[i].replay()
        ev1.record(ext)
        ext.synchronize()
        k = replays_for(min_seconds, steps, CTL.max(ev0.elapsed_time(ev1) * 1e-3 / ncopies))
        n = 0
        for _ in range(warmup * k):
            graphs[n % ncopies].replay()
            n += 1
        ext.synchronize()
        CTL.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(ctx.dev_index)
        if rank == 0:
            sampler.start()
        ev0.record(ext)
        for _ in range(steps * k):
            graphs[n % ncopies].replay()
            n += 1
        ev1.record(ext)
        ext.synchronize()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
    ms_total = CTL.max(ev0.elapsed_time(ev1))
    ms_step = ms_total / steps
    s_layer = ms_total * 1e-3 / (steps * k)
    # a bounded wait that ran out (one-shot all-reduce, mbarrier rings) leaves its code in the device error word
    status = max(CTL.all_gather(int(dev.device_status())))

    def metric_value(sec):
        if wl["unit"] == "GB/s":
            return total_bytes / sec / 1e9
        if wl["unit"] == "TFLOP/s":
            return flop / sec / 1e12
        return wl["T"] / sec

    value = metric_value(s_layer)
    e2e = None
    if with_e2e:
        # end to end: host activations in, host result out, every pass over the layer.  A single GPU launches
        # the layer eagerly through the API; with several GPUs the pass replays the captured graph between
        # the two copies, so that host launch cost does not hide the collectives.
        host_x = torch.from_numpy(x_host.view(np.uint8).reshape(-1).copy()).pin_memory()
        host_y = torch.empty((out_elems * 2,), dtype=torch.uint8).pin_memory()
        lib = ub.lib()
        e2e_graph = world > 1

        def e2e_pass(i):
            lib.ub_memcpy_htod(dev._handle, ctypes.c_void_p(d_x.ptr), ctypes.c_void_p(host_x.data_ptr()), host_x.numel())
            if e2e_graph:
                with torch.cuda.stream(ext):
                    graphs[i % ncopies].replay()
                out = layers[i % ncopies].out
            else:
                out = forward(layers[i % ncopies])
            lib.ub_memcpy_dtoh(dev._handle, ctypes.c_void_p(host_y.data_ptr()), ctypes.c_void_p(out.ptr), host_y.numel())
            dev.synchronize()

        for i in range(3):
            e2e_pass(i)
        reps = max(1, min(k, int(np.ceil(0.5 / (steps * max(s_layer, 1e-6))))))
        CTL.barrier()
        t0 = time.perf_counter()
        for i in range(steps * reps):
            e2e_pass(i)
        el_s = CTL.max(time.perf_counter() - t0)
        e2e = {"value": metric_value(el_s / (steps * reps)), "unit": wl["unit"],
               "h2d_bytes_per_step": int(host_x.numel()) * reps, "d2h_bytes_per_step": int(host_y.numel()) * reps,
               "launch_mode": "cuda graph" if e2e_graph else "eager"}

    peaks = measured_peaks()
    # per-GPU roofline: this rank's shard bytes (or flop) per pass against one GPU's measured peak
    hbm = shard_bytes / s_layer / 1e9
    tf = flop / world / s_layer / 1e12
    burst = ms_total < 1000.0
    tensor_peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
    if wl["unit"] == "TFLOP/s":
        roof = {"bound": "tensor", "achieved": tf, "peak": tensor_peak, "unit": "TFLOP/s", "frac": tf / tensor_peak,
                "peak_kind": "burst" if burst else "sustained"}
    else:
        roof = {"bound": "hbm", "achieved": hbm, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": hbm / peaks["hbm_gbs"],
                "tensor_frac": tf / tensor_peak}
    roof.update({"traffic": profile_traffic(wl_name), "peak_source": peaks["source"], "per_gpu": True,
                 "algorithmic_bytes_per_pass_per_gpu": shard_bytes, "algorithmic_flops_per_pass": flop,
                 "pass_us": s_layer * 1e6})
    launches = steps * k * layers[0].launches_per_forward
    fused_note = kind == "tp" and world > 1 and getattr(layers[0], "fused", None) is not None and wl["M"] == 1
    # NCCL keeps a communicator alive while a CUDA graph that captured its collectives exists, and
    # ncclCommDestroy waits for those references: release the graphs before anything else is torn down
    dev.synchronize()
    graphs.clear()
    g_ = None
    del layers
    import gc
    gc.collect()
    CTL.barrier()
    return dict(value=value, ms_per_step=ms_step, launches=launches, e2e=e2e, roofline=roof, clocks=clocks,
                dtype="u4+f16 scales -> f32 accumulate", ncopies=ncopies, replays_per_step=k,
                timed_seconds=ms_total * 1e-3, launch_mode="cuda graph", device_status=status, allreduce_check=check,
                allreduce=("in the epilogue of the row-split matmuls (peer stores, last CTA reduces)" if fused_note else
                           ("one-shot peer-memory kernel up to 64 KB, NCCL above" if world > 1 and ctx.oneshot_limit
                            else ("NCCL" if world > 1 else "none"))))


def describe(wl_name, wl, n_gpus, res=None):
    k = res["replays_per_step"] if res else 1
    if "kind" in wl:
        cfg = {"workload": "%s: %s; one step = %d passes over the layer; consecutive passes use distinct weight "
                           "copies (>= 300 MB per GPU in total, larger than L2)" % (wl_name, wl["desc"], k),
               "M": wl.get("M"), "format": "Q4_K", "l2_policy": "inputs larger than L2",
               "parallelism": "%s%d" % (wl["kind"], n_gpus)}
        if res:
            cfg.update({"launch_mode": res["launch_mode"], "weight_copies": res["ncopies"], "allreduce": res["allreduce"]})
    else:
        per_replay = wl["copies"] * wl.get("passes", 1)
        cfg = {"workload": "%s: %s; one step = %d graph replays of %d matmuls over %d distinct weight copies (%.0f MB, "
                           "larger than L2)" % (wl_name, wl["desc"], k, per_replay, wl["copies"],
                                                wl["copies"] * wl["N"] * wl_row_bytes(wl) / 1e6),
               "N": wl["N"], "K": wl["K"], "M": wl["M"], "format": wl_format(wl),
               "l2_policy": "inputs larger than L2", "parallelism": "replicas x%d" % n_gpus}
    if res:
        cfg["replays_per_step"] = k
        cfg["timed_region_s"] = round(res["timed_seconds"], 3)
    return cfg


def short_record(wl_name, wl, n_gpus, res):
    """A secondary / sharded result as carried inside the headline line."""
    rec = {"workload": wl_name, "metric": METRIC_OF[wl["unit"]], "value": res["value"], "unit": wl["unit"],
           "ms_per_step": res["ms_per_step"], "config": describe(wl_name, wl, n_gpus, res),
           "roofline": res["roofline"], "gpu_launches": res["launches"], "clocks": res["clocks"]}
    if "kind" in wl:
        rec["scaling"] = "strong"
        rec["device_status"] = res["device_status"]
        if res["allreduce_check"]:
            rec["allreduce_check"] = res["allreduce_check"]
    return rec


METRIC_OF = {"GB/s": "weight_GBps", "TFLOP/s": "TFLOPS", "tok/s": "moe_tokens_per_s"}
SECONDARY = ["c1", "c2_m4", "c2_m8", "c2_m16", "c3"]   # single-GPU configurations carried by the default line
SHARDED = ["c5_m1", "c5_m512", "c4"]          # strong-scaling configurations carried at every GPU count


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_m1", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU baseline sample")
    ap.add_argument("--min-seconds", type=float, default=2.0, help="least duration of the timed region")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    metric = METRIC_OF[wl["unit"]]
    sharded = "kind" in wl

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
                "config": describe(args.workload, wl, args.gpus),
                "cpu_baseline": {"value": value, "unit": wl["unit"], "cores": cores, "kind": "port",
                                 "sample": "each step: " + sample},
                "e2e": {"value": value, "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if world > 1:
        # leave NCCL's communicator-initialisation lines on: they are the record of how many ranks the
        # data path's communicator really spans
        # (on stderr when this script is the one that switches them on, so that stdout stays the one JSON line)
        if os.environ.get("NCCL_DEBUG", "").upper() not in ("INFO", "TRACE"):
            os.environ["NCCL_DEBUG"] = "INFO"
            os.environ["NCCL_DEBUG_SUBSYS"] = "INIT"
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    import torch
    import torch.distributed as dist

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        # the control plane (barriers, max over ranks, unique-id hand-over) is a CPU group: torch creates no
        # NCCL communicator of its own
        dist.init_process_group("gloo")
    global CTL
    CTL = Control(torch, dist, world)
    ctx = None
    try:
        extras = args.workload == "c2_m1" and not args.no_extras
        if sharded:
            ctx = ShardedContext(rank, world, torch)
            res = run_sharded(ctx, args.workload, wl, args.steps, args.warmup, args.min_seconds)
        else:
            res = run_linear(args.workload, wl, args.steps, args.warmup, args.min_seconds, rank, world, torch)
        secondary, sharded_recs = [], []
        if extras:
            torch.cuda.empty_cache()
            if world == 1:
                for name in SECONDARY:
                    try:
                        r = run_linear(name, WORKLOADS[name], args.steps, args.warmup, min(args.min_seconds, 1.0), rank,
                                       world, torch, with_e2e=False)
                        secondary.append(short_record(name, WORKLOADS[name], world, r))
                    except Exception as exc:  # a secondary record must not take the headline down
                        secondary.append({"workload": name, "error": repr(exc)})
                    torch.cuda.empty_cache()
            ctx = ShardedContext(rank, world, torch)
            for name in SHARDED:
                try:
                    r = run_sharded(ctx, name, WORKLOADS[name], args.steps, args.warmup, min(args.min_seconds, 1.0),
                                    with_e2e=False)
                    sharded_recs.append(short_record(name, WORKLOADS[name], world, r))
                except Exception as exc:
                    sharded_recs.append({"workload": name, "error": repr(exc)})
                torch.cuda.empty_cache()
        if ctx is not None:
            ctx.close()
            ctx = None
        if rank == 0:
            cpu = None
            if world == 1:
                arm = CpuArm(wl)
                v, sample = arm.run(args.cpu_seconds)
                cpu = {"value": v, "unit": wl["unit"], "cores": arm.cores, "kind": "port", "sample": sample}
            line = {"metric": metric, "value": res["value"], "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                    "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": res["dtype"],
                    "data": "synthetic", "config": describe(args.workload, wl, world, res),
                    "roofline": res["roofline"], "cpu_baseline": cpu, "e2e": res["e2e"],
                    "gpu_launches": res["launches"], "clocks": res["clocks"]}
            if res.get("e2e_per_call"):
                line["e2e_per_call"] = res["e2e_per_call"]
            if sharded:
                line["device_status"] = res["device_status"]
                if res["allreduce_check"]:
                    line["allreduce_check"] = res["allreduce_check"]
            if secondary:
                line["secondary"] = secondary
            if sharded_recs:
                line["sharded"] = sharded_recs
            bad = [r for r in ([line] if sharded else []) + sharded_recs if r.get("device_status")]
            if bad:
                line["error"] = "device error word set (a bounded device-side wait ran out): " + ", ".join(
                    "%s=%d" % (r.get("workload", args.workload), r["device_status"]) for r in bad)
            sys.stdout.flush()
            print(json.dumps(line), flush=True)
    finally:
        if ctx is not None:
            try:
                ctx.close()
            except Exception:
                pass
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
