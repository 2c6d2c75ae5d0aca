#!/usr/bin/env python
"""Headline benchmark: strict-FP32 SGEMM TFLOP/s on the square 16384^3 problem, sharded
along M over the GPUs of one box (one process per GPU, no data-path collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one C = A.B over this rank's M-shard (rows = 16384/N) through the C-ABI
library.  `value` is whole-job TFLOP/s with operands resident in HBM; `e2e` is the same
metric through the same call with pinned HOST operands (H2D of A-shard and B, D2H of the
C-shard inside the timed region).  Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_TOTAL = int(os.environ.get("TT_BENCH_N", "16384"))
METRIC = "sgemm_fp32_tflops"
UNIT = "TFLOP/s"

# DRAM bytes (read + write) per launch of sgemm_simt_kernel from one ncu capture, keyed by problem
# edge.  8192 is captured; 16384 is that capture scaled (reads x 8, writes x 4), because a
# 3 GB / 157 ms launch is too large to capture.
NCU_TRAFFIC_BYTES = {8192: 2241620992 + 260361984, 16384: 8 * 2241620992 + 4 * 260361984}


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            # the upper half of the samples are the ones taken under load
            sm_sorted = sorted(sm)
            out["sm_mhz"] = statistics.median(sm_sorted[len(sm_sorted) // 2:])
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def cpu_reference_sample(steps, warmup, rows_hint=None):
    """Times the CPU restatement of the reference's SIMD matmul (all host threads) on a
    bounded row-slab of the same 16384^3 workload.  Returns (tflops, info dict)."""
    import numpy as np

    import oracle
    threads = oracle.set_threads("auto")
    n = N_TOTAL
    rng = np.random.default_rng(0)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    rows = rows_hint or max(threads, 8)
    # grow the slab until one step is at least ~1.5 s of work (bounded by 16 doublings)
    a = rng.uniform(-1, 1, (rows, n)).astype(np.float32)
    for _ in range(16):
        t0 = time.perf_counter()
        oracle.matmul2d(a, b, rows, n, n, n, 1, n, 1)
        dt = time.perf_counter() - t0
        if dt >= 1.5 or rows >= n:
            break
        rows = min(n, rows * 2)
        a = rng.uniform(-1, 1, (rows, n)).astype(np.float32)
    for _ in range(warmup):
        oracle.matmul2d(a, b, rows, n, n, n, 1, n, 1)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.matmul2d(a, b, rows, n, n, n, 1, n, 1)
    dt = (time.perf_counter() - t0) / steps
    tflops = 2.0 * rows * n * n / dt / 1e12
    info = {"value": tflops, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "rows %d of %d (x %d x %d), %d step(s) of %.2f s, C restatement of "
                      "CpuKernels.MatMul2D Axpy path, row-parallel" % (rows, n, n, n, steps, dt)}
    return tflops, dt, info


def time_calls(fn, iters, warmup=3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def peaks(sms, max_mhz):
    """Roofline denominators: FP32 FMA peak derived from the device (the measured-peaks file has no
    FP32 SIMT figure), TF32 dense peak = half the measured BF16 burst figure (same tensor pipe,
    twice the operand width), HBM bandwidth as measured."""
    out = {"fp32_ffma_tflops": sms * 128 * 2 * max_mhz * 1e6 / 1e12}
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        out["tf32_tflops"] = pk["bf16_tflops"] / 2.0
        out["hbm_gbs"] = pk["hbm_gbs"]
        out["source"] = "of measured (MEASURED_PEAKS.json); TF32 = half the BF16 burst figure, derived"
    except (OSError, KeyError, ValueError):
        out["tf32_tflops"] = 1590.0 / 2.0
        out["hbm_gbs"] = 6650.0
        out["source"] = "of fallback (1.59 PFLOP/s BF16, 6.65 TB/s)"
    return out


def sgemm_sweep(rt, sms, max_mhz):
    """Benchmark config 5 on one GPU: M = N = K in {512 ... 8192} x {strict FP32, TF32, 3xTF32},
    TFLOP/s and fraction of the pipe's peak per entry (the north-star fractions are quoted at
    8192^3), with cuBLAS through torch.matmul on the same box, same operands, same event timing as
    the stated comparator (`cublas_same_box`, `vs_cublas` = cuBLAS time / our time; never on the
    product path).  3xTF32 has no cuBLAS counterpart and is compared with cuBLAS strict FP32."""
    import torch

    from tensotron_b200.runtime import TT_MATH_3XTF32, TT_MATH_FP32, TT_MATH_TF32
    pk = peaks(sms, max_mhz)
    out = {"peaks": pk, "sizes": {}}
    for n in (512, 1024, 2048, 4096, 8192):
        a = torch.rand(n * n, device="cuda") * 2 - 1
        b = torch.rand(n * n, device="cuda") * 2 - 1
        c = torch.empty((n, n), device="cuda")
        flop = 2.0 * n ** 3
        iters = {512: 200, 1024: 100, 2048: 50, 4096: 20, 8192: 5}[n]
        entry = {}
        lib = {}
        for name, mode in (("fp32", TT_MATH_FP32), ("tf32", TT_MATH_TF32)):
            ms_lib = cublas_ms(a, b, n, n, n, "NN", mode, iters)
            lib[name] = {"ms": ms_lib, "tflops": flop / ms_lib / 1e9}
        for name, mode in (("fp32", TT_MATH_FP32), ("tf32", TT_MATH_TF32), ("3xtf32", TT_MATH_3XTF32)):
            rt.SetCuBlasMathMode(mode)
            it = iters if name != "fp32" or n < 8192 else 5
            ms = time_calls(lambda: rt.LaunchMatMul(a, b, c, n, n, n, n, 1, n, 1), it)
            tf = flop / ms / 1e9
            e = {"tflops": tf, "ms": ms}
            if name == "fp32":
                e["frac_of_fp32_ffma_peak"] = tf / pk["fp32_ffma_tflops"]
                e["vs_cublas"] = lib["fp32"]["ms"] / ms
            else:
                pipe = tf * (3 if name == "3xtf32" else 1)
                e["tensor_pipe_tflops"] = pipe
                e["frac_of_tf32_peak"] = pipe / pk["tf32_tflops"]
                e["vs_cublas"] = lib["tf32" if name == "tf32" else "fp32"]["ms"] / ms
            entry[name] = e
        entry["cublas_same_box"] = lib
        out["sizes"][str(n)] = entry
        del a, b, c
    rt.SetCuBlasMathMode(TT_MATH_FP32)
    return out


def timed_max_ms(fn, iters, world, warmup=3):
    """CUDA-event time per call after warm-up, bracketed by a barrier, max over the ranks."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def sgemm_16384_tensor_modes(rt, rank, world, sms, max_mhz):
    """The headline product (16384^3, rows of A and C sharded over the ranks, B replicated, no
    collective) in the tensor-core modes: whole-job TFLOP/s at this N, max-over-ranks time."""
    import torch

    from tensotron_b200.runtime import TT_MATH_3XTF32, TT_MATH_FP32, TT_MATH_TF32
    n = N_TOTAL
    rows = n // world
    gen = torch.Generator(device="cuda").manual_seed(4321 + rank)
    a = torch.rand((rows, n), generator=gen, device="cuda") * 2 - 1
    gen.manual_seed(98)
    b = torch.rand((n, n), generator=gen, device="cuda") * 2 - 1
    c = torch.empty((rows, n), device="cuda")
    pk = peaks(sms, max_mhz)
    out = {"rows_per_gpu": rows}
    for name, mode, iters in (("tf32", TT_MATH_TF32, 10), ("3xtf32", TT_MATH_3XTF32, 5)):
        rt.SetCuBlasMathMode(mode)
        ms = timed_max_ms(lambda: rt.LaunchMatMul(a, b, c, rows, n, n, n, 1, n, 1), iters, world)
        tf = 2.0 * n ** 3 / ms / 1e9
        pipe = tf * (3 if name == "3xtf32" else 1)
        out[name] = {"tflops": tf, "ms": ms, "tensor_pipe_tflops_per_gpu": pipe / world,
                     "frac_of_tf32_peak": pipe / world / pk["tf32_tflops"]}
    rt.SetCuBlasMathMode(TT_MATH_FP32)
    rt.Check()
    return out


def small_configs(rt):
    """Configs 1 and 2 (latency-bound): device time per call under CUDA-graph replay, the regime
    the reference runs small networks in, plus the eager host cost and the launch counts."""
    import time

    import torch

    def replay_us(fn, iters=20, replays=10):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        host_us = (time.perf_counter() - t0) / iters * 1e6
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (iters * replays) * 1e3, host_us

    out = {}
    a = torch.rand((256, 512), device="cuda") * 2 - 1
    b = torch.rand((512, 256), device="cuda") * 2 - 1
    c = torch.empty((256, 256), device="cuda")
    l0 = rt.Stats()["launches"]
    rt.LaunchMatMul(a, b, c, 256, 256, 512, 512, 1, 256, 1)
    launches = rt.Stats()["launches"] - l0
    us, host = replay_us(lambda: rt.LaunchMatMul(a, b, c, 256, 256, 512, 512, 1, 256, 1))
    out["matmul_256x256x512"] = {"graph_replay_us": us, "eager_host_us": host, "launches": launches,
                                 "tflops": 2.0 * 256 * 256 * 512 / us / 1e6}
    x = torch.randn((64, 128), device="cuda")
    w = (torch.rand((64, 128), device="cuda") * 2 - 1) / 128 ** 0.5
    bias = torch.zeros(64, device="cuda")
    y, dy = torch.empty((64, 64), device="cuda"), torch.randn((64, 64), device="cuda")
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(bias)

    def fwd_bwd():
        rt.LaunchLinearForward(x, w, bias, y, 64, 64, 128, 1)
        rt.LaunchLinearBackward(x, w, y, dy, dx, dw, db, 64, 64, 128, 1)

    l0 = rt.Stats()["launches"]
    fwd_bwd()
    launches = rt.Stats()["launches"] - l0
    us, host = replay_us(fwd_bwd)
    out["linear_relu_64x128x64_fwd_bwd"] = {"graph_replay_us": us, "eager_host_us": host, "launches": launches}

    # The reference's replay sweep (examples/Tensotron.Examples/BenchExample.cs:140-176): Tanh MLPs,
    # MSE loss, ClipGradNorm(0.5), Adam(1e-3); whole training step per replayed graph node set.
    # The control / PPO sized networks run as ONE launch (tt_mlp_train_step); the 128-256-256-10
    # entry is too wide for one cluster and runs layer by layer.
    from tensotron_b200.mlp import MlpTrainer
    for name, dims, batch in (("ctrl_net_b1", [8, 64, 64, 2], 1), ("ppo_b64", [8, 64, 64, 2], 64),
                              ("ppo_b512", [8, 64, 64, 2], 512), ("critic_4_32_32_1_b64", [4, 32, 32, 1], 64),
                              ("mlp_b256_128_256_256_10", [128, 256, 256, 10], 256)):
        tr = MlpTrainer(dims, rt=rt, lr=1e-3, seed=3, act="tanh", loss="mse", max_grad_norm=0.5, fused="auto")
        xs = torch.rand((batch, dims[0]), device="cuda") - 0.5
        ts = torch.zeros((batch, dims[-1]), device="cuda")
        l0 = rt.Stats()["launches"]
        tr.step(xs, ts)
        launches = rt.Stats()["launches"] - l0
        us, host = replay_us(lambda: tr.step(xs, ts), iters=10)
        out["train_step_" + name] = {"graph_replay_us": us, "eager_host_us": host, "launches": launches,
                                     "one_launch": bool(tr.last_step_fused), "batch": batch, "dims": dims}
    return out


def bmm_config3(rt, rank=0, world=1):
    """Config 3: A [32,1,384,256] x B [1,16,256,192] -> [32,16,384,192] through LaunchMatMulBatched
    (the reference issues 512 cuBLAS calls), the outer batch axis (32) split over the ranks --
    each rank one launch over its 32 / world entries of A, B replicated, no collective.  FP32, TF32
    and 3xTF32; whole-job numbers with the max-over-ranks time.  In TF32 the 151 MB output write
    makes it HBM-bound, so achieved GB/s of algorithmic bytes (per GPU) is reported too."""
    import torch

    from tensotron_b200 import runtime
    from tensotron_b200.mlp import shard_rows
    from tensotron_b200.runtime import TT_MATH_3XTF32, TT_MATH_FP32, TT_MATH_TF32
    i0, i1 = shard_rows(32, world, rank)
    nb = i1 - i0
    gen = torch.Generator(device="cuda").manual_seed(7)
    a = (torch.rand((32, 1, 384, 256), generator=gen, device="cuda") * 2 - 1)[i0:i1].contiguous()
    gen.manual_seed(8)
    b = torch.rand((1, 16, 256, 192), generator=gen, device="cuda") * 2 - 1
    c = torch.empty((max(nb, 1), 16, 384, 192), device="cuda")
    dims, aBs, bBs = runtime.broadcast_batch([nb, 1], [98304, 98304], [1, 16], [786432, 49152])
    flop = 512 * 2.0 * 384 * 192 * 256
    nbytes = 4.0 * (32 * 384 * 256 + b.numel() * world + 32 * 16 * 384 * 192)   # whole job; B once per GPU
    out = {"algorithmic_bytes": nbytes, "flop": flop, "batch_entries_per_gpu": nb, "hbm_peak_gbs": peaks(148, 1965.0)["hbm_gbs"]}

    def call():
        if nb > 0:
            rt.LaunchMatMulBatched(a, b, c, nb * 16, 384, 192, 256, 256, 1, 192, 1, dims, aBs, bBs)

    for name, mode in (("fp32", TT_MATH_FP32), ("tf32", TT_MATH_TF32), ("3xtf32", TT_MATH_3XTF32)):
        rt.SetCuBlasMathMode(mode)
        ms = timed_max_ms(call, 20, world)
        out[name] = {"ms": ms, "tflops": flop / ms / 1e9, "hbm_gbs_per_gpu": nbytes / world / ms / 1e6,
                     "frac_of_hbm": nbytes / world / ms / 1e6 / out["hbm_peak_gbs"]}
    rt.SetCuBlasMathMode(TT_MATH_FP32)
    rt.Check()
    return out


def mlp_steps_per_s(rt, rank, world, local_rank, pg, steps=10, warmup=3):
    """Config 4: 784-4096-4096-4096-10 MLP, global batch 8192 split over the ranks,
    cross-entropy on random labels, Adam lr 1e-3.  Gradient exchange: the peer-memory path
    (weight-gradient tiles stored into the owner's memory from the GEMM epilogue, owner-side
    sum + Adam, parameters stored back to every rank); the per-layer NCCL all-reduce form
    (plain Adam on one GPU) is timed beside it ("*_nccl")."""
    import torch
    import torch.distributed as dist

    from tensotron_b200.mlp import MlpTrainer, shard_rows
    from tensotron_b200.runtime import TT_MATH_FP32, TT_MATH_TF32
    res = {"scaling": "strong: global batch 8192 split over the ranks (the '*_weak' runs keep 8192 rows per rank)"}
    runs = [("fp32", TT_MATH_FP32, "peer", 8192), ("tf32", TT_MATH_TF32, "peer", 8192),
            ("fp32_nccl", TT_MATH_FP32, "nccl", 8192), ("tf32_nccl", TT_MATH_TF32, "nccl", 8192)]
    if world > 1:
        runs += [("fp32_weak", TT_MATH_FP32, "peer", 8192 * world), ("tf32_weak", TT_MATH_TF32, "peer", 8192 * world)]
    x = y = None
    cur_gb = 0
    for name, mode, exchange, gb in runs:
        if gb != cur_gb:
            del x, y
            s, e = shard_rows(gb, world, rank)
            gen = torch.Generator(device="cuda").manual_seed(0)
            x = torch.randn((gb, 784), generator=gen, device="cuda")[s:e].contiguous()
            gen.manual_seed(1)
            y = torch.randint(0, 10, (gb,), generator=gen, device="cuda", dtype=torch.int32)[s:e].contiguous()
            cur_gb = gb
        tr, err = None, None
        try:
            tr = MlpTrainer([784, 4096, 4096, 4096, 10], rt=rt, device=local_rank, lr=1e-3, seed=2,
                            process_group=pg, math_mode=mode, exchange=exchange)
        except Exception as ex:     # e.g. peer mapping refused by the platform: report, keep the other runs
            err = "%s: %s" % (type(ex).__name__, ex)
        if world > 1:
            # every rank skips the run when any rank failed to set it up (a rank that went on alone
            # would wait in its first collective for the others)
            ok = torch.tensor([0.0 if err else 1.0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0.0 and err is None:
                err = "set-up failed on another rank"
        if err is not None:
            if tr is not None:
                tr.close()
            res[name] = {"error": err}
            continue
        for _ in range(warmup):
            tr.step(x, y, global_batch=gb)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            loss = tr.step(x, y, global_batch=gb)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        lt = loss.double().clone()
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(lt)
        ms = t.item() / steps
        res[name] = {"steps_per_s": 1e3 / ms, "ms_per_step": ms, "loss": lt.item(), "exchange": exchange,
                     "global_batch": gb,
                     "tflops": 1756.5 * (gb / 8192.0) / ms}      # 1756.5 GFLOP of GEMM work per 8192 rows
        rt.Check()
        tr.close()
        del tr
    if world > 1:
        # run-to-run bit stability of the NCCL form (algorithm and protocol pinned): two runs of
        # three steps from the same initial state must end in identical parameters on every rank
        s, e = shard_rows(8192, world, rank)
        gen = torch.Generator(device="cuda").manual_seed(0)
        xs = torch.randn((8192, 784), generator=gen, device="cuda")[s:e].contiguous()
        gen.manual_seed(1)
        ys = torch.randint(0, 10, (8192,), generator=gen, device="cuda", dtype=torch.int32)[s:e].contiguous()
        finals = []
        for _ in range(2):
            tr = MlpTrainer([784, 4096, 4096, 4096, 10], rt=rt, device=local_rank, lr=1e-3, seed=2,
                            process_group=pg, math_mode=TT_MATH_FP32, exchange="nccl")
            for _ in range(3):
                tr.step(xs, ys, global_batch=8192)
            torch.cuda.synchronize()
            finals.append(tr.params.clone())
            tr.close()
            del tr
        same = torch.tensor([1.0 if torch.equal(finals[0], finals[1]) else 0.0], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        res["nccl_bitwise_repeatable"] = bool(same.item() == 1.0)
        res["nccl_pinned"] = {"NCCL_ALGO": os.environ.get("NCCL_ALGO"), "NCCL_PROTO": os.environ.get("NCCL_PROTO")}
    rt.SetCuBlasMathMode(TT_MATH_FP32)
    return res


def cublas_ms(a, b, M, N, K, lay, mode, iters):
    """Comparator, never on the product path: the same product through torch.matmul (cuBLAS),
    strict FP32 (allow_tf32 off) for math mode 0, TF32 math otherwise.  a / b are flat operands in
    the storage LAYOUT names."""
    import torch
    a2 = a.view(M, K) if lay[0] == "N" else a.view(K, M).t()
    b2 = b.view(K, N) if lay[1] == "N" else b.view(N, K).t()
    out = torch.empty(M, N, device=a.device)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = mode != 0
    try:
        return time_calls(lambda: torch.matmul(a2, b2, out=out), iters)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def check_row_slab(a, b, c, n, count=16):
    """`count` rows of C = A.B (spread over the shard, all columns) against the CPU oracle:
    max |err| and the strict-FP32 acceptance bound 1e-5 * sqrt(K) * max|A| * max|B|."""
    import numpy as np
    import torch

    import oracle
    rows = a.shape[0]
    idx = sorted(set([0, rows - 1] + [int(v) for v in np.random.default_rng(5).choice(rows, size=min(rows, count) - 2, replace=False)]))
    sel = torch.tensor(idx, device=a.device)
    a_rows = a.index_select(0, sel).cpu().numpy()
    b_host = b.cpu().numpy()
    got = c.index_select(0, sel).cpu().numpy()
    oracle.set_threads("auto")
    exp = oracle.matmul2d(a_rows, b_host, len(idx), n, n, n, 1, n, 1)
    err = float(np.abs(got - exp).max())
    bound = float(1e-5 * np.sqrt(n) * np.abs(a_rows).max() * np.abs(b_host).max())
    return {"max_err": err, "bound": bound, "ok": bool(err <= bound), "rows_checked": len(idx),
            "against": "CPU oracle (C restatement of CpuKernels.MatMul2D) on the same operands"}


def run_one(spec):
    """--one MxNxK LAYOUT VARIANT MODE ITERS [graph] [cublas]: times one GEMM shape through the C-ABI
    library (the command the ncu captures summarised under profiles/ run).  LAYOUT is NN / NT /
    TN (N = the operand is stored row-major as given, T = stored transposed and read through
    swapped strides); VARIANT as in tt_set_variant (0 = automatic); MODE is the math mode
    (0 strict FP32, 3 TF32, 4 3xTF32).  With the trailing word `graph` the ITERS launches are
    also captured into one CUDA graph and replayed: device time without per-call host cost."""
    import torch

    from tensotron_b200.runtime import TensorRuntime
    M, N, K = (int(x) for x in spec[0].split("x"))
    lay, variant, mode, iters = spec[1], int(spec[2]), int(spec[3]), int(spec[4])
    rt = TensorRuntime(0, 2048 << 20)
    rt.SetCuBlasMathMode(mode)
    rt.SetVariant(variant)
    a = torch.rand(M * K, device="cuda") * 2 - 1
    b = torch.rand(K * N, device="cuda") * 2 - 1
    c = torch.empty(M, N, device="cuda")
    aMs, aKs = (K, 1) if lay[0] == "N" else (1, M)
    bKs, bNs = (N, 1) if lay[1] == "N" else (1, K)
    call = lambda: rt.LaunchMatMul(a, b, c, M, N, K, aMs, aKs, bKs, bNs)
    ms = time_calls(call, iters)
    rt.Check()
    print("ok %dx%dx%d %s v%d m%d: %.4f ms %.2f TF/s" % (M, N, K, lay, variant, mode, ms, 2.0 * M * N * K / ms / 1e9))
    if "cublas" in spec[5:]:
        # comparator only: the library GEMM (cuBLAS through torch.matmul) on the same operands
        ms_lib = cublas_ms(a, b, M, N, K, lay, mode, iters)
        print("   cuBLAS (torch.matmul, allow_tf32=%s): %.4f ms %.2f TF/s  -> ours / cuBLAS = %.3f"
              % (mode != 0, ms_lib, 2.0 * M * N * K / ms_lib / 1e9, ms_lib / ms))
    if "graph" in spec[5:]:
        t0 = time.perf_counter()
        for _ in range(iters):
            call()
        host_us = (time.perf_counter() - t0) / iters * 1e6
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                call()
        us = time_calls(g.replay, 5, warmup=1) / iters * 1e3
        print("   graph replay: %.2f us per launch (%.2f TF/s); host call cost %.2f us"
              % (us, 2.0 * M * N * K / us / 1e6, host_us))


def run_one_bmm(spec):
    """--one-bmm MODE ITERS [transposed_b]: times benchmark config 3, A [32,1,384,256] x
    B [1,16,256,192] -> [32,16,384,192], as one LaunchMatMulBatched call.  With `transposed_b` B is
    stored [1,16,192,256] and read through bKs = 1, bNs = 256."""
    import torch

    from tensotron_b200 import runtime
    from tensotron_b200.runtime import TensorRuntime
    mode, iters = int(spec[0]), int(spec[1])
    tb = len(spec) > 2 and spec[2] == "transposed_b"
    rt = TensorRuntime(0, 1 << 30)
    rt.SetCuBlasMathMode(mode)
    a = torch.rand((32, 1, 384, 256), device="cuda") * 2 - 1
    b = torch.rand((1, 16, 192, 256) if tb else (1, 16, 256, 192), device="cuda") * 2 - 1
    c = torch.empty((32, 16, 384, 192), device="cuda")
    dims, aBs, bBs = runtime.broadcast_batch([32, 1], [98304, 98304], [1, 16], [786432, 49152])
    bKs, bNs = (1, 256) if tb else (192, 1)
    ms = time_calls(lambda: rt.LaunchMatMulBatched(a, b, c, 512, 384, 192, 256, 256, 1, bKs, bNs, dims, aBs, bBs), iters)
    rt.Check()
    nbytes = 4.0 * (a.numel() + b.numel() + c.numel())
    print("ok bmm config 3 m%d%s: %.1f us %.2f TF/s %.0f GB/s of algorithmic bytes" % (
        mode, " (B transposed)" if tb else "", ms * 1e3, 512 * 2.0 * 384 * 192 * 256 / ms / 1e9, nbytes / ms / 1e6))


def run_one_mlp(spec):
    """--one-mlp ROWS MODE EXCHANGE STEPS: runs STEPS training steps of the benchmark MLP
    (784-4096-4096-4096-10, cross-entropy, Adam) on ROWS rows on one GPU -- ROWS = 1024 is one rank's
    share of the 8-GPU strong-scaling run -- and prints the time per step.  EXCHANGE is `peer` (the
    exchange calls at world size 1) or `none` (plain backward + one Adam launch).  The command the
    per-kernel launch list of a data-parallel rank's step is captured from."""
    import torch

    from tensotron_b200.mlp import MlpTrainer
    from tensotron_b200.runtime import TensorRuntime
    rows, mode, exchange, steps = int(spec[0]), int(spec[1]), spec[2], int(spec[3])
    rt = TensorRuntime(0, 1024 << 20)
    tr = MlpTrainer([784, 4096, 4096, 4096, 10], rt=rt, lr=1e-3, seed=2, math_mode=mode,
                    exchange="peer" if exchange == "peer" else "nccl")
    x = torch.randn((rows, 784), device="cuda")
    y = torch.randint(0, 10, (rows,), device="cuda", dtype=torch.int32)
    ms = time_calls(lambda: tr.step(x, y, global_batch=8192), steps)
    rt.Check()
    print("ok mlp 784-4096x3-10 rows %d m%d %s: %.3f ms per step (%.1f TF/s of GEMM work)"
          % (rows, mode, exchange, ms, 1756.5 * rows / 8192.0 / ms))
    tr.close()


def run_one_step(spec):
    """--one-step DIMS BATCH STEPS: times the one-launch training step (tt_mlp_train_step) of a small
    Tanh MLP with MSE loss, ClipGradNorm(0.5) and Adam(1e-3) -- DIMS like 8,64,64,2 -- eagerly and
    under CUDA-graph replay (10 steps per graph)."""
    import torch

    from tensotron_b200.mlp import MlpTrainer
    from tensotron_b200.runtime import TensorRuntime
    dims, batch, steps = [int(v) for v in spec[0].split(",")], int(spec[1]), int(spec[2])
    rt = TensorRuntime(0, 64 << 20)
    tr = MlpTrainer(dims, rt=rt, lr=1e-3, seed=3, act="tanh", loss="mse", max_grad_norm=0.5, fused=True)
    x = torch.rand((batch, dims[0]), device="cuda") - 0.5
    t = torch.zeros((batch, dims[-1]), device="cuda")
    ms = time_calls(lambda: tr.step(x, t), steps, warmup=5)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(10):
            tr.step(x, t)
    us = time_calls(g.replay, 10, warmup=2) / 10 * 1e3
    rt.Check()
    print("ok one-launch step %s batch %d: %.2f us eager, %.2f us per step under graph replay"
          % (spec[0], batch, ms * 1e3, us))


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU path on the host cores, rank 0 only."""
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    tflops, dt, info = cpu_reference_sample(steps, min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "sgemm_fp32 %d^3 (C = A.B, row-major, uniform[-1,1))" % N_TOTAL,
                   "note": "reference = CPU restatement of the C# SIMD backend (no .NET on this box); "
                           "each step is a bounded row-slab of the workload"},
        "cpu_baseline": info,
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def bind_to_gpu_numa_node(local_rank):
    """Runs this rank on the CPUs of the NUMA node its GPU hangs off, before any pinned host buffer is
    allocated: first-touch then places the buffers in that node's memory, so the host <-> device copies
    of the end-to-end leg do not cross the socket interconnect.  Returns the node, or None when the
    platform does not say (no sysfs entry, a single node, a container without the CPUs)."""
    try:
        import torch
        pr = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError):
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--one", nargs="+", metavar="ARG", help="MxNxK LAYOUT VARIANT MODE ITERS [graph]: time one GEMM shape and exit")
    ap.add_argument("--one-bmm", nargs="+", metavar="ARG", help="MODE ITERS [transposed_b]: time benchmark config 3 and exit")
    ap.add_argument("--one-mlp", nargs="+", metavar="ARG", help="ROWS MODE EXCHANGE STEPS: time the benchmark MLP step on ROWS rows and exit")
    ap.add_argument("--one-step", nargs="+", metavar="ARG", help="DIMS BATCH STEPS: time the one-launch small-MLP training step and exit")
    ap.add_argument("--one-small", action="store_true", help="time the latency-bound small configurations (graph replay) and exit")
    args = ap.parse_args()
    if args.one_small:
        from tensotron_b200.runtime import TensorRuntime
        print(json.dumps(small_configs(TensorRuntime(0, 256 << 20)), indent=1))
        return
    if args.one:
        return run_one(args.one)
    if args.one_bmm:
        return run_one_bmm(args.one_bmm)
    if args.one_mlp:
        return run_one_mlp(args.one_mlp)
    if args.one_step:
        return run_one_step(args.one_step)
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    rank = env_int("RANK", 0)
    world = env_int("WORLD_SIZE", 1)
    local_rank = env_int("LOCAL_RANK", 0)

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    from tensotron_b200.runtime import TT_MATH_FP32, TensorRuntime

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # One algorithm and one protocol for every NCCL all-reduce of the gradient exchange's
        # "nccl" form: the order in which the ranks' contributions are added is then fixed, and the
        # step is bit-stable from run to run (checked below, `nccl_bitwise_repeatable`).
        os.environ.setdefault("NCCL_ALGO", "Ring")
        os.environ.setdefault("NCCL_PROTO", "Simple")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # raises if the CUDA library is missing: no fallback.  4.25 GiB workspace: 3xTF32 keeps hi / lo
    # copies of both operands there (16384^3 on one GPU: 2 x (1 + 1) GiB).
    rt = TensorRuntime(local_rank, 4352 << 20)
    rt.SetCuBlasMathMode(TT_MATH_FP32)
    n = N_TOTAL
    if n % world != 0:
        raise SystemExit("world size must divide %d" % n)
    rows = n // world
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    a = torch.rand((rows, n), generator=gen, device="cuda") * 2 - 1     # this rank's M-shard of A
    gen.manual_seed(99)
    b = torch.rand((n, n), generator=gen, device="cuda") * 2 - 1        # B replicated
    c = torch.empty((rows, n), device="cuda")
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        rt.LaunchMatMul(a, b, c, rows, n, n, n, 1, n, 1)

    for _ in range(args.warmup):
        step()
    barrier()
    rt.ResetCounters()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = rt.Stats()["launches"]
    clocks = sampler.stop() if rank == 0 else None
    rt.Check()

    # ---- correctness of the very call that was timed (outside the timed region): a sample of rows
    # of this rank's C against the CPU oracle at the strict-FP32 bound ----
    check = None
    if rank == 0:
        check = check_row_slab(a, b, c, n)

    # ---- end to end: pinned host operands, copies inside the timed region ----
    # B: the job's inputs cross PCIe once.  Each rank copies a 1 / world row slice of B from its
    # host buffer and one NCCL all-gather lands the whole B in every rank's local HBM (the GEMM's
    # operands and tensor maps are local memory only).
    brow = n // world
    all_cpus = os.sched_getaffinity(0)
    numa = bind_to_gpu_numa_node(local_rank)   # first touch of the pinned buffers below happens on the GPU's node
    ha = torch.empty((rows, n), pin_memory=True).copy_(a)
    hb = torch.empty((brow, n), pin_memory=True).copy_(b[rank * brow:(rank + 1) * brow])
    hc = torch.empty((rows, n), pin_memory=True).zero_()
    os.sched_setaffinity(0, all_cpus)          # the host buffers are placed: give the CPU legs their cores back
    e2e_steps = max(1, min(args.steps, 10))

    # Every step copies its operands from pinned host memory and returns its C-shard to the
    # host.  A step is cut into row chunks on three streams (H2D, compute, D2H) so the copies
    # of one chunk overlap the GEMM of another; two device buffer sets alternate between
    # steps so step j+1 may start copying while step j still computes.
    n_chunks = 4 if rows % 4 == 0 and rows >= 1024 else 1
    crow = rows // n_chunks
    s_h2d, s_d2h = torch.cuda.Stream(), torch.cuda.Stream()
    sets = [(a, b, c), (torch.empty_like(a), torch.empty_like(b), torch.empty_like(c))]
    d2h_done = [[None] * n_chunks for _ in range(2)]     # per set, per chunk: event of the last D2H
    comp_done = [None, None]                             # per set: event of the last GEMM reading it

    def e2e_step(j):
        da, db, dc = sets[j % 2]
        with torch.cuda.stream(s_h2d):
            if comp_done[j % 2] is not None:
                s_h2d.wait_event(comp_done[j % 2])       # the set's previous GEMMs are done reading
            db[rank * brow:(rank + 1) * brow].copy_(hb, non_blocking=True)
            if world > 1:
                dist.all_gather_into_tensor(db, db[rank * brow:(rank + 1) * brow])   # in place, on s_h2d
            ev_b = torch.cuda.Event()
            ev_b.record(s_h2d)
            ev_a = []
            for i in range(n_chunks):
                da[i * crow:(i + 1) * crow].copy_(ha[i * crow:(i + 1) * crow], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_h2d)
                ev_a.append(ev)
        stream.wait_event(ev_b)
        for i in range(n_chunks):
            stream.wait_event(ev_a[i])
            if d2h_done[j % 2][i] is not None:
                stream.wait_event(d2h_done[j % 2][i])    # the C chunk was copied out before reuse
            rt.LaunchMatMul(da[i * crow:(i + 1) * crow], db, dc[i * crow:(i + 1) * crow],
                            crow, n, n, n, 1, n, 1, stream=stream)
            ev_c = torch.cuda.Event()
            ev_c.record(stream)
            with torch.cuda.stream(s_d2h):
                s_d2h.wait_event(ev_c)
                hc[i * crow:(i + 1) * crow].copy_(dc[i * crow:(i + 1) * crow], non_blocking=True)
                ev_d = torch.cuda.Event()
                ev_d.record(s_d2h)
            d2h_done[j % 2][i] = ev_d
        comp_done[j % 2] = ev_c

    def e2e_drain():
        for per_set in d2h_done:
            for ev in per_set:
                if ev is not None:
                    stream.wait_event(ev)

    e2e_step(0)
    e2e_drain()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    s_h2d.wait_event(e0)
    for j in range(e2e_steps):
        e2e_step(j + 1)
    e2e_drain()                                          # the last result has reached the host
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    del sets, s_h2d, s_d2h

    del ha, hb, hc
    extras = {}
    if not args.no_extras:
        pg = dist.group.WORLD if world > 1 else None
        del a, b, c
        torch.cuda.empty_cache()
        def guarded(name, fn):
            # an extra never costs the headline line: a failure is reported in its place
            try:
                extras[name] = fn()
            except Exception as ex:
                extras[name] = {"error": "%s: %s" % (type(ex).__name__, ex)}

        props0 = torch.cuda.get_device_properties(local_rank)
        sms0 = props0.multi_processor_count
        mhz0 = 1965.0
        if world > 1:
            mt = torch.tensor([(clocks or {}).get("sm_max_mhz") or 0.0], device="cuda", dtype=torch.float64)
            dist.broadcast(mt, 0)
            mhz0 = mt.item() or 1965.0
        else:
            mhz0 = (clocks or {}).get("sm_max_mhz") or 1965.0
        # short, latency- and bandwidth-bound measurements first, the long tensor-pipe runs (which heat
        # the part into its power cap) last
        guarded("bmm_32x16_384x256x192", lambda: bmm_config3(rt, rank, world))
        if world == 1:
            guarded("small_configs", lambda: small_configs(rt))
            guarded("sgemm_sweep", lambda: sgemm_sweep(rt, sms0, mhz0))
        guarded("mlp_784_4096x3_10_batch8192", lambda: mlp_steps_per_s(rt, rank, world, local_rank, pg))
        guarded("sgemm_16384_tensor_modes", lambda: sgemm_16384_tensor_modes(rt, rank, world, sms0, mhz0))

    t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()

    if rank == 0:
        flop_total = 2.0 * n * n * n
        ms_per_step = ms / args.steps
        value = flop_total / (ms_per_step * 1e-3) / 1e12
        e2e_value = flop_total / (e2e_ms / e2e_steps * 1e-3) / 1e12
        props = torch.cuda.get_device_properties(local_rank)
        sms = props.multi_processor_count
        max_mhz = (clocks or {}).get("sm_max_mhz") or 1965.0
        peak = sms * 128 * 2 * max_mhz * 1e6 / 1e12           # FP32 FFMA lanes x 2 flop x clock
        per_gpu = value / world
        roof = {
            "bound": "fp32_ffma", "achieved": per_gpu, "peak": peak, "unit": UNIT,
            "frac": per_gpu / peak, "traffic": NCU_TRAFFIC_BYTES.get(n) if world == 1 else None,
            "traffic_is_scaled": n != 8192,
            "traffic_note": "ncu DRAM bytes per launch; 16384 is the 8192^3 capture scaled (reads x 8, writes x 4)",
            "peak_source": "derived: %d SMs x 128 FP32 lanes x 2 x %.0f MHz (max SM clock); the "
                           "measured-peaks file has no FP32 SIMT figure" % (sms, max_mhz),
            "kernel": "sgemm_simt_kernel<MN-major A (transposed once into the workspace), N-major B>, whole waves of "
                      "256x128 tiles, a remainder of at most half a wave cut into k-aligned ranges; "
                      "`achieved` is over the whole step, transposition included",
            "algorithmic_flops_per_launch": 2.0 * rows * n * n,
        }
        if clocks and clocks.get("sm_mhz"):
            roof["frac_at_sampled_clock"] = per_gpu / (sms * 128 * 2 * clocks["sm_mhz"] * 1e6 / 1e12)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "sgemm_fp32 %d^3 (C = A.B, row-major, uniform[-1,1)), strict FP32, "
                                   "sharded along M over %d GPU(s)" % (n, world),
                       "rows_per_gpu": rows, "l2": "operands (%.0f MiB A-shard + %.0f MiB B) exceed the 126 MB L2"
                       % (rows * n * 4 / 2 ** 20, n * n * 4 / 2 ** 20)},
            "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")} if clocks else None,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": (rows * n + brow * n) * 4 * world,
                    "d2h_bytes_per_step": rows * n * 4 * world, "steps": e2e_steps,
                    "per_rank": "H2D %d rows of A + %d rows of B, D2H %d rows of C" % (rows, brow, rows),
                    "b_placement": "local" if world == 1 else "each rank copies 1/%d of B from the host, one NCCL all-gather "
                                   "lands the whole B in every rank's HBM" % world,
                    "pipeline": "%d row chunks per step on H2D / compute / D2H streams, two buffer sets" % n_chunks,
                    "host_numa_node": numa},
            "gpu_launches": launches,
            "check": check,
            "roofline": roof,
        }
        if extras:
            line["extras"] = extras
        if world == 1 and not args.no_cpu_baseline:
            _, _, info = cpu_reference_sample(1, 0)
            line["cpu_baseline"] = info
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
