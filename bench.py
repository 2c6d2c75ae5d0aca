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
NCU_TRAFFIC_BYTES = {8192: 3366821376 + 254345472, 16384: 8 * 3366821376 + 4 * 254345472}


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


def sgemm_modes_8192(rt, sms, max_mhz):
    """North-star sizes: 8192^3 in strict FP32, TF32 and 3xTF32 (single GPU)."""
    import torch

    from tensotron_b200.runtime import TT_MATH_3XTF32, TT_MATH_FP32, TT_MATH_TF32
    n = 8192
    a = torch.rand((n, n), device="cuda") * 2 - 1
    b = torch.rand((n, n), device="cuda") * 2 - 1
    c = torch.empty((n, n), device="cuda")
    flop = 2.0 * n ** 3
    fp32_peak = sms * 128 * 2 * max_mhz * 1e6 / 1e12
    tf32_peak = None
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        tf32_peak = peaks["bf16_tflops"] / 2.0
        src = "derived: half of the measured BF16 burst peak (MEASURED_PEAKS.json)"
    except (OSError, KeyError, ValueError):
        tf32_peak = 1590.0 / 2.0
        src = "derived: half of the fallback BF16 peak (1.59 PFLOP/s)"
    out = {}
    for name, mode, iters in (("fp32", TT_MATH_FP32, 5), ("tf32", TT_MATH_TF32, 20), ("3xtf32", TT_MATH_3XTF32, 10)):
        rt.SetCuBlasMathMode(mode)
        ms = time_calls(lambda: rt.LaunchMatMul(a, b, c, n, n, n, n, 1, n, 1), iters)
        tf = flop / ms / 1e9
        if name == "fp32":
            out[name] = {"tflops": tf, "ms": ms, "frac_of_fp32_ffma_peak": tf / fp32_peak}
        else:
            pipe = tf * (3 if name == "3xtf32" else 1)
            out[name] = {"tflops": tf, "ms": ms, "tensor_pipe_tflops": pipe,
                         "frac_of_tf32_peak": pipe / tf32_peak}
    rt.SetCuBlasMathMode(TT_MATH_FP32)
    out["tf32_peak_tflops"] = tf32_peak
    out["tf32_peak_source"] = src
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

    # RL-policy shape: 8-64-64-2 MLP, batch 64, whole training step (forward, cross-entropy,
    # backward, Adam) as one replayed graph
    from tensotron_b200.mlp import MlpTrainer
    tr = MlpTrainer([8, 64, 64, 2], rt=rt, lr=1e-3, seed=3)
    xs = torch.randn((64, 8), device="cuda")
    ys = torch.randint(0, 2, (64,), device="cuda", dtype=torch.int32)
    l0 = rt.Stats()["launches"]
    tr.step(xs, ys)
    launches = rt.Stats()["launches"] - l0
    us, host = replay_us(lambda: tr.step(xs, ys), iters=10)
    out["mlp_8_64_64_2_batch64_train_step"] = {"graph_replay_us": us, "eager_host_us": host, "launches": launches}
    return out


def bmm_config3(rt):
    """Config 3: A [32,1,384,256] x B [1,16,256,192] -> [32,16,384,192], one launch through
    LaunchMatMulBatched (the reference issues 512 cuBLAS calls); FP32 and TF32.  In TF32 the
    151 MB output write makes it HBM-bound, so achieved GB/s is reported too."""
    import torch

    from tensotron_b200 import runtime
    from tensotron_b200.runtime import TT_MATH_FP32, TT_MATH_TF32
    a = torch.rand((32, 1, 384, 256), device="cuda") * 2 - 1
    b = torch.rand((1, 16, 256, 192), device="cuda") * 2 - 1
    c = torch.empty((32, 16, 384, 192), device="cuda")
    dims, aBs, bBs = runtime.broadcast_batch([32, 1], [98304, 98304], [1, 16], [786432, 49152])
    flop = 512 * 2.0 * 384 * 192 * 256
    nbytes = 4.0 * (a.numel() + b.numel() + c.numel())
    out = {"algorithmic_bytes": nbytes, "flop": flop}
    for name, mode in (("fp32", TT_MATH_FP32), ("tf32", TT_MATH_TF32)):
        rt.SetCuBlasMathMode(mode)
        ms = time_calls(lambda: rt.LaunchMatMulBatched(a, b, c, 512, 384, 192, 256, 256, 1, 192, 1, dims, aBs, bBs), 20)
        out[name] = {"ms": ms, "tflops": flop / ms / 1e9, "hbm_gbs": nbytes / ms / 1e6}
    rt.SetCuBlasMathMode(TT_MATH_FP32)
    try:
        out["hbm_peak_gbs"] = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except (OSError, KeyError, ValueError):
        out["hbm_peak_gbs"] = 6650.0
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
        try:
            tr = MlpTrainer([784, 4096, 4096, 4096, 10], rt=rt, device=local_rank, lr=1e-3, seed=2,
                            process_group=pg, math_mode=mode, exchange=exchange)
        except Exception as ex:     # e.g. peer mapping refused by the platform: report, keep the other runs
            res[name] = {"error": "%s: %s" % (type(ex).__name__, ex)}
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
    args = ap.parse_args()
    if args.one:
        return run_one(args.one)
    if args.one_bmm:
        return run_one_bmm(args.one_bmm)
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # raises if the CUDA library is missing: no fallback.  2.5 GiB workspace: 3xTF32 keeps
    # hi/lo copies of both 8192^2 operands there.
    rt = TensorRuntime(local_rank, 2560 << 20)
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

    # ---- end to end: pinned host operands, copies inside the timed region ----
    ha = torch.empty((rows, n), pin_memory=True).copy_(a)
    hb = torch.empty((n, n), pin_memory=True).copy_(b)
    hc = torch.empty((rows, n), pin_memory=True)
    e2e_steps = max(1, min(args.steps, 5))

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
            db.copy_(hb, non_blocking=True)
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

        guarded("mlp_784_4096x3_10_batch8192", lambda: mlp_steps_per_s(rt, rank, world, local_rank, pg))
        if world == 1:
            props0 = torch.cuda.get_device_properties(local_rank)
            guarded("bmm_32x16_384x256x192", lambda: bmm_config3(rt))
            guarded("small_configs", lambda: small_configs(rt))
            guarded("sgemm_8192", lambda: sgemm_modes_8192(rt, props0.multi_processor_count,
                                                           (clocks or {}).get("sm_max_mhz") or 1965.0))

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
            "traffic_note": "ncu DRAM bytes per launch; 16384 is the 8192^3 capture scaled (reads x 8, writes x 4)",
            "peak_source": "derived: %d SMs x 128 FP32 lanes x 2 x %.0f MHz (max SM clock); the "
                           "measured-peaks file has no FP32 SIMT figure" % (sms, max_mhz),
            "kernel": "sgemm_simt_kernel<MN-major A (transposed once into the workspace), N-major B>; "
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
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": (rows * n + n * n) * 4,
                    "d2h_bytes_per_step": rows * n * 4, "steps": e2e_steps,
                    "pipeline": "%d row chunks per step on H2D / compute / D2H streams, two buffer sets" % n_chunks},
            "gpu_launches": launches,
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
