"""Time one GEMM through the C-ABI library (also the command the ncu captures in profiles/ use).

    python -m tensotron_b200.run_gemm MxNxK LAYOUT VARIANT MODE ITERS [graph]

With the trailing word `graph` the ITERS launches are captured into one CUDA graph and the
graph is replayed: that is device time without per-call host overhead, the regime the
reference runs small networks in (native graph replay).

LAYOUT is NN / NT / TN (operand storage as in cuBLAS naming: N = row-major as given, T = the
operand is stored transposed and read through swapped strides); VARIANT as in tt_set_variant
(0 = automatic); MODE is the math mode (0 strict FP32, 3 TF32, 4 3xTF32).
"""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from tensotron_b200.runtime import TensorRuntime
M, N, K = (int(x) for x in sys.argv[1].split("x")); lay = sys.argv[2]; variant = int(sys.argv[3]); mode = int(sys.argv[4]); iters = int(sys.argv[5])
rt = TensorRuntime(0, 2048 << 20)
rt.SetCuBlasMathMode(mode); rt.SetVariant(variant)
a = torch.rand(M * K, device="cuda") * 2 - 1
b = torch.rand(K * N, device="cuda") * 2 - 1
c = torch.empty(M, N, device="cuda")
aMs, aKs = (K, 1) if lay[0] == "N" else (1, M)
bKs, bNs = (N, 1) if lay[1] == "N" else (1, K)
for _ in range(3):
    rt.LaunchMatMul(a, b, c, M, N, K, aMs, aKs, bKs, bNs)
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(iters):
    rt.LaunchMatMul(a, b, c, M, N, K, aMs, aKs, bKs, bNs)
e1.record(); torch.cuda.synchronize()
rt.Check()
ms = e0.elapsed_time(e1) / iters
print("ok %dx%dx%d %s v%d m%d: %.3f ms %.2f TF/s" % (M, N, K, lay, variant, mode, ms, 2.0 * M * N * K / ms / 1e9))
if len(sys.argv) > 6 and sys.argv[6] == "graph":
    import time
    t0 = time.perf_counter()
    for _ in range(iters):
        rt.LaunchMatMul(a, b, c, M, N, K, aMs, aKs, bKs, bNs)
    host_us = (time.perf_counter() - t0) / iters * 1e6
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            rt.LaunchMatMul(a, b, c, M, N, K, aMs, aKs, bKs, bNs)
    g.replay(); torch.cuda.synchronize()
    e0.record()
    for _ in range(5):
        g.replay()
    e1.record(); torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / (5 * iters) * 1e3
    print("   graph replay: %.2f us per launch (%.2f TF/s); host call cost %.2f us" % (us, 2.0 * M * N * K / us / 1e6, host_us))
