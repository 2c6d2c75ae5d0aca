"""Time one GEMM through the C-ABI library (also the command the ncu captures in profiles/ use).

    python -m tensotron_b200.run_gemm MxNxK LAYOUT VARIANT MODE ITERS

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
