"""Time the broadcast batched product of benchmark config 3 through the C-ABI library (also the
command the ncu captures in profiles/ use).

    python -m tensotron_b200.run_bmm MODE ITERS [transposed_b]

A [32,1,384,256] x B [1,16,256,192] -> C [32,16,384,192] in one LaunchMatMulBatched call; MODE is
the math mode (0 strict FP32, 3 TF32, 4 3xTF32).  With `transposed_b` B is stored [1,16,192,256]
and read through bKs = 1, bNs = 256.
"""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from tensotron_b200 import runtime
from tensotron_b200.runtime import TensorRuntime
mode, iters = int(sys.argv[1]), int(sys.argv[2])
tb = len(sys.argv) > 3 and sys.argv[3] == "transposed_b"
rt = TensorRuntime(0, 1 << 30)
rt.SetCuBlasMathMode(mode)
a = torch.rand((32, 1, 384, 256), device="cuda") * 2 - 1
b = torch.rand((1, 16, 192, 256) if tb else (1, 16, 256, 192), device="cuda") * 2 - 1
c = torch.empty((32, 16, 384, 192), device="cuda")
dims, aBs, bBs = runtime.broadcast_batch([32, 1], [98304, 98304], [1, 16], [786432, 49152])
bKs, bNs = (1, 256) if tb else (192, 1)
call = lambda: rt.LaunchMatMulBatched(a, b, c, 512, 384, 192, 256, 256, 1, bKs, bNs, dims, aBs, bBs)
for _ in range(3):
    call()
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(iters):
    call()
e1.record(); torch.cuda.synchronize()
rt.Check()
ms = e0.elapsed_time(e1) / iters
nbytes = 4.0 * (a.numel() + b.numel() + c.numel())
print("ok bmm config 3 m%d%s: %.1f us %.2f TF/s %.0f GB/s of algorithmic bytes" % (
    mode, " (B transposed)" if tb else "", ms * 1e3, 512 * 2.0 * 384 * 192 * 256 / ms / 1e9, nbytes / ms / 1e6))
