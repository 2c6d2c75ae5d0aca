"""B200-native matmul engine for Tensotron's CUDA backend.

The product is the C-ABI library ``libtensotron_gemm.so`` (include/tensotron_gemm.h,
sources under tensotron_b200/csrc).  This package is the host-side mirror of the
reference's runtime / op surface for that path, used by the tests and benchmarks:

  runtime.TensorRuntime  -- LaunchMatMul / LaunchMatMulBatched and friends over ctypes
  ops                    -- MatMul / MatMulNT / Bmm / Linear forward + backward closures

There is no CPU or library fallback: if the CUDA library cannot be loaded, importing
``runtime`` raises.
"""
from .runtime import TensorRuntime, TensotronGemmError, load_library  # noqa: F401
