// Host entry of the tcgen05 (TF32 / 3xTF32) GEMM path.
#pragma once
#include <cuda_runtime.h>

#include "gemm_common.h"

namespace tt {
namespace tf32 {

// One-time per-device kernel attribute setup (called from tt_create).
int init_device();

// Enqueues the tensor-core GEMM when the operands qualify.  Returns 0 on success,
// TT_ERR_UNSUPPORTED (3) when the shape / strides are outside what the kernel takes
// (the caller then uses the strict-FP32 path), another status on a launch failure.
// 3xTF32 (math_mode 4) keeps the hi/lo copies of both operands in `workspace` and needs
// 2 x (span(A) + span(B)) floats of it.  *launches receives the kernels enqueued;
// forced_mt = 1 / 2 pins the tile height (128 / 256 rows), 0 lets the heuristic choose.
int try_launch(int math_mode, cudaStream_t st, const float* a, const float* b, float* c, int M,
               int N, int K, int aMs, int aKs, int bKs, int bNs, int batch_count, int batch_rank,
               const int* batch_dims, const int* a_bs, const int* b_bs, const Epilogue& epi,
               int num_sms, unsigned int* status, void* workspace, size_t workspace_bytes,
               int* launches, int forced_mt);

}  // namespace tf32
}  // namespace tt
