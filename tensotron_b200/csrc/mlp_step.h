// Host entry of the one-launch training step for small MLPs (mlp_step.cu).
#pragma once
#include <cuda_runtime.h>

#include "../../include/tensotron_gemm.h"

namespace tt {
namespace mlp_step {

constexpr int MAX_LAYERS = TT_MLP_MAX_LAYERS;
constexpr int MAX_WIDTH = 64;     // widest layer (inputs and outputs alike)
constexpr int MAX_ROWS = 64;      // batch rows per CTA
constexpr int MAX_CLUSTER = 16;   // CTAs of the cluster (8 where 16 cannot be scheduled)
constexpr int MAX_SMEM_BYTES = 200 * 1024;

// One-time per-context kernel attribute set-up (called from tt_create).
int init_device();

// Enqueues the step.  TT_ERR_UNSUPPORTED when the network or the batch is outside what one
// cluster holds (the caller then runs the step layer by layer).  *n_ctas receives the cluster size.
int launch(cudaStream_t st, const tt_mlp_desc* net, float* params, float* m, float* v, float* adv, float* grads_out,
           const float* x, const void* target, float* loss_out, unsigned int* status, int batch, float lr, float b1,
           float b2, float eps, float max_norm, float clip_eps, int advance, int* n_ctas);

}  // namespace mlp_step
}  // namespace tt
