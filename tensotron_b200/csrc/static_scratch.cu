// tt_softmax_cross_entropy_static: the cross-entropy entry point for callers that must
// not allocate device memory.
//
// The regular entry (tt_softmax_cross_entropy) parks its per-row losses in the workspace
// a handle obtained from tt_create owns, and tt_create calls cudaMalloc.  Some hosts cannot
// go that way: a runtime whose own pool allocator has claimed the device heap and does not
// tolerate foreign allocations, or a component that is only handed a stream and buffers and
// has no say over device memory at all.  For them the same two kernels run here against a
// scratch array that is part of the library image: it exists on every GPU that loads the
// library, from load until the process exits, and costs TT_STATIC_CE_MAX_ROWS floats
// (256 KiB) there.
//
// Host code cannot pass the array's name to a kernel (on the host the name is only a
// stand-in); the device address is looked up once per device with cudaGetSymbolAddress
// while that device is current.  The first call on a device performs that look-up, so make
// it before starting any stream capture.  Nothing here calls cudaMalloc, cudaFree or an
// allocating library routine.
//
// The array is shared by all calls and keeps whatever the last call left in it.  Every row
// slot that a call reads is written by that same call first, so nothing has to be cleared;
// but two calls whose kernels overlap on the GPU (different streams) race on it.
#include "../../include/tensotron_gemm.h"

#include <cuda_runtime.h>
#include <math.h>

namespace {

static __device__ __align__(256) float g_static_row_loss[TT_STATIC_CE_MAX_ROWS];

// The two kernels below repeat the arithmetic and the summation order of the handle-based
// entry's kernels (one warp per row with a fixed shuffle tree; a single-CTA strided sum
// followed by a fixed shared-memory tree), so both entries return identical bits.
__global__ void __launch_bounds__(256)
static_ce_rows_kernel(const float* __restrict__ logits, const int* __restrict__ labels,
                      float* __restrict__ dlogits, float* __restrict__ row_loss, int rows,
                      int classes, float scale)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const float* x = logits + static_cast<long long>(warp) * classes;
    float mx = -INFINITY;
    for (int j = lane; j < classes; j += 32) mx = fmaxf(mx, x[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
    for (int j = lane; j < classes; j += 32) s += expf(x[j] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float lse = logf(s) + mx;
    const int label = labels[warp];
    if (row_loss && lane == 0) row_loss[warp] = -(x[label] - lse);
    if (dlogits) {
        float* d = dlogits + static_cast<long long>(warp) * classes;
        for (int j = lane; j < classes; j += 32)
            d[j] = (expf(x[j] - lse) - (j == label ? 1.f : 0.f)) * scale;
    }
}

__global__ void __launch_bounds__(1024)
static_sum_kernel(const float* __restrict__ v, float* __restrict__ out, int n, float scale)
{
    __shared__ float red[1024];
    float t = 0.f;
    for (int i = threadIdx.x; i < n; i += 1024) t += v[i];
    red[threadIdx.x] = t;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *out = red[0] * scale;
}

constexpr int MAX_DEVICES = 64;
float* g_row_loss_addr[MAX_DEVICES] = {};  // device address of the array, per device ordinal

// Device address of the scratch array on the current device (set-up on first use).
int scratch_address(float** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return TT_ERR_CUDA;
    if (!g_row_loss_addr[dev]) {
        float* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_row_loss);
        if (e != cudaSuccess || !ptr) return TT_ERR_CUDA;
        g_row_loss_addr[dev] = ptr;
    }
    *out = g_row_loss_addr[dev];
    return TT_OK;
}

}  // namespace

extern "C" TT_API int tt_softmax_cross_entropy_static(void* stream, const float* logits,
                                                      const int* labels, float* dlogits, float* loss,
                                                      int rows, int classes, float scale)
{
    if (rows < 0 || classes <= 0 || !logits || !labels) return TT_ERR_INVALID_ARG;
    if (rows > TT_STATIC_CE_MAX_ROWS) return TT_ERR_STATIC_LIMIT;
    if (rows == 0) return TT_OK;
    float* row_loss = nullptr;
    if (loss) {
        const int rc = scratch_address(&row_loss);
        if (rc != TT_OK) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps_per_block = 8;
    static_ce_rows_kernel<<<(rows + warps_per_block - 1) / warps_per_block, 256, 0, st>>>(
        logits, labels, dlogits, row_loss, rows, classes, scale);
    if (loss) static_sum_kernel<<<1, 1024, 0, st>>>(row_loss, loss, rows, scale);
    return cudaGetLastError() == cudaSuccess ? TT_OK : TT_ERR_CUDA;
}
