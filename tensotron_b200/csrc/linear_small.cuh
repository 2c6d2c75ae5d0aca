// Backward of a small Linear layer as ONE launch.
//
// The reference runs the backward of Linear + activation as separate ops: the activation's
// backward, the bias gradient (a clone of g and a column sum with atomics), dX = g . W and
// dW = g^T . X (src/Tensotron/TensorOps.LinearNT.cs:36-44, src/Tensotron/TensorOps.cs:76-100,143-147).
// For the layer sizes of small networks (64 x 128 x 64 and the like) each of those is a few
// microseconds of launch and memory latency around well under a microsecond of arithmetic, so here
// one grid computes all of them: CTAs [0, tiles_dx) own 32 x 32 tiles of dX, the others 32 x 32 tiles
// of dW, and the dW CTAs of the first tile column also add up the bias gradient of their 32 rows.
// g = dy * act'(y) is formed while the operand tile is loaded and never written to memory.
// Every output is one accumulator walked in ascending contraction index with fused multiply-adds
// (the summation rule of the large kernels); the bias gradient is a sum in ascending row order.
#pragma once
#include <cuda_runtime.h>

#include "elementwise.cuh"

namespace tt {
namespace lin_small {

constexpr int T = 32, THREADS = 256, PER = (T * T) / THREADS;

struct Params {
    const float* x;    // (M, K)
    const float* w;    // (N, K)
    const float* y;    // (M, N) forward output, read when act != 0
    const float* dy;   // (M, N)
    float* dx;         // (M, K) or null
    float* dw;         // (N, K)
    float* db;         // (N) or null
    int M, N, K, act;
    int tiles_dx;      // CTAs that compute dX (0 when dx is null)
    int tiles_k;       // 32-column tiles along K (both outputs have K columns)
};

__global__ void __launch_bounds__(THREADS) linear_bwd_small_kernel(const Params p)
{
    __shared__ float As[T][T + 1];   // [contraction][output row]
    __shared__ float Bs[T][T + 1];   // [contraction][output column]
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const bool is_dx = static_cast<int>(blockIdx.x) < p.tiles_dx;
    const int t = is_dx ? blockIdx.x : blockIdx.x - p.tiles_dx;
    const int r0 = (t / p.tiles_k) * T, c0 = (t % p.tiles_k) * T;
    const int R = is_dx ? p.M : p.N;            // rows of this output
    const int LC = is_dx ? p.N : p.M;           // contraction length
    const float* bsrc = is_dx ? p.w : p.x;      // (LC, K)
    const bool with_db = !is_dx && c0 == 0 && p.db != nullptr;

    float ra[PER], rb[PER];
    const auto fetch = [&](int l0) {
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = tid + e * THREADS;
            // the operand g is contiguous along the contraction for dX and along the rows for dW
            const int rr = is_dx ? idx / T : idx % T, ll = is_dx ? idx % T : idx / T;
            float v = 0.f;
            if (r0 + rr < R && l0 + ll < LC) {
                const long long gi = is_dx ? static_cast<long long>(r0 + rr) * p.N + (l0 + ll)
                                           : static_cast<long long>(l0 + ll) * p.N + (r0 + rr);
                v = __ldg(p.dy + gi);
                if (p.act != 0) v = ew::act_grad(__ldg(p.y + gi), v, p.act);
            }
            ra[e] = v;
            const int bl = idx / T, bc = idx % T;
            rb[e] = (l0 + bl < LC && c0 + bc < p.K) ? __ldg(bsrc + static_cast<long long>(l0 + bl) * p.K + (c0 + bc)) : 0.f;
        }
    };

    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    float dbacc = 0.f;
    fetch(0);
    for (int l0 = 0; l0 < LC; l0 += T) {
#pragma unroll
        for (int e = 0; e < PER; e++) {
            const int idx = tid + e * THREADS;
            const int rr = is_dx ? idx / T : idx % T, ll = is_dx ? idx % T : idx / T;
            As[ll][rr] = ra[e];
            Bs[idx / T][idx % T] = rb[e];
        }
        __syncthreads();
        if (l0 + T < LC) fetch(l0 + T);
        if (with_db && tid < T) {
#pragma unroll 8
            for (int ll = 0; ll < T; ll++) dbacc += As[ll][tid];     // rows beyond M hold zeros
        }
#pragma unroll 8
        for (int kk = 0; kk < T; kk++) {
            const float a0 = As[kk][2 * ty], a1 = As[kk][2 * ty + 1];
            const float b0 = Bs[kk][2 * tx], b1 = Bs[kk][2 * tx + 1];
            acc[0][0] = fmaf(a0, b0, acc[0][0]);
            acc[0][1] = fmaf(a0, b1, acc[0][1]);
            acc[1][0] = fmaf(a1, b0, acc[1][0]);
            acc[1][1] = fmaf(a1, b1, acc[1][1]);
        }
        __syncthreads();
    }
    float* out = is_dx ? p.dx : p.dw;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = r0 + 2 * ty + i;
        if (r >= R) continue;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int c = c0 + 2 * tx + j;
            if (c < p.K) out[static_cast<long long>(r) * p.K + c] = acc[i][j];
        }
    }
    if (with_db && tid < T && r0 + tid < p.N) p.db[r0 + tid] = dbacc;
}

}  // namespace lin_small
}  // namespace tt
