// Any-stride, any-alignment FP32 GEMM (plain loads, no TMA): the total fallback that
// keeps the LaunchMatMul / LaunchMatMulBatched contract defined for every stride
// combination (odd leading dimensions, unaligned sub-views, "TT" strides, tiny
// shapes).  64x64x16 tiles, 256 threads, 4x4 accumulators per thread, ascending-k
// summation with one accumulator per output (bit-stable).
#pragma once
#include "gemm_common.h"

namespace tt {
namespace generic {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

struct Params {
    const float* a;
    const float* b;
    float* c;
    GemmShape shape;
    BatchDesc batch;
    Epilogue epi;
    int aMs, aKs, bKs, bNs;
};

__device__ __forceinline__ float act_apply(float v, int act)
{
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return tanhf(v);
    return v;
}

__global__ void __launch_bounds__(THREADS) gemm_generic_kernel(const Params p)
{
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];

    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;
    const int tiles_per_mat = p.shape.tiles_m * p.shape.tiles_n;
    // Thread->element mapping of the tile loads follows the contiguous axis so the
    // global reads coalesce for K-major and MN-major operands alike.
    const bool a_kmaj = p.aKs == 1 || p.aMs != 1;
    const bool b_kmaj = p.bKs == 1 || p.bNs != 1;

    for (long long w = blockIdx.x; w < p.shape.work; w += gridDim.x) {
        const int bidx = static_cast<int>(w / tiles_per_mat);
        const int t = static_cast<int>(w - static_cast<long long>(bidx) * tiles_per_mat);
        const int tm = t / p.shape.tiles_n, tn = t % p.shape.tiles_n;
        long long a_off = 0, b_off = 0;
        int br = bidx;
        for (int ax = p.batch.rank - 1; ax >= 0; ax--) {
            const int d = p.batch.dims[ax];
            const int bi = br % d;
            br /= d;
            a_off += static_cast<long long>(bi) * p.batch.a_stride[ax];
            b_off += static_cast<long long>(bi) * p.batch.b_stride[ax];
        }
        const float* A = p.a + a_off;
        const float* B = p.b + b_off;
        const int m0 = tm * BM, n0 = tn * BN;

        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

        // Global loads of k-tile i+1 are issued into registers before the FMAs of k-tile i,
        // so the global-memory latency overlaps the arithmetic.
        float ra[(BM * BK) / THREADS], rb[(BN * BK) / THREADS];
        const auto fetch = [&](int k0) {
#pragma unroll
            for (int e = 0; e < (BM * BK) / THREADS; e++) {
                const int idx = tid + e * THREADS;
                const int kk = a_kmaj ? (idx % BK) : (idx / BM);
                const int mm = a_kmaj ? (idx / BK) : (idx % BM);
                const int gm = m0 + mm, gk = k0 + kk;
                ra[e] = (gm < p.shape.M && gk < p.shape.K)
                            ? __ldg(A + static_cast<long long>(gm) * p.aMs + static_cast<long long>(gk) * p.aKs)
                            : 0.f;
            }
#pragma unroll
            for (int e = 0; e < (BN * BK) / THREADS; e++) {
                const int idx = tid + e * THREADS;
                const int kk = b_kmaj ? (idx % BK) : (idx / BN);
                const int nn = b_kmaj ? (idx / BK) : (idx % BN);
                const int gn = n0 + nn, gk = k0 + kk;
                rb[e] = (gn < p.shape.N && gk < p.shape.K)
                            ? __ldg(B + static_cast<long long>(gn) * p.bNs + static_cast<long long>(gk) * p.bKs)
                            : 0.f;
            }
        };
        if (p.shape.K > 0) fetch(0);
        for (int k0 = 0; k0 < p.shape.K; k0 += BK) {
#pragma unroll
            for (int e = 0; e < (BM * BK) / THREADS; e++) {
                const int idx = tid + e * THREADS;
                As[a_kmaj ? (idx % BK) : (idx / BM)][a_kmaj ? (idx / BK) : (idx % BM)] = ra[e];
            }
#pragma unroll
            for (int e = 0; e < (BN * BK) / THREADS; e++) {
                const int idx = tid + e * THREADS;
                Bs[b_kmaj ? (idx % BK) : (idx / BN)][b_kmaj ? (idx / BK) : (idx % BN)] = rb[e];
            }
            __syncthreads();
            if (k0 + BK < p.shape.K) fetch(k0 + BK);
#pragma unroll
            for (int kk = 0; kk < BK; kk++) {
                const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
                const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
                const float a[4] = {av.x, av.y, av.z, av.w};
                const float b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            __syncthreads();
        }

        float* C = p.c + static_cast<long long>(bidx) * p.shape.M * p.shape.N;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int gm = m0 + ty * 4 + i;
            if (gm >= p.shape.M) continue;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int gn = n0 + tx * 4 + j;
                if (gn >= p.shape.N) continue;
                float v = acc[i][j];
                if (p.epi.bias) v += __ldg(p.epi.bias + gn);
                C[static_cast<long long>(gm) * p.shape.N + gn] = act_apply(v, p.epi.act);
            }
        }
    }
}

}  // namespace generic
}  // namespace tt
