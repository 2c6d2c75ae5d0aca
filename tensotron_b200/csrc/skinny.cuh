// FP32 kernels for products with one tiny dimension (<= 16): the 10-class output layer of
// an MLP, value heads, matrix-vector products (a tiny K is left to the any-stride kernel,
// which measured faster there).  A 128-wide tile would waste > 90 % of its
// FMAs on them; they are HBM-bound streams of the one large operand instead, so each kernel
// reads that operand exactly once with 128-bit loads and keeps the small one in registers or
// L1.  One accumulator per output, a k order that depends on the output row only, fixed
// reduction trees: results are bit-stable run to run.
//
//   skinny_n_kernel  C (M x N<=16) = A (M x K, K-major) . B (N x K, K-major)^T     reads A once
//   skinny_m_kernel  C (M<=16 x N) = A (K x M)^T        . B (K x N, N-major)      reads B once
//                    (K is cut into ranges across CTAs; partials are added in range order)
#pragma once
#include "gemm_common.h"

namespace tt {
namespace skinny {

constexpr int MAXD = 16;

__device__ __forceinline__ float act_apply(float v, int act)
{
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return tanhf(v);
    return v;
}

// ---- small N ---------------------------------------------------------------------------------
// One CTA per ROWS rows of A (N <= NT).  The 8 warps of the CTA cut K into 8 contiguous slices,
// so a row's K elements are in flight from 8 warps at once (one warp walking a whole row is
// latency-bound: 86 us for any M up to 8192 at K = 4096).  Lanes stride over their slice in
// float4 steps; every lane keeps ROWS x N partial sums; a fixed xor-shuffle tree adds the 32
// lanes, shared memory the 8 warps in warp order: the summation order is a function of the
// shape only.  More rows per CTA cut the L1 traffic for the small operand relative to the large one.
template <int ROWS, int NT>
__global__ void __launch_bounds__(256)
skinny_n_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                int M, int N, int K, int aMs, int bNs, Epilogue epi)
{
    __shared__ float part[8][ROWS][NT];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * ROWS;
    float acc[ROWS][NT];
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int n = 0; n < NT; n++) acc[r][n] = 0.f;
    // slice of this warp: a multiple of 128 k (one float4 per lane and step)
    const int steps = (K + 127) / 128;
    const int per_warp = (steps + 7) / 8;
    const int s_begin = warp * per_warp;
    const int s_end = min(steps, s_begin + per_warp);
    // CTAs start at different steps of their slices (rotated by the CTA index): rows are a
    // power-of-two number of bytes apart, and thousands of warps walking them in lockstep from the
    // same offsets would keep hitting the same memory channels.  The order is a function of the
    // row only.
    const int span = s_end - s_begin;
    const int rot = span > 0 ? static_cast<int>(blockIdx.x % span) : 0;
    const auto step_k = [&](int i) {
        int it = s_begin + i + rot;
        if (it >= s_end) it -= span;
        return it * 128 + lane * 4;
    };
    const auto load_a = [&](int k, float4 (&av)[ROWS]) {
#pragma unroll
        for (int r = 0; r < ROWS; r++)
            // (streaming load: A is read once and must not push the small operand out of L1)
            av[r] = (k < K && m0 + r < M) ? __ldcs(reinterpret_cast<const float4*>(a + static_cast<long long>(m0 + r) * aMs + k))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    const auto fma_step = [&](int k, const float4 (&av)[ROWS]) {
        if (k >= K) return;
#pragma unroll
        for (int n = 0; n < NT; n++) {
            if (n < N) {
                const float4 bv = __ldg(reinterpret_cast<const float4*>(b + static_cast<long long>(n) * bNs + k));
#pragma unroll
                for (int r = 0; r < ROWS; r++) {
                    float s = acc[r][n];
                    s = fmaf(av[r].x, bv.x, s);
                    s = fmaf(av[r].y, bv.y, s);
                    s = fmaf(av[r].z, bv.z, s);
                    s = fmaf(av[r].w, bv.w, s);
                    acc[r][n] = s;
                }
            }
        }
    };
    // two steps per iteration: the loads of both are issued before the first FMA, which doubles
    // the bytes a warp keeps in flight
    int i = 0;
    for (; i + 1 < span; i += 2) {
        const int k0 = step_k(i), k1 = step_k(i + 1);
        float4 a0[ROWS], a1[ROWS];
        load_a(k0, a0);
        load_a(k1, a1);
        fma_step(k0, a0);
        fma_step(k1, a1);
    }
    if (i < span) {
        const int k0 = step_k(i);
        float4 a0[ROWS];
        load_a(k0, a0);
        fma_step(k0, a0);
    }
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int n = 0; n < NT; n++) {
            if (n < N) {
                float s = acc[r][n];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) part[warp][r][n] = s;
            }
        }
    __syncthreads();
    for (int e = threadIdx.x; e < ROWS * NT; e += blockDim.x) {
        const int r = e / NT, n = e % NT;
        if (n < N && m0 + r < M) {
            float s = part[0][r][n];
#pragma unroll
            for (int w = 1; w < 8; w++) s += part[w][r][n];
            if (epi.bias) s += __ldg(epi.bias + n);
            c[static_cast<long long>(m0 + r) * N + n] = act_apply(s, epi.act);
        }
    }
}

// ---- small M ---------------------------------------------------------------------------------
// Each thread owns 4 adjacent columns of C and all M rows; the CTA's 4 k lanes walk this CTA's
// k range; lanes are added in lane order through shared memory and the result goes to
// partial[range][M][N] (or straight to C when there is a single range).
__global__ void __launch_bounds__(256)
skinny_m_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                int M, int N, int K, int aMs, int aKs, int bKs, int kspan, Epilogue epi, int direct)
{
    __shared__ float4 red[4][64];
    const int cl = threadIdx.x & 63;
    const int kl = threadIdx.x >> 6;
    const int n = (blockIdx.x * 64 + cl) * 4;
    const int k0 = blockIdx.y * kspan;
    const int k1 = min(K, k0 + kspan);
    float4 acc[MAXD];
#pragma unroll
    for (int m = 0; m < MAXD; m++) acc[m] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n < N) {
        for (int k = k0 + kl; k < k1; k += 4) {
            const float4 bv = *reinterpret_cast<const float4*>(b + static_cast<long long>(k) * bKs + n);
#pragma unroll
            for (int m = 0; m < MAXD; m++) {
                if (m < M) {
                    const float av = __ldg(a + static_cast<long long>(m) * aMs + static_cast<long long>(k) * aKs);
                    acc[m].x = fmaf(av, bv.x, acc[m].x);
                    acc[m].y = fmaf(av, bv.y, acc[m].y);
                    acc[m].z = fmaf(av, bv.z, acc[m].z);
                    acc[m].w = fmaf(av, bv.w, acc[m].w);
                }
            }
        }
    }
    float* dst = out + (direct ? 0ll : static_cast<long long>(blockIdx.y) * M * N);
#pragma unroll
    for (int m = 0; m < MAXD; m++) {
        if (m < M) {                       // uniform across the CTA
            red[kl][cl] = acc[m];
            __syncthreads();
            if (kl == 0 && n < N) {
                float4 s = red[0][cl];
#pragma unroll
                for (int l = 1; l < 4; l++) {
                    const float4 q = red[l][cl];
                    s.x += q.x; s.y += q.y; s.z += q.z; s.w += q.w;
                }
                if (direct) {
                    if (epi.bias) {
                        const float4 bb = __ldg(reinterpret_cast<const float4*>(epi.bias + n));
                        s.x += bb.x; s.y += bb.y; s.z += bb.z; s.w += bb.w;
                    }
                    s.x = act_apply(s.x, epi.act); s.y = act_apply(s.y, epi.act);
                    s.z = act_apply(s.z, epi.act); s.w = act_apply(s.w, epi.act);
                }
                *reinterpret_cast<float4*>(dst + static_cast<long long>(m) * N + n) = s;
            }
            __syncthreads();
        }
    }
}

// C[i] = act(sum over ranges (ascending) of partial[range][i] + bias[i % N]); 4 elements per thread.
__global__ void __launch_bounds__(256)
skinny_reduce_kernel(const float* __restrict__ partial, float* __restrict__ c, long long count4, int N,
                     int ranges, long long range_stride, Epilogue epi)
{
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count4) return;
    float4 s = reinterpret_cast<const float4*>(partial)[i];
    for (int r = 1; r < ranges; r++) {
        const float4 q = reinterpret_cast<const float4*>(partial + r * range_stride)[i];
        s.x += q.x; s.y += q.y; s.z += q.z; s.w += q.w;
    }
    if (epi.bias) {
        const int n = static_cast<int>((i * 4) % N);
        const float4 bb = __ldg(reinterpret_cast<const float4*>(epi.bias + n));
        s.x += bb.x; s.y += bb.y; s.z += bb.z; s.w += bb.w;
    }
    s.x = act_apply(s.x, epi.act); s.y = act_apply(s.y, epi.act);
    s.z = act_apply(s.z, epi.act); s.w = act_apply(s.w, epi.act);
    reinterpret_cast<float4*>(c)[i] = s;
}

}  // namespace skinny
}  // namespace tt
