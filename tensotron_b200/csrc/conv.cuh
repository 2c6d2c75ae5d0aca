// Conv2d through the batched GEMM engine.
//
// The reference computes Conv2d as Im2Col -> MatMul((1, O, K), (N, K, L)) -> broadcast bias add
// (src/Tensotron/TensorOps.Conv.cs:60-80; K = C*kh*kw, L = Ho*Wo), with its backward falling out
// of autograd: the bias gradient is a reduction of g over batch and positions, dW is the
// broadcast-reduced batched product g . col^T, dcol = W^T . g, and Col2Im scatters dcol back with
// atomics (src/Tensotron/Kernels.cs:784-814).  Here the same products run on the batched kernels of
// this library, as one launch each:
//   forward   im2col writes the columns with one extra row of ones (and zero rows up to a multiple
//             of 4), the weights are packed with the bias as one extra column: the GEMM
//             [W | b] . [col ; 1] adds the bias as the last term of every output's k sum, so there
//             is no separate bias pass over the output;
//   dW        one batched product with the batch axis summed inside the k loop (ascending n);
//   dcol      one batched product with W broadcast over the batch;
//   dx        col2im as a GATHER: every input pixel adds the windows that cover it in ascending
//             kernel-offset order -- a fixed order, no atomics;
//   dbias     one CTA per output channel, fixed-order sum over batch and positions.
// The support kernels are streaming kernels (one thread per output element, writes coalesced).
#pragma once
#include <cuda_runtime.h>

namespace tt {
namespace conv {

struct Shape {
    int n, c, h, w, o, kh, kw, stride, pad, dil;
    int ho, wo;
    int K, L, Kp;   // K = c*kh*kw, L = ho*wo, Kp = K + 1 rounded up to a multiple of 4
};

// col[n][k][l]: k < K gathers x (0 outside the image), k == K is 1, K < k < Kp is 0.
static __global__ void __launch_bounds__(256) im2col_kernel(const float* __restrict__ x, float* __restrict__ col, Shape s)
{
    const long long total = static_cast<long long>(s.n) * s.Kp * s.L;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int l = static_cast<int>(i % s.L);
        const long long t = i / s.L;
        const int k = static_cast<int>(t % s.Kp);
        const int n = static_cast<int>(t / s.Kp);
        float v = 0.f;
        if (k < s.K) {
            const int kj = k % s.kw, t2 = k / s.kw, ki = t2 % s.kh, c = t2 / s.kh;
            const int ow = l % s.wo, oh = l / s.wo;
            const int ih = oh * s.stride - s.pad + ki * s.dil, iw = ow * s.stride - s.pad + kj * s.dil;
            if (ih >= 0 && ih < s.h && iw >= 0 && iw < s.w)
                v = x[((static_cast<long long>(n) * s.c + c) * s.h + ih) * s.w + iw];
        } else if (k == s.K) {
            v = 1.f;
        }
        col[i] = v;
    }
}

// wp[o][k]: k < K copies w, k == K is bias[o] (0 without a bias), K < k < Kp is 0.
static __global__ void __launch_bounds__(256) pack_weight_kernel(const float* __restrict__ w, const float* __restrict__ bias,
                                                                float* __restrict__ wp, int o, int K, int Kp)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= o * Kp) return;
    const int k = i % Kp, oo = i / Kp;
    wp[i] = k < K ? w[oo * K + k] : (k == K && bias ? bias[oo] : 0.f);
}

// dx[n][c][ih][iw] = sum over the kernel offsets (ki, kj), ascending, of dcol[n][(c*kh+ki)*kw+kj][oh*wo+ow]
// for the output position (oh, ow) whose window puts that offset on the pixel, if there is one.
static __global__ void __launch_bounds__(256) col2im_kernel(const float* __restrict__ dcol, float* __restrict__ dx, Shape s)
{
    const long long total = static_cast<long long>(s.n) * s.c * s.h * s.w;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int iw = static_cast<int>(i % s.w);
        long long t = i / s.w;
        const int ih = static_cast<int>(t % s.h);
        t /= s.h;
        const int c = static_cast<int>(t % s.c);
        const int n = static_cast<int>(t / s.c);
        const float* base = dcol + static_cast<long long>(n) * s.K * s.L;
        float sum = 0.f;
        for (int ki = 0; ki < s.kh; ki++) {
            const int hh = ih + s.pad - ki * s.dil;
            if (hh < 0 || hh % s.stride != 0) continue;
            const int oh = hh / s.stride;
            if (oh >= s.ho) continue;
            for (int kj = 0; kj < s.kw; kj++) {
                const int ww = iw + s.pad - kj * s.dil;
                if (ww < 0 || ww % s.stride != 0) continue;
                const int ow = ww / s.stride;
                if (ow >= s.wo) continue;
                sum += base[static_cast<long long>((c * s.kh + ki) * s.kw + kj) * s.L + oh * s.wo + ow];
            }
        }
        dx[i] = sum;
    }
}

// dbias[o] = sum over n (ascending) and l of g[n][o][l]: one CTA per channel, each thread a strided
// slice of the positions of every n in ascending order, then a shared-memory tree of fixed shape.
static __global__ void __launch_bounds__(256) bias_grad_kernel(const float* __restrict__ g, float* __restrict__ dbias,
                                                              int n, int o, int L)
{
    __shared__ float red[256];
    const int oo = blockIdx.x;
    float t = 0.f;
    for (int nn = 0; nn < n; nn++) {
        const float* row = g + (static_cast<long long>(nn) * o + oo) * L;
        for (int l = threadIdx.x; l < L; l += 256) t += row[l];
    }
    red[threadIdx.x] = t;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if (threadIdx.x < w) red[threadIdx.x] += red[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) dbias[oo] = red[0];
}

}  // namespace conv
}  // namespace tt
