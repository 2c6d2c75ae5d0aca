// Support kernels around the GEMMs: activation backward fused with a fixed-order
// bias-gradient column sum, softmax cross-entropy, fused Adam, AddInto.  All are
// HBM-bound streaming kernels: 128-bit accesses where alignment allows, grids sized
// from the shape only (never from the SM count) so summation order -- and therefore
// every bit of the result -- is a function of the inputs alone.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tt {
namespace ew {

constexpr int COLSUM_COLS = 128;      // columns per CTA
constexpr int COLSUM_ROW_LANES = 8;   // row lanes per CTA (256 threads = 32 col groups x 8)
constexpr int COLSUM_MAX_CHUNKS = 64;

static inline int colsum_chunks(int M)
{
    int c = M / 64;
    if (c < 1) c = 1;
    if (c > COLSUM_MAX_CHUNKS) c = COLSUM_MAX_CHUNKS;
    return c;
}

__device__ __forceinline__ float act_grad(float y, float dy, int act)
{
    if (act == 1) return y > 0.f ? dy : 0.f;          // ReLU: x > 0 <=> y > 0
    if (act == 2) return dy * (1.f - y * y);          // Tanh
    return dy;
}

// g = dy * act'(y) (written when g != null) and partial[chunk][n] = sum over this
// chunk's rows of g[.,n].  Grid: (ceil(N/128), chunks).  Rows of a chunk are visited
// in ascending order by each row lane; the 8 row lanes are then added in lane order.
template <bool VEC>
__global__ void __launch_bounds__(256)
act_bwd_colsum_kernel(const float* __restrict__ y, const float* __restrict__ dy,
                      float* __restrict__ g, float* __restrict__ partial, int M, int N, int act,
                      int chunks)
{
    __shared__ float red[COLSUM_ROW_LANES][COLSUM_COLS];
    const int cg = threadIdx.x & 31;   // column group (4 columns)
    const int rl = threadIdx.x >> 5;   // row lane
    const int col = blockIdx.x * COLSUM_COLS + cg * 4;
    const int chunk = blockIdx.y;
    const int rows_per = (M + chunks - 1) / chunks;
    const int r0 = chunk * rows_per;
    const int r1 = min(M, r0 + rows_per);
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (col < N) {
        for (int r = r0 + rl; r < r1; r += COLSUM_ROW_LANES) {
            const long long base = static_cast<long long>(r) * N + col;
            float d[4], yy[4] = {0.f, 0.f, 0.f, 0.f};
            if (VEC) {
                const float4 dv = *reinterpret_cast<const float4*>(dy + base);
                d[0] = dv.x; d[1] = dv.y; d[2] = dv.z; d[3] = dv.w;
                if (act) {
                    const float4 yv = *reinterpret_cast<const float4*>(y + base);
                    yy[0] = yv.x; yy[1] = yv.y; yy[2] = yv.z; yy[3] = yv.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    d[j] = (col + j < N) ? dy[base + j] : 0.f;
                    if (act) yy[j] = (col + j < N) ? y[base + j] : 0.f;
                }
            }
            float gg[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                gg[j] = act_grad(yy[j], d[j], act);
                s[j] += gg[j];
            }
            if (g) {
                if (VEC) {
                    *reinterpret_cast<float4*>(g + base) = make_float4(gg[0], gg[1], gg[2], gg[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (col + j < N) g[base + j] = gg[j];
                }
            }
        }
    }
    if (!partial) return;
#pragma unroll
    for (int j = 0; j < 4; j++) red[rl][cg * 4 + j] = s[j];
    __syncthreads();
    if (threadIdx.x < COLSUM_COLS) {
        const int c = blockIdx.x * COLSUM_COLS + threadIdx.x;
        if (c < N) {
            float t = 0.f;
#pragma unroll
            for (int l = 0; l < COLSUM_ROW_LANES; l++) t += red[l][threadIdx.x];
            partial[static_cast<long long>(chunk) * N + c] = t;
        }
    }
}

// out[n] = sum over chunks (ascending) of partial[chunk][n].
static __global__ void colsum_finish_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                     int N, int chunks)
{
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float t = 0.f;
    for (int c = 0; c < chunks; c++) t += partial[static_cast<long long>(c) * N + n];
    out[n] = t;
}

// One warp per row: lse = log(sum exp(x - max)) + max; row_loss = -(x[label] - lse);
// dlogits = (exp(x - lse) - onehot) * scale.  Warp shuffles reduce in a fixed tree.
// A label outside [0, classes) is never used as an index: that row's loss becomes NaN (so the
// summed loss is NaN), its gradient is the plain softmax, and code 7 (DEV_BAD_LABEL of ptx.cuh) is
// recorded in *status when status is not null.  (static: this header is compiled into more than
// one translation unit of the library.)
static __global__ void __launch_bounds__(256)
softmax_ce_rows_kernel(const float* __restrict__ logits, const int* __restrict__ labels,
                       float* __restrict__ dlogits, float* __restrict__ row_loss, int rows,
                       int classes, float scale, unsigned int* status)
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
    const bool label_ok = label >= 0 && label < classes;
    if (lane == 0) {
        if (row_loss) row_loss[warp] = label_ok ? -(x[label] - lse) : __int_as_float(0x7fc00000);
        if (!label_ok && status) atomicCAS(status, 0u, 7u);
    }
    if (dlogits) {
        float* d = dlogits + static_cast<long long>(warp) * classes;
        for (int j = lane; j < classes; j += 32)
            d[j] = (expf(x[j] - lse) - (j == label ? 1.f : 0.f)) * scale;
    }
}

// Single-CTA fixed-order sum: each thread adds a strided slice in ascending order,
// then a shared-memory tree with a fixed shape.  out = scale * sum(v[0..n)).
static __global__ void __launch_bounds__(1024)
sum_fixed_kernel(const float* __restrict__ v, float* __restrict__ out, int n, float scale)
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

// Fixed-order two-level sums for the losses and the gradient norm.  Level 1: block b adds the
// contiguous chunk [b * chunk, (b + 1) * chunk) -- each thread a strided slice in ascending order,
// then a shared-memory tree of fixed shape -- and writes partial[b]; the number of blocks is a
// function of n alone (reduce_blocks), never of the SM count.  Level 2: sum_fixed_kernel over the
// partials.  MODE 0: sum of (a[i] - b[i])^2, and d[i] = dscale * (a[i] - b[i]) when d is not
// null (MseLoss forward + backward, src/Tensotron/TensorOps.Losses.cs:29-61).  MODE 1: sum of
// a[i]^2 (ClipGradNorm's sum of squares, src/Tensotron/Optimizers.cs:399-406).
constexpr int REDUCE_CHUNK = 4096;
static inline int reduce_blocks(long long n)
{
    long long b = (n + REDUCE_CHUNK - 1) / REDUCE_CHUNK;
    return static_cast<int>(b < 1 ? 1 : (b > 1024 ? 1024 : b));
}

template <int MODE>
static __global__ void __launch_bounds__(256)
reduce_partial_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ d,
                      float* __restrict__ partial, long long n, float dscale)
{
    __shared__ float red[256];
    const long long per = (n + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x;
    const long long hi = lo + per < n ? lo + per : n;
    float t = 0.f;
    for (long long i = lo + threadIdx.x; i < hi; i += 256) {
        if (MODE == 0) {
            const float diff = a[i] - b[i];
            t += diff * diff;
            if (d) d[i] = dscale * diff;
        } else {
            t += a[i] * a[i];
        }
    }
    red[threadIdx.x] = t;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}

// g[i] *= clamp(max_norm / (sqrt(*sumsq) + eps), 0, 1); *norm_out = sqrt(*sumsq) when not null
// (ClipGradNorm, src/Tensotron/Optimizers.cs:409-416: applied unconditionally, so nothing
// branches on the host).
static __global__ void __launch_bounds__(256)
clip_scale_kernel(float* __restrict__ g, const float* __restrict__ sumsq, long long n, float max_norm, float eps,
                  float* __restrict__ norm_out)
{
    const float total = sqrtf(*sumsq);
    const float coef = fminf(fmaxf(max_norm / (total + eps), 0.f), 1.f);
    if (norm_out && blockIdx.x == 0 && threadIdx.x == 0) *norm_out = total;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) g[i] *= coef;
}

// dst[kept...] = sum over the reduced axes of src, each output by one thread that walks the reduced
// index space in row-major (ascending) order: ReduceGradToShape
// (src/Tensotron/TensorOps.cs:76-100) without its atomic chunked reduction.  Up to 8 axes;
// kept / red: extents and source strides (elements) of the kept and of the reduced axes.
struct ReduceAxes {
    int n_kept, n_red;
    int kept_dim[8], red_dim[8];
    long long kept_stride[8], red_stride[8];
};

static __global__ void __launch_bounds__(256)
reduce_axes_kernel(const float* __restrict__ src, float* __restrict__ dst, ReduceAxes ax, long long n_out,
                   long long n_red)
{
    const long long o = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (o >= n_out) return;
    long long rem = o, base = 0;
    for (int i = ax.n_kept - 1; i >= 0; i--) {
        const long long c = rem % ax.kept_dim[i];
        rem /= ax.kept_dim[i];
        base += c * ax.kept_stride[i];
    }
    float t = 0.f;
    for (long long r = 0; r < n_red; r++) {
        long long q = r, off = base;
        for (int i = ax.n_red - 1; i >= 0; i--) {
            const long long c = q % ax.red_dim[i];
            q /= ax.red_dim[i];
            off += c * ax.red_stride[i];
        }
        t += src[off];
    }
    dst[o] = t;
}

// adv = [t, 1/(1-b1^t), 1/(1-b2^t)]; one thread.
static __global__ void adam_advance_kernel(float* adv, float b1, float b2)
{
    const float t = adv[0] + 1.f;
    adv[0] = t;
    adv[1] = 1.f / (1.f - powf(b1, t));
    adv[2] = 1.f / (1.f - powf(b2, t));
}

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, float b1,
                                         float omb1, float b2, float omb2, float lr, float eps,
                                         float ibc1, float ibc2, float cwd, float dfac)
{
    const float gi = g + cwd * p;
    const float mi = b1 * m + omb1 * gi;
    const float vi = b2 * v + omb2 * gi * gi;
    m = mi;
    v = vi;
    const float step = (mi * ibc1) / (sqrtf(vi * ibc2) + eps);
    p = p * dfac - lr * step;
}

template <bool VEC>
__global__ void __launch_bounds__(256)
adam_step_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                 float* __restrict__ v, const float* __restrict__ adv, long long n, float b1,
                 float b2, float lr, float eps, float cwd, float dfac)
{
    const float ibc1 = adv[1], ibc2 = adv[2];
    const float omb1 = 1.f - b1, omb2 = 1.f - b2;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (VEC) {
        const long long n4 = n >> 2;
        for (; i < n4; i += stride) {
            float4 pp = reinterpret_cast<float4*>(p)[i];
            const float4 gg = reinterpret_cast<const float4*>(g)[i];
            float4 mm = reinterpret_cast<float4*>(m)[i];
            float4 vv = reinterpret_cast<float4*>(v)[i];
            adam_one(pp.x, gg.x, mm.x, vv.x, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
            adam_one(pp.y, gg.y, mm.y, vv.y, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
            adam_one(pp.z, gg.z, mm.z, vv.z, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
            adam_one(pp.w, gg.w, mm.w, vv.w, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
            reinterpret_cast<float4*>(p)[i] = pp;
            reinterpret_cast<float4*>(m)[i] = mm;
            reinterpret_cast<float4*>(v)[i] = vv;
        }
        // scalar tail
        for (long long t = (n4 << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
             t < n; t += stride)
            adam_one(p[t], g[t], m[t], v[t], b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
    } else {
        for (; i < n; i += stride)
            adam_one(p[i], g[i], m[i], v[i], b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
    }
}

// dst[c * ld_dst + r] = src[r * ld_src + c] for an R x C matrix (R, C, both leading dimensions
// multiples of 4, both bases 16-byte aligned).  64 x 64 tiles through shared memory, 128-bit
// accesses on both sides.  Used to bring a large K-major GEMM operand into the MN-major form the
// FMA kernel reads without a shared-memory transposition.
static __global__ void __launch_bounds__(256)
transpose_kernel(const float* __restrict__ src, float* __restrict__ dst, int R, int C, long long ld_src,
                 long long ld_dst)
{
    __shared__ float t[64][65];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int q = threadIdx.x & 15, p = threadIdx.x >> 4;   // 16 float4 columns x 16 rows per pass
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = p + 16 * i, c = q * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r0 + r < R && c0 + c < C)
            v = *reinterpret_cast<const float4*>(src + static_cast<long long>(r0 + r) * ld_src + c0 + c);
        t[r][c] = v.x; t[r][c + 1] = v.y; t[r][c + 2] = v.z; t[r][c + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int c = p + 16 * i, r = q * 4;                // dst row c0 + c, dst columns r0 + r ..
        if (c0 + c < C && r0 + r < R)
            *reinterpret_cast<float4*>(dst + static_cast<long long>(c0 + c) * ld_dst + r0 + r) =
                make_float4(t[r][c], t[r + 1][c], t[r + 2][c], t[r + 3][c]);
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
add_into_kernel(float* __restrict__ target, const float* __restrict__ source, long long n)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (VEC) {
        const long long n4 = n >> 2;
        for (; i < n4; i += stride) {
            float4 t = reinterpret_cast<float4*>(target)[i];
            const float4 s = reinterpret_cast<const float4*>(source)[i];
            t.x += s.x; t.y += s.y; t.z += s.z; t.w += s.w;
            reinterpret_cast<float4*>(target)[i] = t;
        }
        for (long long t = (n4 << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
             t < n; t += stride)
            target[t] += source[t];
    } else {
        for (; i < n; i += stride) target[i] += source[i];
    }
}

}  // namespace ew
}  // namespace tt
