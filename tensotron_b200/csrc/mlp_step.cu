// tt_mlp_train_step: the whole training step of a small MLP as ONE kernel launch.
//
// The reference trains its control / PPO-sized networks (8 -> 64 -> 64 -> 2 and 4 -> 32 -> 32 -> 1,
// Tanh, batch 1 ... 512: showcase/Tensotron.Showcase/Rl/ActorCritic.cs:21-32,
// examples/Tensotron.Examples/BenchExample.cs:140-146) as forward + MseLoss + backward +
// ClipGradNorm + Adam, one launch per op, and its own measurements call that step 95 % host /
// launch bound.  For such a network everything fits on chip: 4866 parameters are 19 KB.  So the
// step runs as one thread-block cluster.  CTA c of the cluster
//   1. loads the parameters and its share of the batch rows into shared memory;
//   2. runs the forward pass, the loss, and the backward pass for its rows, all operands in shared
//      memory, leaving its partial weight / bias gradients there in the flat parameter layout;
//   3. after a cluster barrier, sums slice c of the gradients over all CTAs of the cluster
//      (distributed-shared-memory loads, ascending CTA rank: a fixed order) and the squares of
//      that slice; after a second barrier every CTA adds the per-slice sums of squares in rank
//      order, which gives every CTA the same gradient norm and clip coefficient
//      (src/Tensotron/Optimizers.cs:394-416: coef = clamp(maxNorm / (norm + eps), 0, 1), applied
//      unconditionally);
//   4. runs Adam (ew::adam_one, the arithmetic of tt_adam_step) on its slice and writes the new
//      parameters and moments to global memory.
// No atomics and no flag spinning anywhere: the only cross-CTA synchronisation is the hardware
// cluster barrier, and all CTAs of a cluster are co-scheduled by construction.
//
// The step is a chain of short dependent phases, and the first thing that bounds it is the
// instruction stream itself: code that runs once per launch is fetched from L2 line by line.  So
// the kernel is written for a small footprint: global -> shared copies are cp.async loops (no
// register staging, nothing unrolled), the two product forms are out-of-line functions shared by
// all their uses, the transcendental functions exist once, and the optimizer loop is rolled with
// its operands (moments prefetched by cp.async, summed gradients) in shared memory.
//
// Every operand keeps its natural row-major layout in shared memory; the only transposed copy is
// W^T (made once per launch), which the forward pass needs.  A thread owns 2 x 4 output blocks and
// walks the contraction index l in ascending order with one accumulator per output and fused
// multiply-adds (the summation rule of the large kernels).  Two forms cover the three products:
//   rows form   C[i][j] = sum_l P[i][l] * Q[l][j]   forward (x, W^T) and dX (g, W)
//   outer form  C[i][j] = sum_l P[l][i] * Q[l][j]   dW (g, x)
// Lanes of a warp differ in the column block j first, so the Q reads and the float4 stores of the
// results are contiguous and free of bank conflicts, and the P reads are broadcasts.
#include "../../include/tensotron_gemm.h"

#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <string.h>

#include "elementwise.cuh"
#include "mlp_step.h"
#include "ptx.cuh"

namespace cg = cooperative_groups;

namespace tt {
namespace mlp_step {

constexpr int THREADS = 256;

__host__ __device__ constexpr int pad4(int v) { return (v + 3) & ~3; }

// Shared-memory plan, identical on host and device.  All offsets in floats.
struct Plan {
    int n_layers, act, loss;
    int dims[MAX_LAYERS + 1];
    int rows;                 // batch rows per CTA (padded to a multiple of 4 for the layouts: rp)
    int rp;
    int total;                // floats of the flat parameter buffer (mlp layout: W_l (out,in), b_l, padded to 4)
    int w_off[MAX_LAYERS], b_off[MAX_LAYERS];   // flat offsets
    int k_magic[MAX_LAYERS];  // floor(2^20 / K_l) + 1: (rel * magic) >> 20 == rel / K_l for rel < 4096, K_l <= 64
    // shared-memory offsets
    int s_w[MAX_LAYERS];      // W_l      [N][Kp]
    int s_wt[MAX_LAYERS];     // W_l^T    [K][Np + 4]  (the extra 4 floats of pitch keep the transposing stores
                              //                         of 8 consecutive k in 8 different bank groups)
    int s_par;                // the parameters as loaded, flat layout [total] (biases; Adam's p)
    int s_grad;               // partial gradients, flat layout [total]
    int s_act[MAX_LAYERS + 1];   // activation l [rp][Dp_l]   (l = 0: the input)
    int s_g[2];               // gradient ping-pong [rp][gw], gw = widest padded layer output
    int gw;
    int s_red;                // 64 floats: block-reduction scratch [0, 32); [32 + 2r], [33 + 2r]: loss and
                              // sum-of-squares parts received from CTA r
    int per4;                 // float4s of the flat buffer one CTA owns in the optimizer part
    int s_m, s_v, s_sum;      // this CTA's slice of the moments and of the summed gradients [4 * per4] each
    int floats;               // total shared floats
};

inline Plan make_plan(const tt_mlp_desc& net, int rows, int ctas)
{
    Plan p;
    memset(&p, 0, sizeof(p));
    p.n_layers = net.n_layers;
    p.act = net.act;
    p.loss = net.loss;
    for (int i = 0; i <= net.n_layers; i++) p.dims[i] = net.dims[i];
    p.rows = rows;
    p.rp = pad4(rows);
    int cur = 0;
    for (int l = 0; l < net.n_layers; l++) {
        p.w_off[l] = cur;
        p.k_magic[l] = (1 << 20) / net.dims[l] + 1;
        cur += net.dims[l + 1] * net.dims[l];
        p.b_off[l] = cur;
        cur += net.dims[l + 1];
        cur = pad4(cur);
    }
    p.total = cur;
    int off = 0, widest = 4;
    p.s_par = off; off += p.total;
    for (int l = 0; l < net.n_layers; l++) {
        const int K = net.dims[l], N = net.dims[l + 1];
        // a weight matrix whose rows are whole float4s is used where the flat copy has it
        if ((K & 3) == 0) { p.s_w[l] = p.s_par + p.w_off[l]; }
        else              { p.s_w[l] = off;  off += pad4(N) * pad4(K); }
        p.s_wt[l] = off; off += pad4(K) * (pad4(N) + 4);
        if (pad4(N) > widest) widest = pad4(N);
    }
    p.s_grad = off; off += p.total;
    for (int l = 0; l <= net.n_layers; l++) {
        p.s_act[l] = off;  off += p.rp * pad4(net.dims[l]);
    }
    p.gw = widest;
    for (int i = 0; i < 2; i++) {
        p.s_g[i] = off;  off += p.rp * widest;
    }
    p.s_red = off; off += 64;
    p.per4 = ((p.total >> 2) + ctas - 1) / ctas;
    p.s_m = off;   off += 4 * p.per4;
    p.s_v = off;   off += 4 * p.per4;
    p.s_sum = off; off += 4 * p.per4;
    p.floats = off;
    return p;
}

struct Args {
    Plan plan;
    float* params;
    float* m;
    float* v;
    float* adv;
    float* grads_out;      // may be null
    const float* x;
    const void* target;    // float (batch, out) for MSE, int32 (batch) for cross-entropy
    float* loss_out;       // may be null
    unsigned int* status;  // handle status word (bad labels), may be null
    int batch;
    float lr, b1, b2, eps, max_norm, clip_eps;
    int advance;
    int x_vec;             // the input rows of every CTA start on 16 bytes and are whole float4s: copied by cp.async
};

// The functions below are deliberately NOT inlined: each exists once in the kernel's code.
__device__ __forceinline__ float act_one(float v, int act)
{
    if (act == TT_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == TT_ACT_TANH) return tanhf(v);
    return v;
}
// four values per call, so the four tanh chains overlap
__device__ __noinline__ float4 act_fwd4(float4 v, int act)
{
    return make_float4(act_one(v.x, act), act_one(v.y, act), act_one(v.z, act), act_one(v.w, act));
}

// 1 / (1 - b^t) for both moments, Adam's bias corrections (the arithmetic of tt_adam_advance); one
// call, so the two powf chains overlap
__device__ __noinline__ float2 inv_bias_corrections(float b1, float b2, float t)
{
    return make_float2(1.f / (1.f - powf(b1, t)), 1.f / (1.f - powf(b2, t)));
}

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(__cvta_generic_to_global(gmem_src))
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_but_last() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// acc[0..3] += a * b as two packed two-wide FP32 FMAs (each lane an IEEE fused multiply-add, so
// the bits equal four scalar fmaf).
__device__ __forceinline__ void fma_row4(float (&acc)[4], float a, const float4 b)
{
    const float2 ap = make_float2(a, a);
    float2 r;
    r = __ffma2_rn(ap, make_float2(b.x, b.y), make_float2(acc[0], acc[1])); acc[0] = r.x; acc[1] = r.y;
    r = __ffma2_rn(ap, make_float2(b.z, b.w), make_float2(acc[2], acc[3])); acc[2] = r.x; acc[3] = r.y;
}

// Outer form: out[i * ldo + j] = sum_l P[l * ldp + i] * Q[l * ldq + j] for i < I, j < J (l ascending,
// one accumulator per output, fused multiply-add).  A thread owns IB x 4 output blocks (IB = 4 halves
// the shared-memory bytes per FMA and is used when it still gives every second thread a block).
// ldp >= I rounded up to IB, ldq >= J rounded up to 4; what lies in those roundings may be
// anything, it only reaches outputs that are not written.  Used for dW (P = g, Q = x, out = the
// flat gradient).
template <int IB>
__device__ __noinline__ void product_outer(const float* __restrict__ P, int ldp, const float* __restrict__ Q, int ldq,
                                           int I, int J, int L, float* __restrict__ out, int ldo)
{
    const int ib_n = (I + IB - 1) / IB, jb_n = (J + 3) >> 2;
    const bool vec = (ldo & 3) == 0;
    for (int blk = threadIdx.x; blk < ib_n * jb_n; blk += THREADS) {
        const int jb = blk % jb_n, ib = blk / jb_n;
        const float* pp = P + IB * ib;
        const float* qq = Q + 4 * jb;
        float acc[IB][4];
#pragma unroll
        for (int r = 0; r < IB; r++) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
#pragma unroll 4
        for (int l = 0; l < L; l++) {
            const float4 b = *reinterpret_cast<const float4*>(qq + l * ldq);
            if constexpr (IB == 4) {
                const float4 a = *reinterpret_cast<const float4*>(pp + l * ldp);
                fma_row4(acc[0], a.x, b);
                fma_row4(acc[1], a.y, b);
                fma_row4(acc[2], a.z, b);
                fma_row4(acc[3], a.w, b);
            } else {
                const float2 a = *reinterpret_cast<const float2*>(pp + l * ldp);
                fma_row4(acc[0], a.x, b);
                fma_row4(acc[1], a.y, b);
            }
        }
#pragma unroll
        for (int r = 0; r < IB; r++) {
            const int i = IB * ib + r, j0 = 4 * jb;
            if (i >= I) continue;
            float* d = out + i * ldo + j0;
            if (vec) {
                *reinterpret_cast<float4*>(d) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
            } else {
                d[0] = acc[r][0];
                if (j0 + 1 < J) d[1] = acc[r][1];
                if (j0 + 2 < J) d[2] = acc[r][2];
                if (j0 + 3 < J) d[3] = acc[r][3];
            }
        }
    }
}

// Rows form: acc[i][j] = sum_l P[i * ldp + l] * Q[l * ldq + j], same rules.  The P rows are read four l
// at a time (ldp a multiple of 4); the l beyond a multiple of 4 are done one by one, so nothing past
// L enters a sum.  Rows i >= I of P are read (into results that are not written): P must have
// I rounded up to 2 rows.  What is written (128 bits per row and column block, ldo a multiple of 4):
//   forward (FWD)  out[i][j] = act(acc + aux[j])                      aux = the bias vector, 0 beyond J
//   backward       out[i][j] = acc * act'(aux[i * lda + j])           aux = the layer's forward output
constexpr int ROWS_FWD = 0, ROWS_BWD = 1;
__device__ __noinline__ void product_rows(const float* __restrict__ P, int ldp, const float* __restrict__ Q, int ldq,
                                          int I, int J, int L, int mode, int act, const float* __restrict__ aux, int lda,
                                          float* __restrict__ out, int ldo)
{
    const int ib_n = (I + 1) >> 1, jb_n = (J + 3) >> 2;
    const int L4 = L & ~3;
    // Few output blocks (a handful of batch rows): the contraction is cut over the four 8-lane
    // groups of a warp, so a thread's chain of dependent FMAs is a quarter as long; the four partial
    // sums are added by a fixed xor-shuffle tree ((q0 + q1) + (q2 + q3), the same bits in all lanes).
    const bool cut = ib_n * jb_n * 4 <= THREADS && L4 >= 16;
    const int lane = threadIdx.x & 31;
    const int kq = cut ? lane >> 3 : 0;
    const int first = cut ? (threadIdx.x >> 5) * 8 + (lane & 7) : threadIdx.x;
    const int groups = L4 >> 2, gpq = cut ? (groups + 3) >> 2 : groups;
    const int l_lo = 4 * min(groups, kq * gpq), l_hi = 4 * min(groups, (kq + 1) * gpq);
    const int nblk = ib_n * jb_n;
    const int blk_end = cut ? ((nblk + 7) & ~7) : nblk;      // whole 8-lane groups enter the shuffles together
    for (int blk = first; blk < blk_end; blk += THREADS) {
        const bool live = blk < nblk;
        const int jb = live ? blk % jb_n : 0, ib = live ? blk / jb_n : 0;
        const float* p0 = P + (2 * ib) * ldp;
        const float* qq = Q + 4 * jb;
        float acc[2][4];
#pragma unroll
        for (int r = 0; r < 2; r++) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
#pragma unroll 2
        for (int l = l_lo; l < l_hi; l += 4) {
            float4 a[2];
#pragma unroll
            for (int r = 0; r < 2; r++) a[r] = *reinterpret_cast<const float4*>(p0 + r * ldp + l);
            const float4 b0 = *reinterpret_cast<const float4*>(qq + l * ldq);
            const float4 b1 = *reinterpret_cast<const float4*>(qq + (l + 1) * ldq);
            const float4 b2 = *reinterpret_cast<const float4*>(qq + (l + 2) * ldq);
            const float4 b3 = *reinterpret_cast<const float4*>(qq + (l + 3) * ldq);
#pragma unroll
            for (int r = 0; r < 2; r++) {
                fma_row4(acc[r], a[r].x, b0);
                fma_row4(acc[r], a[r].y, b1);
                fma_row4(acc[r], a[r].z, b2);
                fma_row4(acc[r], a[r].w, b3);
            }
        }
        if (!cut || kq == 3) {
#pragma unroll 1
            for (int l = L4; l < L; l++) {
                const float4 b = *reinterpret_cast<const float4*>(qq + l * ldq);
#pragma unroll
                for (int r = 0; r < 2; r++) fma_row4(acc[r], p0[r * ldp + l], b);
            }
        }
        if (cut) {
#pragma unroll
            for (int r = 0; r < 2; r++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[r][j] += __shfl_xor_sync(0xffffffffu, acc[r][j], 8);
                    acc[r][j] += __shfl_xor_sync(0xffffffffu, acc[r][j], 16);
                }
            if (kq != 0) continue;
        }
        if (!live) continue;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int i = 2 * ib + r, j0 = 4 * jb;
            if (i >= I) continue;
            float4 v;
            if (mode == ROWS_FWD) {
                // (reading up to 3 floats past the bias vector stays inside the shared-memory block;
                // those lanes are zeroed below)
                v = make_float4(acc[r][0] + aux[j0], acc[r][1] + aux[j0 + 1], acc[r][2] + aux[j0 + 2], acc[r][3] + aux[j0 + 3]);
                if (act != TT_ACT_NONE) v = act_fwd4(v, act);
                if (j0 + 1 >= J) v.y = 0.f;
                if (j0 + 2 >= J) v.z = 0.f;
                if (j0 + 3 >= J) v.w = 0.f;
            } else {
                const float4 y = *reinterpret_cast<const float4*>(aux + i * lda + j0);
                v = make_float4(ew::act_grad(y.x, acc[r][0], act), ew::act_grad(y.y, acc[r][1], act),
                                ew::act_grad(y.z, acc[r][2], act), ew::act_grad(y.w, acc[r][3], act));
            }
            *reinterpret_cast<float4*>(out + i * ldo + j0) = v;
        }
    }
}

// Sum of v over the CTA in a fixed order: each thread's value, then a shared-memory tree.
__device__ __noinline__ float block_sum(float v, float* scratch /* >= 32 floats */)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; w++) t += scratch[w];
    return t;
}

__global__ void __launch_bounds__(THREADS, 1) mlp_train_step_kernel(const Args a)
{
    extern __shared__ float4 smem4[];
    float* s = reinterpret_cast<float*>(smem4);
    const Plan& p = a.plan;
    cg::cluster_group cluster = cg::this_cluster();
    const int C = static_cast<int>(cluster.num_blocks());
    const int c = static_cast<int>(cluster.block_rank());
    const int tid = threadIdx.x;
    const int L = p.n_layers;
    const int row0 = c * p.rows;                                  // first batch row of this CTA
    const int nrows = max(0, min(p.rows, a.batch - row0));        // rows that exist
    const int NO = p.dims[L], NOp = pad4(NO);
    const int total4 = p.total >> 2;
    const int lo4 = min(total4, c * p.per4), hi4 = min(total4, lo4 + p.per4);   // the optimizer slice of this CTA

    // ---- 1. global -> shared ---------------------------------------------------------------------
    // Everything the step reads from global memory is requested here, before anything waits:
    // the parameters and the input rows (first cp.async group), this CTA's slice of the Adam
    // moments (second group, consumed after the two cluster barriers), the step state and each
    // thread's first loss target (registers).
#pragma unroll 1
    for (int i = tid; i < total4; i += THREADS) cp_async16(s + p.s_par + 4 * i, a.params + 4 * i);
    const int K0 = p.dims[0];
    if (a.x_vec) {
        const float* xr = a.x + static_cast<long long>(row0) * K0;
#pragma unroll 1
        for (int i = tid; i < (nrows * K0) >> 2; i += THREADS) cp_async16(s + p.s_act[0] + 4 * i, xr + 4 * i);
    }
    cp_async_commit();
#pragma unroll 1
    for (int i = lo4 + tid; i < hi4; i += THREADS) {
        cp_async16(s + p.s_m + 4 * (i - lo4), a.m + 4 * i);
        cp_async16(s + p.s_v + 4 * (i - lo4), a.v + 4 * i);
    }
    cp_async_commit();
    const float adv_t = a.adv[0], adv_ibc1 = a.adv[1], adv_ibc2 = a.adv[2];
    float tgt_first = 0.f;
    int label_first = 0;
    if (p.loss == TT_LOSS_MSE) {
        if (tid < nrows * NO) tgt_first = static_cast<const float*>(a.target)[static_cast<long long>(row0) * NO + tid];
    } else if (tid < nrows) {
        label_first = static_cast<const int*>(a.target)[row0 + tid];
    }
    // Only the gradient buffer has to start at zero (its padding floats between the layers are
    // summed like everything else).  The paddings of the operand tiles may hold anything: a
    // product reads them only into outputs that are never written.
#pragma unroll 1
    for (int i = tid; i < total4; i += THREADS) reinterpret_cast<float4*>(s + p.s_grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!a.x_vec) {
        const int Kp = pad4(K0);
#pragma unroll 1
        for (int i = tid; i < nrows * K0; i += THREADS)
            s[p.s_act[0] + (i / K0) * Kp + (i % K0)] = a.x[static_cast<long long>(row0) * K0 + i];
    }
    cp_async_wait_all_but_last();
    __syncthreads();
    // Row-major W with rows padded to whole float4s (only layers whose K is not a multiple of 4:
    // the others are used in place in the flat copy), then W^T for the forward pass: thread <->
    // (k, four rows n): four reads down a column of W (lanes on consecutive k), one 128-bit store
    // into row k of W^T.
#pragma unroll 1
    for (int l = 0; l < L; l++) {
        const int K = p.dims[l], N = p.dims[l + 1], Kp = pad4(K);
        if ((K & 3) == 0) continue;
        const float* src = s + p.s_par + p.w_off[l];
        float* w = s + p.s_w[l];
#pragma unroll 1
        for (int i = tid; i < N * K; i += THREADS) w[(i / K) * Kp + (i % K)] = src[i];
    }
    __syncthreads();
#pragma unroll 1
    for (int l = 0; l < L; l++) {
        const int K = p.dims[l], N = p.dims[l + 1], Kp = pad4(K), Npt = pad4(N) + 4, n4_n = (N + 3) >> 2;
        const float* w = s + p.s_w[l];
        float* wt = s + p.s_wt[l];
#pragma unroll 2
        for (int i = tid; i < K * n4_n; i += THREADS) {
            const int n4 = i / K, k = i - n4 * K;
            float4 v;
            v.x = w[(4 * n4) * Kp + k];
            v.y = 4 * n4 + 1 < N ? w[(4 * n4 + 1) * Kp + k] : 0.f;
            v.z = 4 * n4 + 2 < N ? w[(4 * n4 + 2) * Kp + k] : 0.f;
            v.w = 4 * n4 + 3 < N ? w[(4 * n4 + 3) * Kp + k] : 0.f;
            *reinterpret_cast<float4*>(wt + k * Npt + 4 * n4) = v;
        }
    }
    __syncthreads();

    // ---- 2a. forward: y[r][n] = act(sum_k x[r][k] * W^T[k][n] + b[n]) ---------------------------------
#pragma unroll 1
    for (int l = 0; l < L; l++) {
        const int K = p.dims[l], N = p.dims[l + 1];
        product_rows(s + p.s_act[l], pad4(K), s + p.s_wt[l], pad4(N) + 4, nrows, N, K, ROWS_FWD,
                     l + 1 < L ? p.act : TT_ACT_NONE, s + p.s_par + p.b_off[l], 0, s + p.s_act[l + 1], pad4(N));
        __syncthreads();
    }

    // ---- 2b. loss and its gradient w.r.t. the network output ---------------------------------
    const float* out = s + p.s_act[L];
    int gcur = 0;                         // ping-pong index of the current upstream gradient
    float* g = s + p.s_g[gcur];
    const int gw = p.gw;                  // row pitch of the gradient buffers
    float loss_part = 0.f;
    if (p.loss == TT_LOSS_MSE) {
        // mean over batch x outputs of (o - t)^2; d/do = 2 (o - t) / count   (TensorOps.Losses.cs:29-61)
        const float* tgt = static_cast<const float*>(a.target);
        const float inv = 1.f / (static_cast<float>(a.batch) * static_cast<float>(NO));
#pragma unroll 1
        for (int i = tid; i < nrows * NO; i += THREADS) {
            const int r = i / NO, n = i - r * NO;
            const float d = out[r * NOp + n] - (i == tid ? tgt_first : tgt[static_cast<long long>(row0) * NO + i]);
            loss_part += d * d;
            g[r * gw + n] = (2.f * inv) * d;
        }
        loss_part *= inv;
    } else {
        // softmax cross-entropy, mean over the batch, int32 labels (TensorOps.Losses.cs:97-108)
        const int* labels = static_cast<const int*>(a.target);
        const float inv = 1.f / static_cast<float>(a.batch);
#pragma unroll 1
        for (int r = tid; r < nrows; r += THREADS) {
            float mx = -INFINITY;
#pragma unroll 1
            for (int n = 0; n < NO; n++) mx = fmaxf(mx, out[r * NOp + n]);
            float se = 0.f;
#pragma unroll 1
            for (int n = 0; n < NO; n++) se += expf(out[r * NOp + n] - mx);
            const float lse = logf(se) + mx;
            const int label = r == tid ? label_first : labels[row0 + r];
            const bool ok = label >= 0 && label < NO;
            if (!ok && a.status) atomicCAS(a.status, 0u, 7u);
            loss_part += ok ? -(out[r * NOp + label] - lse) * inv : __int_as_float(0x7fc00000);
#pragma unroll 1
            for (int n = 0; n < NO; n++)
                g[r * gw + n] = (expf(out[r * NOp + n] - lse) - (n == label ? 1.f : 0.f)) * inv;
        }
    }
    float* red = s + p.s_red;
    const float loss_cta = block_sum(loss_part, red);
    __syncthreads();

    // ---- 2c. backward -------------------------------------------------------------------------
    float* grad = s + p.s_grad;
#pragma unroll 1
    for (int l = L - 1; l >= 0; l--) {
        const int K = p.dims[l], N = p.dims[l + 1], Kp = pad4(K);
        // dW[n][k] = sum_r g[r][n] * x[r][k]
        if (((N + 3) >> 2) * ((K + 3) >> 2) * 2 >= THREADS) product_outer<4>(g, gw, s + p.s_act[l], Kp, N, K, nrows, grad + p.w_off[l], K);
        else                                                product_outer<2>(g, gw, s + p.s_act[l], Kp, N, K, nrows, grad + p.w_off[l], K);
        // db[n] = sum_r g[r][n], ascending r
        float* db = grad + p.b_off[l];
#pragma unroll 1
        for (int n = tid; n < N; n += THREADS) {
            float t = 0.f;
#pragma unroll 4
            for (int r = 0; r < nrows; r++) t += g[r * gw + n];
            db[n] = t;
        }
        if (l > 0) {
            // dx[r][k] = sum_n g[r][n] * W[n][k], then through the activation of layer l - 1
            float* gn = s + p.s_g[gcur ^ 1];
            product_rows(g, gw, s + p.s_w[l], Kp, nrows, K, N, ROWS_BWD, p.act, s + p.s_act[l], Kp, gn, gw);
            __syncthreads();
            gcur ^= 1;
            g = gn;
        }
    }

    // ---- 3. cluster-wide gradient sum (slice per CTA), gradient norm ---------------------------
    // The optimizer's bias corrections (two powf) are register work that depends on nothing of this
    // step: they fill the time between arriving at the first cluster barrier and its completion.
    cluster.barrier_arrive();
    float t = adv_t, ibc1 = adv_ibc1, ibc2 = adv_ibc2;
    if (a.advance) {
        t += 1.f;
        const float2 ibc = inv_bias_corrections(a.b1, a.b2, t);
        ibc1 = ibc.x;
        ibc2 = ibc.y;
    }
    cluster.barrier_wait();
    float sq = 0.f;
    float* own = s + p.s_sum;             // the summed gradients of this CTA's slice
#pragma unroll 1
    for (int i = lo4 + tid; i < hi4; i += THREADS) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int r = 0; r < C; r++) {        // (unrolled: four remote loads in flight, still added in rank order)
            const float4 q = reinterpret_cast<const float4*>(cluster.map_shared_rank(grad, r))[i];
            sum.x += q.x; sum.y += q.y; sum.z += q.z; sum.w += q.w;
        }
        sq += sum.x * sum.x; sq += sum.y * sum.y; sq += sum.z * sum.z; sq += sum.w * sum.w;
        reinterpret_cast<float4*>(own)[i - lo4] = sum;
    }
    const float sq_cta = block_sum(sq, red);
    // Every CTA hands its two partial sums (loss, sum of squares of its slice) to every CTA of the
    // cluster: thread r stores them into slot c of CTA r's shared memory.  After the barrier each
    // CTA adds the slots it holds in rank order, and nothing reads another CTA's shared memory any
    // more, so a CTA may finish while the others are still in their Adam loops.
    if (tid < C) {
        float* rr = cluster.map_shared_rank(red, tid);
        rr[32 + 2 * c] = loss_cta;
        rr[33 + 2 * c] = sq_cta;
    }
    cluster.sync();
    float total_sq = 0.f, loss_total = 0.f;
#pragma unroll 4
    for (int r = 0; r < C; r++) {
        loss_total += red[32 + 2 * r];
        total_sq += red[33 + 2 * r];
    }
    float coef = 1.f;
    if (a.max_norm > 0.f) {
        const float norm = sqrtf(total_sq);
        coef = fminf(fmaxf(a.max_norm / (norm + a.clip_eps), 0.f), 1.f);
    }
    if (c == 0 && tid == 0 && a.loss_out) *a.loss_out = loss_total;

    // ---- 4. Adam on this CTA's slice ------------------------------------------------------------
    const float omb1 = 1.f - a.b1, omb2 = 1.f - a.b2;
    cp_async_wait_all();                  // each thread consumes the moments it requested itself
#pragma unroll 1
    for (int i = lo4 + tid; i < hi4; i += THREADS) {
        float4 gg = reinterpret_cast<const float4*>(own)[i - lo4];
        if (a.max_norm > 0.f) { gg.x *= coef; gg.y *= coef; gg.z *= coef; gg.w *= coef; }
        float4 pp = reinterpret_cast<const float4*>(s + p.s_par)[i];
        float4 mm = reinterpret_cast<const float4*>(s + p.s_m)[i - lo4];
        float4 vv = reinterpret_cast<const float4*>(s + p.s_v)[i - lo4];
        ew::adam_one(pp.x, gg.x, mm.x, vv.x, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        ew::adam_one(pp.y, gg.y, mm.y, vv.y, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        ew::adam_one(pp.z, gg.z, mm.z, vv.z, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        ew::adam_one(pp.w, gg.w, mm.w, vv.w, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        reinterpret_cast<float4*>(a.params)[i] = pp;
        reinterpret_cast<float4*>(a.m)[i] = mm;
        reinterpret_cast<float4*>(a.v)[i] = vv;
        if (a.grads_out) reinterpret_cast<float4*>(a.grads_out)[i] = gg;
    }
    // (every CTA read the step state into registers before the first cluster barrier)
    if (c == 0 && tid == 0 && a.advance) {
        a.adv[0] = t;
        a.adv[1] = ibc1;
        a.adv[2] = ibc2;
    }
}


// Largest cluster the device schedules for this kernel at its largest shared-memory size: 16
// (needs the non-portable attribute) where possible, else the portable 8.
static int g_max_cluster = 8;

int init_device()
{
    if (cudaFuncSetAttribute(mlp_train_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM_BYTES) != cudaSuccess) return 1;
    g_max_cluster = 8;
    if (cudaFuncSetAttribute(mlp_train_step_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(MAX_CLUSTER, 1, 1);
        cfg.blockDim = dim3(THREADS, 1, 1);
        cfg.dynamicSmemBytes = MAX_SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = MAX_CLUSTER;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, mlp_train_step_kernel, &cfg) == cudaSuccess && n >= 1) g_max_cluster = MAX_CLUSTER;
        else cudaGetLastError();
    } else {
        cudaGetLastError();
    }
    return 0;
}

int launch(cudaStream_t st, const tt_mlp_desc* net, float* params, float* m, float* v, float* adv, float* grads_out,
           const float* x, const void* target, float* loss_out, unsigned int* status, int batch, float lr, float b1,
           float b2, float eps, float max_norm, float clip_eps, int advance, int* n_ctas)
{
    if (net->n_layers < 1 || net->n_layers > MAX_LAYERS) return TT_ERR_UNSUPPORTED;
    for (int i = 0; i <= net->n_layers; i++)
        if (net->dims[i] < 1 || net->dims[i] > MAX_WIDTH) return TT_ERR_UNSUPPORTED;
    if (batch < 1 || batch > g_max_cluster * MAX_ROWS) return TT_ERR_UNSUPPORTED;
    // Cluster size: about 8 rows per CTA up to the largest cluster, then more rows per CTA.  The
    // choice depends on the batch only, so the summation order does too.
    // At least four CTAs: the optimizer part (a slice of the parameters per CTA) is worth
    // spreading even when one CTA holds all the rows.
    int C = g_max_cluster < 4 ? g_max_cluster : 4;
    while (C < g_max_cluster && batch > 8 * C) C *= 2;
    int rows = (batch + C - 1) / C;
    Plan plan = make_plan(*net, rows, C);
    if (static_cast<size_t>(plan.floats) * sizeof(float) > MAX_SMEM_BYTES) return TT_ERR_UNSUPPORTED;
    // the flat buffers are moved 128 bits at a time
    const auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!aligned16(params) || !aligned16(m) || !aligned16(v) || !aligned16(grads_out)) return TT_ERR_UNSUPPORTED;
    Args a;
    a.plan = plan;
    a.params = params; a.m = m; a.v = v; a.adv = adv; a.grads_out = grads_out;
    a.x = x; a.target = target; a.loss_out = loss_out; a.status = status;
    a.batch = batch;
    a.lr = lr; a.b1 = b1; a.b2 = b2; a.eps = eps; a.max_norm = max_norm; a.clip_eps = clip_eps;
    a.advance = advance;
    a.x_vec = (net->dims[0] % 4 == 0) && aligned16(x);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(C, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(plan.floats) * sizeof(float);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, mlp_train_step_kernel, a) != cudaSuccess) {
        cudaGetLastError();
        return TT_ERR_CUDA;
    }
    if (n_ctas) *n_ctas = C;
    return TT_OK;
}

}  // namespace mlp_step
}  // namespace tt
