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
// Every small product is C[i][j] = sum_l P[l][i] * Q[l][j] on operands stored with the contraction
// index outermost, so a thread reads 2 + 4 consecutive values per l and does 8 FMAs, in ascending l
// (one accumulator per output, fused multiply-add: the same summation rule as the large kernels).
// That needs each activation and each gradient in both orientations, which the producing
// product writes for free from its 2 x 4 register block.
#include "../../include/tensotron_gemm.h"

#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <string.h>

#include "elementwise.cuh"
#include "mlp_step.h"

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
    // shared-memory offsets
    int s_w[MAX_LAYERS];      // W_l natural  [N][Kp]
    int s_wt[MAX_LAYERS];     // W_l^T        [K][Np]
    int s_grad;               // partial gradients, flat layout [total]
    int s_act[MAX_LAYERS + 1];   // activation l natural [rp][Dp_l]   (l = 0: the input)
    int s_actt[MAX_LAYERS + 1];  // activation l transposed [D_l][rp]
    int s_g[2], s_gt[2];      // gradient ping-pong: natural [rp][Wp], transposed [W][rp], W = widest layer output
    int s_red;                // 64 floats: block-reduction scratch; [32..48) this CTA's published partial sums
    int floats;               // total shared floats
};

inline Plan make_plan(const tt_mlp_desc& net, int rows)
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
        cur += net.dims[l + 1] * net.dims[l];
        p.b_off[l] = cur;
        cur += net.dims[l + 1];
        cur = pad4(cur);
    }
    p.total = cur;
    int off = 0, widest = 4;
    for (int l = 0; l < net.n_layers; l++) {
        const int K = net.dims[l], N = net.dims[l + 1];
        p.s_w[l] = off;  off += N * pad4(K);
        p.s_wt[l] = off; off += K * pad4(N);
        if (pad4(N) > widest) widest = pad4(N);
    }
    p.s_grad = off; off += p.total;
    for (int l = 0; l <= net.n_layers; l++) {
        p.s_act[l] = off;  off += p.rp * pad4(net.dims[l]);
        p.s_actt[l] = off; off += net.dims[l] * p.rp;
    }
    for (int i = 0; i < 2; i++) {
        p.s_g[i] = off;  off += p.rp * widest;
        p.s_gt[i] = off; off += widest * p.rp;
    }
    p.s_red = off; off += 64;
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
};

__device__ __forceinline__ float act_fwd(float v, int act)
{
    if (act == TT_ACT_RELU) return v > 0.f ? v : 0.f;
    if (act == TT_ACT_TANH) return tanhf(v);
    return v;
}

// C[i][j] = sum_l P[l * ldp + i] * Q[l * ldq + j] for i < I, j < J (l ascending, one accumulator
// per output, fused multiply-add).  ldp >= pad-to-2(I), ldq >= pad4(J), both buffers readable (zero
// or finite) up to those paddings.  Each thread owns 2 x 4 output blocks; `emit(i, j, value)` is
// called for every in-range output.
template <typename Emit>
__device__ __forceinline__ void small_gemm(const float* __restrict__ P, int ldp, const float* __restrict__ Q, int ldq,
                                           int I, int J, int L, Emit emit)
{
    const int ib_n = (I + 1) >> 1, jb_n = (J + 3) >> 2;
    for (int blk = threadIdx.x; blk < ib_n * jb_n; blk += THREADS) {
        const int ib = blk % ib_n, jb = blk / ib_n;
        const float* pp = P + 2 * ib;
        const float* qq = Q + 4 * jb;
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
        for (int l = 0; l < L; l++) {
            const float2 a = *reinterpret_cast<const float2*>(pp + l * ldp);
            const float4 b = *reinterpret_cast<const float4*>(qq + l * ldq);
            acc[0][0] = fmaf(a.x, b.x, acc[0][0]); acc[0][1] = fmaf(a.x, b.y, acc[0][1]);
            acc[0][2] = fmaf(a.x, b.z, acc[0][2]); acc[0][3] = fmaf(a.x, b.w, acc[0][3]);
            acc[1][0] = fmaf(a.y, b.x, acc[1][0]); acc[1][1] = fmaf(a.y, b.y, acc[1][1]);
            acc[1][2] = fmaf(a.y, b.z, acc[1][2]); acc[1][3] = fmaf(a.y, b.w, acc[1][3]);
        }
#pragma unroll
        for (int di = 0; di < 2; di++)
#pragma unroll
            for (int dj = 0; dj < 4; dj++) {
                const int i = 2 * ib + di, j = 4 * jb + dj;
                if (i < I && j < J) emit(i, j, acc[di][dj]);
            }
    }
}

// Sum of v over the CTA in a fixed order: each thread's value, then a shared-memory tree.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
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
    const int L = p.n_layers, rp = p.rp;
    const int row0 = c * p.rows;                                  // first batch row of this CTA
    const int nrows = max(0, min(p.rows, a.batch - row0));        // rows that exist

    // ---- 1. clear, load parameters (both orientations) and the input rows -------------------
    for (int i = tid; i < p.floats; i += THREADS) s[i] = 0.f;
    __syncthreads();
    // parameters: 128-bit loads over the flat buffer (all in flight at once), each element
    // scattered into the natural and the transposed copy of its weight matrix
    for (int i4 = tid; i4 < (p.total >> 2); i4 += THREADS) {
        const float4 q = reinterpret_cast<const float4*>(a.params)[i4];
        const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int flat = 4 * i4 + j;
            for (int l = 0; l < L; l++) {
                if (flat >= p.w_off[l] && flat < p.b_off[l]) {
                    const int K = p.dims[l], rel = flat - p.w_off[l];
                    const int n = rel / K, k = rel - n * K;
                    s[p.s_w[l] + n * pad4(K) + k] = e[j];
                    s[p.s_wt[l] + k * pad4(p.dims[l + 1]) + n] = e[j];
                }
            }
        }
    }
    {
        const int K = p.dims[0], Kp = pad4(K);
        for (int i = tid; i < nrows * K; i += THREADS) {
            const int r = i / K, k = i - r * K;
            const float val = a.x[static_cast<long long>(row0 + r) * K + k];
            s[p.s_act[0] + r * Kp + k] = val;
            s[p.s_actt[0] + k * rp + r] = val;
        }
    }
    __syncthreads();

    // ---- 2a. forward ------------------------------------------------------------------------
    for (int l = 0; l < L; l++) {
        const int K = p.dims[l], N = p.dims[l + 1], Np = pad4(N);
        const float* bias = a.params + p.b_off[l];
        const int act = l + 1 < L ? p.act : TT_ACT_NONE;
        float* y = s + p.s_act[l + 1];
        float* yt = s + p.s_actt[l + 1];
        // y[r][n] = sum_k x^T[k][r] * W^T[k][n]
        small_gemm(s + p.s_actt[l], rp, s + p.s_wt[l], Np, nrows, N, K, [&](int r, int n, float v) {
            v = act_fwd(v + __ldg(bias + n), act);
            y[r * Np + n] = v;
            yt[n * rp + r] = v;
        });
        __syncthreads();
    }

    // ---- 2b. loss and its gradient w.r.t. the network output ---------------------------------
    const int NO = p.dims[L], NOp = pad4(NO);
    const float* out = s + p.s_act[L];
    int gcur = 0;                         // ping-pong index of the current upstream gradient
    float* g = s + p.s_g[gcur];
    float* gt = s + p.s_gt[gcur];
    const int gw = (p.s_gt[0] - p.s_g[0]) / rp;   // row pitch of the natural gradient buffers
    float loss_part = 0.f;
    if (p.loss == TT_LOSS_MSE) {
        // mean over batch x outputs of (o - t)^2; d/do = 2 (o - t) / count   (TensorOps.Losses.cs:29-61)
        const float* tgt = static_cast<const float*>(a.target);
        const float inv = 1.f / (static_cast<float>(a.batch) * static_cast<float>(NO));
        for (int i = tid; i < nrows * NO; i += THREADS) {
            const int r = i / NO, n = i - r * NO;
            const float d = out[r * NOp + n] - tgt[static_cast<long long>(row0 + r) * NO + n];
            loss_part += d * d;
            const float gv = (2.f * inv) * d;
            g[r * gw + n] = gv;
            gt[n * rp + r] = gv;
        }
        loss_part *= inv;
    } else {
        // softmax cross-entropy, mean over the batch, int32 labels (TensorOps.Losses.cs:97-108)
        const int* labels = static_cast<const int*>(a.target);
        const float inv = 1.f / static_cast<float>(a.batch);
        for (int r = tid; r < nrows; r += THREADS) {
            float mx = -INFINITY;
            for (int n = 0; n < NO; n++) mx = fmaxf(mx, out[r * NOp + n]);
            float se = 0.f;
            for (int n = 0; n < NO; n++) se += expf(out[r * NOp + n] - mx);
            const float lse = logf(se) + mx;
            const int label = labels[row0 + r];
            const bool ok = label >= 0 && label < NO;
            if (!ok && a.status) atomicCAS(a.status, 0u, 7u);
            loss_part += ok ? -(out[r * NOp + label] - lse) * inv : __int_as_float(0x7fc00000);
            for (int n = 0; n < NO; n++) {
                const float gv = (expf(out[r * NOp + n] - lse) - (n == label ? 1.f : 0.f)) * inv;
                g[r * gw + n] = gv;
                gt[n * rp + r] = gv;
            }
        }
    }
    float* red = s + p.s_red;
    const float loss_cta = block_sum(loss_part, red);
    if (tid == 0) red[32] = loss_cta;     // published: CTA 0 adds the CTAs' parts in rank order
    __syncthreads();

    // ---- 2c. backward -------------------------------------------------------------------------
    float* grad = s + p.s_grad;
    for (int l = L - 1; l >= 0; l--) {
        const int K = p.dims[l], N = p.dims[l + 1], Kp = pad4(K);
        // dW[n][k] = sum_r g[r][n] * x[r][k]
        float* dw = grad + p.w_off[l];
        small_gemm(g, gw, s + p.s_act[l], Kp, N, K, nrows, [&](int n, int k, float v) { dw[n * K + k] = v; });
        // db[n] = sum_r g[r][n], ascending r
        float* db = grad + p.b_off[l];
        for (int n = tid; n < N; n += THREADS) {
            float t = 0.f;
            for (int r = 0; r < nrows; r++) t += g[r * gw + n];
            db[n] = t;
        }
        if (l > 0) {
            // dx[r][k] = sum_n g^T[n][r] * W[n][k], then through the activation of layer l - 1
            const float* h = s + p.s_act[l];
            float* gn = s + p.s_g[gcur ^ 1];
            float* gnt = s + p.s_gt[gcur ^ 1];
            const int act = p.act;
            small_gemm(gt, rp, s + p.s_w[l], Kp, nrows, K, N, [&](int r, int k, float v) {
                const float y = h[r * Kp + k];
                v = ew::act_grad(y, v, act);
                gn[r * gw + k] = v;
                gnt[k * rp + r] = v;
            });
            __syncthreads();
            gcur ^= 1;
            g = gn;
            gt = gnt;
        }
    }
    __syncthreads();

    // ---- 3. cluster-wide gradient sum (slice per CTA), gradient norm ---------------------------
    cluster.sync();
    const int total4 = p.total >> 2;
    const int per4 = (total4 + C - 1) / C;
    const int lo4 = min(total4, c * per4), hi4 = min(total4, lo4 + per4);
    float sq = 0.f;
    // every thread keeps its elements' summed gradients in registers across the second barrier
    constexpr int MAX_OWN = 8;            // float4s per thread: per4 <= THREADS * MAX_OWN (checked on the host)
    float4 own[MAX_OWN];
#pragma unroll
    for (int u = 0; u < MAX_OWN; u++) {
        const int i = lo4 + tid + u * THREADS;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < hi4) {
            for (int r = 0; r < C; r++) {
                const float4 q = reinterpret_cast<const float4*>(cluster.map_shared_rank(grad, r))[i];
                sum.x += q.x; sum.y += q.y; sum.z += q.z; sum.w += q.w;
            }
            sq += sum.x * sum.x; sq += sum.y * sum.y; sq += sum.z * sum.z; sq += sum.w * sum.w;
        }
        own[u] = sum;
    }
    const float sq_cta = block_sum(sq, red);
    if (tid == 0) red[33] = sq_cta;
    cluster.sync();
    float total_sq = 0.f, loss_total = 0.f;
    for (int r = 0; r < C; r++) {
        const float* rr = cluster.map_shared_rank(red, r);
        loss_total += rr[32];
        total_sq += rr[33];
    }
    float coef = 1.f;
    if (a.max_norm > 0.f) {
        const float norm = sqrtf(total_sq);
        coef = fminf(fmaxf(a.max_norm / (norm + a.clip_eps), 0.f), 1.f);
    }
    if (c == 0 && tid == 0 && a.loss_out) *a.loss_out = loss_total;

    // ---- 4. Adam on this CTA's slice ------------------------------------------------------------
    float t = a.adv[0], ibc1 = a.adv[1], ibc2 = a.adv[2];
    if (a.advance) {
        t += 1.f;
        ibc1 = 1.f / (1.f - powf(a.b1, t));
        ibc2 = 1.f / (1.f - powf(a.b2, t));
    }
    const float omb1 = 1.f - a.b1, omb2 = 1.f - a.b2;
#pragma unroll
    for (int u = 0; u < MAX_OWN; u++) {
        const int i = lo4 + tid + u * THREADS;
        if (i >= hi4) continue;
        float4 gg = own[u];
        if (a.max_norm > 0.f) { gg.x *= coef; gg.y *= coef; gg.z *= coef; gg.w *= coef; }
        float4 pp = reinterpret_cast<const float4*>(a.params)[i];
        float4 mm = reinterpret_cast<const float4*>(a.m)[i];
        float4 vv = reinterpret_cast<const float4*>(a.v)[i];
        ew::adam_one(pp.x, gg.x, mm.x, vv.x, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        ew::adam_one(pp.y, gg.y, mm.y, vv.y, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        ew::adam_one(pp.z, gg.z, mm.z, vv.z, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        ew::adam_one(pp.w, gg.w, mm.w, vv.w, a.b1, omb1, a.b2, omb2, a.lr, a.eps, ibc1, ibc2, 0.f, 1.f);
        reinterpret_cast<float4*>(a.params)[i] = pp;
        reinterpret_cast<float4*>(a.m)[i] = mm;
        reinterpret_cast<float4*>(a.v)[i] = vv;
        if (a.grads_out) reinterpret_cast<float4*>(a.grads_out)[i] = gg;
    }
    // Nobody leaves while another CTA may still read its shared memory; the step counter is
    // written after every CTA has read it.
    cluster.sync();
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
    // Cluster size: about 16 rows per CTA up to the largest cluster, then more rows per CTA.  The
    // choice depends on the batch only, so the summation order does too.
    int C = 1;
    while (C < g_max_cluster && batch > 16 * C) C *= 2;
    int rows = (batch + C - 1) / C;
    Plan plan = make_plan(*net, rows);
    if (static_cast<size_t>(plan.floats) * sizeof(float) > MAX_SMEM_BYTES) return TT_ERR_UNSUPPORTED;
    const int per4 = ((plan.total >> 2) + C - 1) / C;
    if (per4 > THREADS * 8) return TT_ERR_UNSUPPORTED;
    Args a;
    a.plan = plan;
    a.params = params; a.m = m; a.v = v; a.adv = adv; a.grads_out = grads_out;
    a.x = x; a.target = target; a.loss_out = loss_out; a.status = status;
    a.batch = batch;
    a.lr = lr; a.b1 = b1; a.b2 = b2; a.eps = eps; a.max_norm = max_norm; a.clip_eps = clip_eps;
    a.advance = advance;
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
