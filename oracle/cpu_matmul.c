/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the matmul hot path.
 *
 * A plain-C restatement of the reference's managed/SIMD CPU matmul
 * (src/Tensotron/CpuKernels.cs:406-572) and of the few elementwise helpers the
 * Linear / MLP-step parity tests need.  Nothing in the product library links or
 * calls this file; it exists so the tests (and the CPU-baseline leg of the
 * benchmark) have an independent answer to compare the CUDA kernels with.
 *
 * Pinning: the reference is C# (.NET 8) and cannot be compiled where this is
 * built, so this restatement is pinned against the reference's own torch golden
 * fixtures (matmul.json / matmul_nd.json, re-derived into tests/golden/) at the
 * reference's fixture tolerance, not against a run of the C# build.
 *
 * Bits that depend on the host SIMD width: the reference's Vector<float>.Count is
 * 8 on AVX2 hosts, so `vw` defaults to 8 here and is a parameter.  The lane order
 * of the horizontal sum (Vector.Dot(v, One)) is internal to the .NET BCL and is
 * NOT pinned by the reference; the order used here is the one `vdpps` + a
 * 128-bit fold gives: ((l0+l1)+(l2+l3)) + ((l4+l5)+(l6+l7)).
 *
 * Build with -O2 -ffp-contract=off: RyuJIT does not contract a*b+c into an FMA.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define VW_MAX 16

/* ---- knobs: CpuKernels.cs:416-418 ---------------------------------------- */
static int g_threads = 1;                 /* CpuKernels.MatMulThreads          */
static long long g_min_flops = 1000000;   /* CpuKernels.MatMulParallelMinFlops */
static int g_vw = 8;                      /* Vector<float>.Count               */

void oracle_set_threads(int t) { g_threads = t < 1 ? 1 : t; }
int oracle_get_threads(void) { return g_threads; }
void oracle_set_min_flops(long long f) { g_min_flops = f; }
void oracle_set_vector_width(int vw) { if (vw >= 1 && vw <= VW_MAX) g_vw = vw; }

static float hsum(const float *v, int vw)
{
    /* pairwise within groups of 4, then fold groups left to right */
    if (vw % 4 != 0) {
        float s = 0.f;
        for (int i = 0; i < vw; i++) s += v[i];
        return s;
    }
    float s = (v[0] + v[1]) + (v[2] + v[3]);
    for (int g = 4; g < vw; g += 4) s += (v[g] + v[g + 1]) + (v[g + 2] + v[g + 3]);
    return s;
}

/* CpuKernels.cs:477-507 -- MatMul2DDot: both operands contiguous along K. */
static void matmul_dot(const float *a, const float *b, float *c, int N, int K,
                       int aMs, int bNs, int mStart, int mEnd)
{
    const int vw = g_vw, step = vw * 4;
    for (int m = mStart; m < mEnd; m++) {
        const float *ar = a + (long long)m * aMs;
        float *cr = c + (long long)m * N;
        for (int n = 0; n < N; n++) {
            const float *br = b + (long long)n * bNs;
            float a0[VW_MAX] = {0}, a1[VW_MAX] = {0}, a2[VW_MAX] = {0}, a3[VW_MAX] = {0};
            int k = 0;
            for (; k <= K - step; k += step) {
                for (int l = 0; l < vw; l++) a0[l] += ar[k + l] * br[k + l];
                for (int l = 0; l < vw; l++) a1[l] += ar[k + vw + l] * br[k + vw + l];
                for (int l = 0; l < vw; l++) a2[l] += ar[k + 2 * vw + l] * br[k + 2 * vw + l];
                for (int l = 0; l < vw; l++) a3[l] += ar[k + 3 * vw + l] * br[k + 3 * vw + l];
            }
            float vacc[VW_MAX];
            for (int l = 0; l < vw; l++) vacc[l] = (a0[l] + a1[l]) + (a2[l] + a3[l]);
            for (; k <= K - vw; k += vw)
                for (int l = 0; l < vw; l++) vacc[l] += ar[k + l] * br[k + l];
            float acc = hsum(vacc, vw);
            for (; k < K; k++) acc += ar[k] * br[k];
            cr[n] = acc;
        }
    }
}

/* CpuKernels.cs:513-540 -- MatMul2DAxpy: B contiguous along N (NN and TN). */
static void matmul_axpy(const float *a, const float *b, float *c, int N, int K,
                        int aMs, int aKs, int bKs, int mStart, int mEnd)
{
    memset(c + (long long)mStart * N, 0, sizeof(float) * (size_t)(mEnd - mStart) * (size_t)N);
    for (int m = mStart; m < mEnd; m++) {
        const float *ar = a + (long long)m * aMs;
        float *cr = c + (long long)m * N;
        for (int k = 0; k < K; k++) {
            /* no skip on av == 0: 0*NaN must stay NaN (CpuKernels.cs:525-526) */
            const float av = ar[(long long)k * aKs];
            const float *br = b + (long long)k * bKs;
            for (int n = 0; n < N; n++) cr[n] = cr[n] + av * br[n];
        }
    }
}

/* CpuKernels.cs:437-455 -- MatMul2DRange: path choice + the scalar fallback. */
static void matmul_range(const float *a, const float *b, float *c, int N, int K,
                         int aMs, int aKs, int bKs, int bNs, int mStart, int mEnd)
{
    if (aKs == 1 && bKs == 1) { matmul_dot(a, b, c, N, K, aMs, bNs, mStart, mEnd); return; }
    if (bNs == 1) { matmul_axpy(a, b, c, N, K, aMs, aKs, bKs, mStart, mEnd); return; }
    for (int m = mStart; m < mEnd; m++) {
        const long long aBase = (long long)m * aMs, cBase = (long long)m * N;
        for (int n = 0; n < N; n++) {
            const long long bBase = (long long)n * bNs;
            float acc = 0.f;
            for (int k = 0; k < K; k++)
                acc += a[aBase + (long long)k * aKs] * b[bBase + (long long)k * bKs];
            c[cBase + n] = acc;
        }
    }
}

typedef struct {
    const float *a, *b; float *c;
    int N, K, aMs, aKs, bKs, bNs, s, e;
} row_job;

static void *row_worker(void *p)
{
    row_job *j = (row_job *)p;
    matmul_range(j->a, j->b, j->c, j->N, j->K, j->aMs, j->aKs, j->bKs, j->bNs, j->s, j->e);
    return NULL;
}

/* CpuKernels.cs:420-432 (gate) and :461-472 (ParallelRows: contiguous row blocks
 * of ceil(M/chunks), one worker per block).  Rows are disjoint and each keeps its
 * K order, so the threaded result is bit-identical to the serial one. */
void oracle_matmul2d(const float *a, const float *b, float *c, int M, int N, int K,
                     int aMs, int aKs, int bKs, int bNs)
{
    const int threads = g_threads;
    if (threads > 1 && M >= 2 && 2LL * M * N * K >= g_min_flops) {
        const int chunks = threads < M ? threads : M;
        const int per = (M + chunks - 1) / chunks;
        pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)chunks);
        row_job *jobs = (row_job *)malloc(sizeof(row_job) * (size_t)chunks);
        int started = 0;
        for (int ci = 0; ci < chunks; ci++) {
            const int s = ci * per;
            if (s >= M) break;
            const int e = s + per < M ? s + per : M;
            row_job j = {a, b, c, N, K, aMs, aKs, bKs, bNs, s, e};
            jobs[started] = j;
            pthread_create(&tid[started], NULL, row_worker, &jobs[started]);
            started++;
        }
        for (int i = 0; i < started; i++) pthread_join(tid[i], NULL);
        free(tid); free(jobs);
        return;
    }
    matmul_range(a, b, c, N, K, aMs, aKs, bKs, bNs, 0, M);
}

/* CpuKernels.cs:542-572 -- MatMulBatched: scalar, single-threaded, output-index
 * order; the batch index is decoded last-axis-fastest over batchDims. */
void oracle_matmul_batched(const float *a, const float *b, float *c, int batchCount,
                           int M, int N, int K, int aMs, int aKs, int bKs, int bNs,
                           int batchRank, const int *batchDims,
                           const int *aBatchStrides, const int *bBatchStrides)
{
    const long long mn = (long long)M * N;
    for (long long idx = 0; idx < (long long)batchCount * mn; idx++) {
        const int bb = (int)(idx / mn);
        const long long rem = idx % mn;
        const int m = (int)(rem / N), n = (int)(rem % N);
        long long aOff = 0, bOff = 0; int br = bb;
        for (int ax = batchRank - 1; ax >= 0; ax--) {
            const int d = batchDims[ax];
            const int bi = br % d;
            br /= d;
            aOff += (long long)bi * aBatchStrides[ax];
            bOff += (long long)bi * bBatchStrides[ax];
        }
        float acc = 0.f;
        const long long aBase = aOff + (long long)m * aMs, bBase = bOff + (long long)n * bNs;
        for (int k = 0; k < K; k++)
            acc += a[aBase + (long long)k * aKs] * b[bBase + (long long)k * bKs];
        c[idx] = acc;
    }
}

/* Same batched contract, but each matrix goes through oracle_matmul2d (threaded).
 * NOT a reference function: a faster checker for full-size batched parity cases,
 * cross-checked against oracle_matmul_batched on small cases by the tests. */
void oracle_matmul_batched_fast(const float *a, const float *b, float *c, int batchCount,
                                int M, int N, int K, int aMs, int aKs, int bKs, int bNs,
                                int batchRank, const int *batchDims,
                                const int *aBatchStrides, const int *bBatchStrides)
{
    for (int bb = 0; bb < batchCount; bb++) {
        long long aOff = 0, bOff = 0; int br = bb;
        for (int ax = batchRank - 1; ax >= 0; ax--) {
            const int d = batchDims[ax];
            const int bi = br % d;
            br /= d;
            aOff += (long long)bi * aBatchStrides[ax];
            bOff += (long long)bi * bBatchStrides[ax];
        }
        oracle_matmul2d(a + aOff, b + bOff, c + (long long)bb * M * N, M, N, K, aMs, aKs, bKs, bNs);
    }
}

/* float64 accumulation of the same contract: the error-budget yardstick (not a restatement
 * of reference code).  Rows are independent; with B contiguous along N the k loop is outermost
 * per row so that B is walked along its rows (the row-slab checks of 8192- and 16384-wide
 * products would otherwise take a cache miss per term).  Row-parallel like oracle_matmul2d. */
typedef struct {
    const float *a, *b; double *c;
    int N, K, aMs, aKs, bKs, bNs, s, e;
} row_job64;

static void *row_worker64(void *p)
{
    row_job64 *j = (row_job64 *)p;
    const int N = j->N, K = j->K;
    for (int m = j->s; m < j->e; m++) {
        double *cr = j->c + (long long)m * N;
        if (j->bNs == 1) {
            for (int n = 0; n < N; n++) cr[n] = 0.0;
            for (int k = 0; k < K; k++) {
                const double av = (double)j->a[(long long)m * j->aMs + (long long)k * j->aKs];
                const float *br = j->b + (long long)k * j->bKs;
                for (int n = 0; n < N; n++) cr[n] += av * (double)br[n];
            }
        } else {
            for (int n = 0; n < N; n++) {
                double acc = 0.0;
                for (int k = 0; k < K; k++)
                    acc += (double)j->a[(long long)m * j->aMs + (long long)k * j->aKs] *
                           (double)j->b[(long long)n * j->bNs + (long long)k * j->bKs];
                cr[n] = acc;
            }
        }
    }
    return NULL;
}

void oracle_matmul2d_f64(const float *a, const float *b, double *c, int M, int N, int K,
                         int aMs, int aKs, int bKs, int bNs)
{
    int chunks = g_threads < M ? g_threads : M;
    if (chunks < 1 || 2LL * M * N * K < g_min_flops) chunks = 1;
    const int per = (M + chunks - 1) / chunks;
    pthread_t tid[256];
    row_job64 jobs[256];
    if (chunks > 256) chunks = 256;
    int started = 0;
    for (int ci = 0; ci < chunks; ci++) {
        const int s = ci * per;
        if (s >= M) break;
        const int e = (ci == chunks - 1 || s + per > M) ? M : s + per;
        row_job64 j = {a, b, c, N, K, aMs, aKs, bKs, bNs, s, e};
        jobs[started] = j;
        if (chunks == 1) { row_worker64(&jobs[0]); return; }
        pthread_create(&tid[started], NULL, row_worker64, &jobs[started]);
        started++;
    }
    for (int i = 0; i < started; i++) pthread_join(tid[i], NULL);
}

/* ---- Linear support ops -------------------------------------------------- */

/* y[m,n] = x[m,n] + bias[n]: the broadcast Add after the Linear GEMM
 * (src/Tensotron/Module.cs:100-105, CpuKernels.cs:24-44 with bStride = [0,1]). */
void oracle_bias_add(const float *x, const float *bias, float *y, int M, int N)
{
    for (long long i = 0; i < (long long)M * N; i++) y[i] = x[i] + bias[i % N];
}

/* act: 0 none, 1 ReLU, 2 Tanh (src/Tensotron/Ops.Unary.cs:89-105). */
void oracle_act_fwd(const float *x, float *y, long long n, int act)
{
    for (long long i = 0; i < n; i++) {
        const float v = x[i];
        y[i] = act == 1 ? (v > 0.f ? v : 0.f) : act == 2 ? tanhf(v) : v;
    }
}

/* gx = Backward(x, y, gy): ReLU -> x>0 ? gy : 0 ; Tanh -> gy*(1-y*y). */
void oracle_act_bwd(const float *x, const float *y, const float *gy, float *gx, long long n, int act)
{
    for (long long i = 0; i < n; i++)
        gx[i] = act == 1 ? (x[i] > 0.f ? gy[i] : 0.f)
              : act == 2 ? gy[i] * (1.f - y[i] * y[i]) : gy[i];
}

/* Bias gradient: sum g over the batch axis, rows visited in order
 * (ReduceGradToShape -> ReduceSum, TensorOps.cs:76-100, CpuKernels.cs:100-135). */
void oracle_colsum(const float *g, float *out, int M, int N)
{
    for (int n = 0; n < N; n++) {
        float acc = 0.f;
        for (int m = 0; m < M; m++) acc += g[(long long)m * N + n];
        out[n] = acc;
    }
}

/* CpuKernels.AddInto (CpuKernels.cs:88-96). */
void oracle_add_into(float *target, const float *source, long long n)
{
    for (long long i = 0; i < n; i++) target[i] += source[i];
}

/* ---- MLP-step support ops ------------------------------------------------- */

/* CrossEntropy(mean) = NllLoss(LogSoftmax(logits)) (TensorOps.Losses.cs:97-108,
 * TensorOps.Reduce.cs:122-141): lse = log(sum exp(x - max)) + max; loss =
 * mean(-(x[t] - lse)).  dlogits = (softmax - onehot) * scale, the closed form of
 * the reference's autograd chain.  `scale` is 1/rows for the mean reduction (a
 * data-parallel shard passes 1/global_rows).  Returns sum of per-row losses * scale. */
float oracle_cross_entropy(const float *logits, const int *labels, float *dlogits,
                           int rows, int classes, float scale)
{
    double total = 0.0;
    for (int r = 0; r < rows; r++) {
        const float *x = logits + (long long)r * classes;
        float mx = x[0];
        for (int j = 1; j < classes; j++) if (x[j] > mx) mx = x[j];
        float s = 0.f;
        for (int j = 0; j < classes; j++) s += expf(x[j] - mx);
        const float lse = logf(s) + mx;
        total += (double)(-(x[labels[r]] - lse));
        if (dlogits)
            for (int j = 0; j < classes; j++) {
                const float p = expf(x[j] - lse);
                dlogits[(long long)r * classes + j] = (p - (j == labels[r] ? 1.f : 0.f)) * scale;
            }
    }
    return (float)(total * (double)scale);
}

/* Adam (Kernels.cs:126-157 AdvanceAdam + AdamStep; CpuKernels.cs:721-736).
 * adv = [t, 1/(1-b1^t), 1/(1-b2^t)] advances first, then the fused update. */
void oracle_adam_step(float *p, const float *g, float *m, float *v, float *adv, long long n,
                      float b1, float b2, float lr, float eps, float coupledWd, float decoupledFactor,
                      int advance)
{
    if (advance) {
        const float t = adv[0] + 1.f;
        adv[0] = t;
        adv[1] = 1.f / (1.f - powf(b1, t));
        adv[2] = 1.f / (1.f - powf(b2, t));
    }
    const float invBc1 = adv[1], invBc2 = adv[2];
    const float omb1 = 1.f - b1, omb2 = 1.f - b2;
    for (long long i = 0; i < n; i++) {
        const float pi = p[i];
        const float gi = g[i] + coupledWd * pi;
        const float mi = b1 * m[i] + omb1 * gi;
        const float vi = b2 * v[i] + omb2 * gi * gi;
        m[i] = mi; v[i] = vi;
        const float step = (mi * invBc1) / (sqrtf(vi * invBc2) + eps);
        p[i] = pi * decoupledFactor - lr * step;
    }
}
