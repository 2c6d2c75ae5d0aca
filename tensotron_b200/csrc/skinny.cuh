// FP32 kernels for products with one tiny dimension (<= 16): the 10-class output layer of
// an MLP, value heads, matrix-vector products.  A 128-wide tile would waste > 90 % of its
// FMAs on them; they are HBM-bound streams of the one large operand instead, so each kernel
// reads that operand exactly once with 128-bit loads and keeps the small one in registers or
// L1.  One accumulator per output, a k order that depends on the output row only, fixed
// reduction trees: results are bit-stable run to run.
//
//   skinny_n_kernel  C (M x N<=16) = A (M x K, K-major) . B (N x K, K-major)^T     reads A once
//   skinny_m_kernel  C (M<=16 x N) = A (K x M)^T        . B (K x N, N-major)      reads B once
//                    (K is cut into ranges across CTAs; partials are added in range order)
//   skinny_k_kernel  C (M x N)     = A (M x K<=16)      . B (K x N, N-major)      writes C once
#pragma once
#include "gemm_common.h"
#include "ptx.cuh"

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

// ---- small N, tall M: TMA-fed stream ----------------------------------------------------------
// The K-cut form above keeps a few kilobytes per warp in flight and sits at a quarter of the HBM
// bandwidth when M is large.  Here the bytes in flight are explicit: a persistent CTA per SM, one
// producer thread that keeps a ring of 4 stages filled by TMA (a stage = 56 rows x 128 k of A, 28 KB,
// plus the matching 128 k of all rows of B), and 7 consumer warps that read both from shared memory
// (256 threads, so the consumers may use 255 registers).  A unit of work is 56 consecutive rows over
// the whole K; warp w owns rows 8w .. 8w+7 of the unit, lane l the four k at 4l of every 128-k chunk, so a lane holds
// 8 x N partial sums over the chunks (visited in an order rotated by the unit index: rows are a
// power-of-two number of bytes apart, and all CTAs walking them from the same offset would keep
// hitting the same memory channels) and a fixed xor-shuffle tree adds the lanes at the end of the
// unit.  One accumulator per lane and output, an order that depends on the row only: bit-stable.
namespace stream {
constexpr int CONSUMER_WARPS = 7, RB = 8 * CONSUMER_WARPS, KC = 128, STAGES = 4, THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int KJ = KC / 128;      // float4s per lane, row and chunk
constexpr int A_BYTES = RB * KC * 4;
template <int NT> struct Cfg {
    static constexpr int B_BYTES = NT * KC * 4;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int OFF_BAR = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 256 + 128;     // barriers + abort word, alignment slack
};
}  // namespace stream

template <int NT>
__global__ void __launch_bounds__(stream::THREADS, 1)
skinny_n_stream_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       float* __restrict__ c, int M, int N, int K, Epilogue epi, unsigned int* status)
{
    using namespace stream;
    using C = Cfg<NT>;
    extern __shared__ uint8_t skinny_smem_raw[];
    uint8_t* smem = skinny_smem_raw + ((128u - (smem_u32(skinny_smem_raw) & 127u)) & 127u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty_bar = full_bar + STAGES;
    volatile uint32_t* cta_abort = reinterpret_cast<volatile uint32_t*>(empty_bar + STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_chunks = (K + KC - 1) / KC;
    const int units = (M + RB - 1) / RB;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], CONSUMER_WARPS);
        }
        *cta_abort = 0u;
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == CONSUMER_WARPS) {
        // ------------------------------- producer -------------------------------
        if (lane != 0) return;
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        uint32_t ps = 0, use = 0;
        bool ok = true;
        for (int unit = blockIdx.x; ok && unit < units; unit += gridDim.x) {
            const int rot = unit % k_chunks;
            for (int i = 0; i < k_chunks; i++) {
                int kc = i + rot;
                if (kc >= k_chunks) kc -= k_chunks;
                if (use > 0 && !mbar_wait_bounded(&empty_bar[ps], (use - 1) & 1u, cta_abort, status, DEV_WAIT_EMPTY)) {
                    ok = false;
                    break;
                }
                uint8_t* sa = smem + ps * C::STAGE_BYTES;
                mbar_arrive_expect_tx(&full_bar[ps], C::STAGE_BYTES);
                tma_load_5d(sa, &map_a, &full_bar[ps], kc * KC, unit * RB, 0, 0, 0);
                tma_load_5d(sa + A_BYTES, &map_b, &full_bar[ps], kc * KC, 0, 0, 0, 0);
                if (++ps == STAGES) { ps = 0; use++; }
            }
        }
        if (!ok) {
            // a wait gave up: wait (with a limit) for the loads this thread issued before leaving
            uint32_t s = ps, u = use;
            for (int i = 0; i < STAGES; i++) {
                if (s == 0) {
                    if (u == 0) break;
                    s = STAGES;
                    u--;
                }
                s--;
                mbar_wait_drain(&full_bar[s], u & 1u);
            }
        }
        return;
    }
    // -------------------------------- consumers --------------------------------
    // Two partial sums per output (the even and the odd pairs of a lane's four k per chunk), so the
    // four multiply-adds of a chunk are two packed two-wide FMAs: the kernel is bound by instruction
    // issue at 10 columns, not by the memory system.  The two are added when the unit is finished.
    uint32_t stage = 0, phase = 0;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        // (more than 8 columns would need over 200 registers for the pairs: those groups keep one sum per output)
        constexpr bool PACK = NT <= 8;
        float2 acc[8][NT];
#pragma unroll
        for (int r = 0; r < 8; r++)
#pragma unroll
            for (int n = 0; n < NT; n++) acc[r][n] = make_float2(0.f, 0.f);
        for (int i = 0; i < k_chunks; i++) {
            if (!mbar_wait_bounded(&full_bar[stage], phase, cta_abort, status, DEV_WAIT_FULL)) return;
            const uint32_t sa0 = smem_u32(smem + stage * C::STAGE_BYTES) + lane * 16;
            // columns in groups of at most 8, so that a group's B fragments and the sums it updates
            // stay in registers (the A fragments are read again per group: shared-memory bandwidth
            // is not what bounds this kernel)
#pragma unroll
            for (int kj = 0; kj < KJ; kj++) {
            const uint32_t sa = sa0 + kj * 512;
            const uint32_t sb = sa + A_BYTES;
#pragma unroll
            for (int n0 = 0; n0 < NT; n0 += 8) {
                constexpr int NG = NT < 8 ? NT : 8;
                float4 bv[NG];
#pragma unroll
                for (int j = 0; j < NG; j++)
                    if (n0 + j < NT) bv[j] = lds128(sb + (n0 + j) * (KC * 4));   // rows >= N of the stage are zero (TMA fill)
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    const int row = 8 * warp + r;
                    const float4 av = lds128(sa + row * (KC * 4));
#pragma unroll
                    for (int j = 0; j < NG; j++) {
                        if (n0 + j < NT) {           // no test against N: straight-line code, zeros for the columns beyond it
                            if constexpr (PACK) {
                                float2 t = acc[r][n0 + j];
                                t = __ffma2_rn(make_float2(av.x, av.y), make_float2(bv[j].x, bv[j].y), t);
                                t = __ffma2_rn(make_float2(av.z, av.w), make_float2(bv[j].z, bv[j].w), t);
                                acc[r][n0 + j] = t;
                            } else {
                                float t = acc[r][n0 + j].x;      // (.y stays zero and is never touched: no register)
                                t = fmaf(av.x, bv[j].x, t);
                                t = fmaf(av.y, bv[j].y, t);
                                t = fmaf(av.z, bv[j].z, t);
                                t = fmaf(av.w, bv[j].w, t);
                                acc[r][n0 + j].x = t;
                            }
                        }
                    }
                }
            }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const int m = unit * RB + 8 * warp + r;
#pragma unroll
            for (int n = 0; n < NT; n++) {
                if (n < N) {
                    float t = PACK ? acc[r][n].x + acc[r][n].y : acc[r][n].x;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                    if (lane == 0 && m < M) {
                        if (epi.bias) t += __ldg(epi.bias + n);
                        c[static_cast<long long>(m) * N + n] = act_apply(t, epi.act);
                    }
                }
            }
        }
    }
}

// ---- small K ---------------------------------------------------------------------------------
// C (M x N) = A (M x K<=16, any strides) . B (K x N, N-major): bound by the write of C.  A CTA owns
// 64 rows x 1024 columns: a thread keeps the K float4 of B for its 4 columns in registers, the A tile
// (64 x K, padded to 16 per row) sits in shared memory and is read as broadcasts, and every
// instruction of a warp stores 512 contiguous bytes of one row.  One accumulator per output, k
// ascending.
constexpr int SK_ROWS = 64, SK_COLS = 1024;
template <int KT4>   // K <= 4 * KT4
__global__ void __launch_bounds__(256)
skinny_k_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                int M, int N, int K, int aMs, int aKs, int bKs, Epilogue epi)
{
    __shared__ __align__(16) float as_[SK_ROWS][4 * KT4];
    const int m0 = blockIdx.y * SK_ROWS;
    const int n = blockIdx.x * SK_COLS + threadIdx.x * 4;
    for (int i = threadIdx.x; i < SK_ROWS * 4 * KT4; i += 256) {
        const int r = i / (4 * KT4), k = i - r * (4 * KT4);
        as_[r][k] = (m0 + r < M && k < K) ? __ldg(a + static_cast<long long>(m0 + r) * aMs + static_cast<long long>(k) * aKs) : 0.f;
    }
    float4 bv[4 * KT4];
#pragma unroll
    for (int k = 0; k < 4 * KT4; k++)
        bv[k] = (k < K && n < N) ? __ldg(reinterpret_cast<const float4*>(b + static_cast<long long>(k) * bKs + n))
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (epi.bias && n < N) bias4 = __ldg(reinterpret_cast<const float4*>(epi.bias + n));
    __syncthreads();
    if (n >= N) return;
    const int rows = min(SK_ROWS, M - m0);
#pragma unroll 2
    for (int r = 0; r < rows; r++) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k4 = 0; k4 < KT4; k4++) {
            const float4 av = *reinterpret_cast<const float4*>(&as_[r][4 * k4]);
            const float a4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 bb = bv[4 * k4 + q];      // zeros beyond K: nothing to test
                acc.x = fmaf(a4[q], bb.x, acc.x);
                acc.y = fmaf(a4[q], bb.y, acc.y);
                acc.z = fmaf(a4[q], bb.z, acc.z);
                acc.w = fmaf(a4[q], bb.w, acc.w);
            }
        }
        acc.x = act_apply(acc.x + bias4.x, epi.act); acc.y = act_apply(acc.y + bias4.y, epi.act);
        acc.z = act_apply(acc.z + bias4.z, epi.act); acc.w = act_apply(acc.w + bias4.w, epi.act);
        *reinterpret_cast<float4*>(c + static_cast<long long>(m0 + r) * N + n) = acc;
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

// ---- small M, TMA-fed ---------------------------------------------------------------------------
// The same product with the bytes in flight made explicit.  CTA (x, y) owns 256 columns and the k
// range y.  A producer thread keeps a ring of 4 stages filled by TMA (a stage = 32 k x 256 columns of
// B, 32 KB); the CTA's slice of the small operand (k range x M, at most 64 KB) is copied into shared
// memory once at the start, M rounded up to 4 per k so a thread fetches it as float4 broadcasts.  The 256
// consumer threads are the 64 column groups x 4 k lanes of skinny_m_kernel and walk k in the same
// order, so for the same k ranges the sums are the same sums.
namespace mstream {
constexpr int KT = 32, NW = 256, STAGES = 4, THREADS = 288, A_FLOATS = 16384;
constexpr int STAGE_BYTES = KT * NW * 4;
constexpr int OFF_A = STAGES * STAGE_BYTES;
constexpr int OFF_RED = OFF_A + A_FLOATS * 4;
constexpr int OFF_BAR = OFF_RED + 4 * 64 * 16;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 128;
}  // namespace mstream

// M <= MT; the k range of a CTA is at most A_FLOATS / MT (a multiple of KT).
template <int MT>
__global__ void __launch_bounds__(mstream::THREADS, 1)
skinny_m_stream_kernel(const __grid_constant__ CUtensorMap map_b, const float* __restrict__ a, float* __restrict__ out,
                       int M, int N, int K, int aMs, int aKs, int kspan, Epilogue epi, int direct, unsigned int* status)
{
    using namespace mstream;
    extern __shared__ uint8_t skinny_smem_raw[];
    uint8_t* smem = skinny_smem_raw + ((128u - (smem_u32(skinny_smem_raw) & 127u)) & 127u);
    float* as_ = reinterpret_cast<float*>(smem + OFF_A);
    float4* red = reinterpret_cast<float4*>(smem + OFF_RED);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* empty_bar = full_bar + STAGES;
    volatile uint32_t* cta_abort = reinterpret_cast<volatile uint32_t*>(empty_bar + STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * NW;
    const int k0 = blockIdx.y * kspan;
    const int k1 = min(K, k0 + kspan);
    const int tiles = (k1 - k0 + KT - 1) / KT;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 8);
        }
        *cta_abort = 0u;
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == 8) {
        // ------------------------------- producer -------------------------------
        if (lane != 0) return;
        prefetch_tensormap(&map_b);
        uint32_t ps = 0, use = 0;
        bool ok = true;
        for (int t = 0; t < tiles; t++) {
            if (use > 0 && !mbar_wait_bounded(&empty_bar[ps], (use - 1) & 1u, cta_abort, status, DEV_WAIT_EMPTY)) {
                ok = false;
                break;
            }
            mbar_arrive_expect_tx(&full_bar[ps], STAGE_BYTES);
            tma_load_5d(smem + ps * STAGE_BYTES, &map_b, &full_bar[ps], n0, k0 + t * KT, 0, 0, 0);
            if (++ps == STAGES) { ps = 0; use++; }
        }
        if (!ok) {
            uint32_t s = ps, u = use;
            for (int i = 0; i < STAGES; i++) {
                if (s == 0) {
                    if (u == 0) break;
                    s = STAGES;
                    u--;
                }
                s--;
                mbar_wait_drain(&full_bar[s], u & 1u);
            }
        }
        return;
    }
    // -------------------------------- consumers --------------------------------
    const int tid = threadIdx.x;          // 0 .. 255
    const int cl = tid & 63, kl = tid >> 6;
    // the small operand's slice: as_[k - k0][m], zero beyond K and for the rows between M and MT (the
    // main loop then needs no test against M: straight-line code)
    for (int i = tid; i < tiles * KT * MT; i += 256) {
        const int kk = i / MT, m = i - kk * MT;
        const int k = k0 + kk;
        as_[i] = (k < K && m < M) ? __ldg(a + static_cast<long long>(m) * aMs + static_cast<long long>(k) * aKs) : 0.f;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float4 acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = make_float4(0.f, 0.f, 0.f, 0.f);
    uint32_t stage = 0, phase = 0;
    const uint32_t as_u32 = smem_u32(as_);
    for (int t = 0; t < tiles; t++) {
        if (!mbar_wait_bounded(&full_bar[stage], phase, cta_abort, status, DEV_WAIT_FULL)) return;
        const uint32_t sb = smem_u32(smem + stage * STAGE_BYTES) + cl * 16;
#pragma unroll 2
        for (int i = 0; i < KT / 4; i++) {
            const int kk = kl + 4 * i;
            const float4 bv = lds128(sb + kk * (NW * 4));
            const uint32_t ap = as_u32 + ((t * KT + kk) * MT) * 4;
#pragma unroll
            for (int j = 0; j < MT / 4; j++) {
                {
                    const float4 av = lds128(ap + j * 16);
                    const float a4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int m = 4 * j + q;
                        {
                            // two packed two-wide FMAs (each lane an IEEE fused multiply-add: the bits
                            // of four scalar fmaf)
                            const float2 ap = make_float2(a4[q], a4[q]);
                            const float2 lo = __ffma2_rn(ap, make_float2(bv.x, bv.y), make_float2(acc[m].x, acc[m].y));
                            const float2 hi = __ffma2_rn(ap, make_float2(bv.z, bv.w), make_float2(acc[m].z, acc[m].w));
                            acc[m] = make_float4(lo.x, lo.y, hi.x, hi.y);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
    }
    const int n = n0 + cl * 4;
    float* dst = out + (direct ? 0ll : static_cast<long long>(blockIdx.y) * M * N);
#pragma unroll
    for (int m = 0; m < MT; m++) {
        if (m < M) {                       // uniform across the CTA
            red[kl * 64 + cl] = acc[m];
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (kl == 0 && n < N) {
                float4 s = red[cl];
#pragma unroll
                for (int l = 1; l < 4; l++) {
                    const float4 q = red[l * 64 + cl];
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
            asm volatile("bar.sync 1, 256;" ::: "memory");
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
