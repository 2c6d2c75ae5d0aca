// Any-stride, any-alignment FP32 GEMM (plain loads, no TMA): the total fallback that
// keeps the LaunchMatMul / LaunchMatMulBatched contract defined for every stride
// combination (odd leading dimensions, unaligned sub-views, "TT" strides, tiny
// shapes).  64x64x16 tiles, 256 threads, 4x4 accumulators per thread, ascending-k
// summation with one accumulator per output (bit-stable).
//
// Small outputs with a long K (a handful of tiles: the latency-bound shapes of small networks)
// are cut along K.  Two forms of the same sum, split by split in ascending k:
//   workspace form  partial tiles go to the handle workspace, generic_reduce_kernel adds them;
//   cluster form    the CTAs that share an output tile are one thread-block cluster (2, 4, 8 or
//                   16 CTAs); each leaves its partial tile in its own shared memory and, after a
//                   cluster barrier, adds 64 / splits rows of the tile over all CTAs of the
//                   cluster through distributed shared memory and stores them with the
//                   epilogue: one launch, no workspace.
#pragma once
#include <cooperative_groups.h>

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
    // split-K: work item w = tile * splits + split covers k in [split*kspan, +kspan); with
    // splits > 1 the raw tile goes to `partial` ([tile][split][BM][BN]) and
    // generic_reduce_kernel adds the splits in order and runs the epilogue.
    int splits, kspan;
    float* partial;
    int c_vec_ok;
};

__device__ __forceinline__ float act_apply(float v, int act)
{
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return tanhf(v);
    return v;
}

template <bool CLUSTER>
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
        const long long unit = w / p.splits;
        const int split = static_cast<int>(w - unit * p.splits);
        const int k_begin = split * p.kspan;
        const int k_end = min(p.shape.K, k_begin + p.kspan);
        const int bidx = static_cast<int>(unit / tiles_per_mat);
        const int t = static_cast<int>(unit - static_cast<long long>(bidx) * tiles_per_mat);
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
        const float* A0 = p.a + a_off;
        const float* B0 = p.b + b_off;
        const int m0 = tm * BM, n0 = tn * BN;

        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

        // Entries of a reduced batch axis are accumulated in ascending order.
        for (int red = 0; red < p.batch.red_count; red++) {
        const float* A = A0 + static_cast<long long>(red) * p.batch.red_a_stride;
        const float* B = B0 + static_cast<long long>(red) * p.batch.red_b_stride;
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
                ra[e] = (gm < p.shape.M && gk < k_end)
                            ? __ldg(A + static_cast<long long>(gm) * p.aMs + static_cast<long long>(gk) * p.aKs)
                            : 0.f;
            }
#pragma unroll
            for (int e = 0; e < (BN * BK) / THREADS; e++) {
                const int idx = tid + e * THREADS;
                const int kk = b_kmaj ? (idx % BK) : (idx / BN);
                const int nn = b_kmaj ? (idx / BK) : (idx % BN);
                const int gn = n0 + nn, gk = k0 + kk;
                rb[e] = (gn < p.shape.N && gk < k_end)
                            ? __ldg(B + static_cast<long long>(gn) * p.bNs + static_cast<long long>(gk) * p.bKs)
                            : 0.f;
            }
        };
        if (k_begin < k_end) fetch(k_begin);
        for (int k0 = k_begin; k0 < k_end; k0 += BK) {
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
            if (k0 + BK < k_end) fetch(k0 + BK);
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
        }  // reduced axis

        if constexpr (CLUSTER) {
            // grid == work: this loop body runs once per CTA, and the CTAs of a cluster are the
            // splits of one tile in ascending order (cluster rank == split)
            namespace cg = cooperative_groups;
            __shared__ __align__(16) float Cs[BM][BN + 4];
            cg::cluster_group cluster = cg::this_cluster();
#pragma unroll
            for (int i = 0; i < 4; i++)
                *reinterpret_cast<float4*>(&Cs[ty * 4 + i][tx * 4]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            cluster.sync();
            const int S = static_cast<int>(cluster.num_blocks()), rank = static_cast<int>(cluster.block_rank());
            const int rows_per = BM / S;
            float* C = p.c + static_cast<long long>(bidx) * p.shape.M * p.shape.N;
            for (int e = tid; e < rows_per * (BN / 4); e += THREADS) {
                const int lr = rank * rows_per + e / (BN / 4), lc = (e % (BN / 4)) * 4;
                float4 sum = *reinterpret_cast<const float4*>(&cluster.map_shared_rank(&Cs[0][0], 0)[lr * (BN + 4) + lc]);
                for (int r = 1; r < S; r++) {
                    const float4 q = *reinterpret_cast<const float4*>(&cluster.map_shared_rank(&Cs[0][0], r)[lr * (BN + 4) + lc]);
                    sum.x += q.x; sum.y += q.y; sum.z += q.z; sum.w += q.w;
                }
                const int gm = m0 + lr, gn0 = n0 + lc;
                if (gm >= p.shape.M) continue;
                float v[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (p.epi.bias && gn0 + j < p.shape.N) v[j] += __ldg(p.epi.bias + gn0 + j);
                    v[j] = act_apply(v[j], p.epi.act);
                }
                float* crow = C + static_cast<long long>(gm) * p.shape.N;
                if (p.c_vec_ok && gn0 + 3 < p.shape.N) {
                    *reinterpret_cast<float4*>(crow + gn0) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (gn0 + j < p.shape.N) crow[gn0 + j] = v[j];
                }
            }
            cluster.sync();     // nobody leaves while its partial tile may still be read
            continue;
        }
        if (p.splits > 1) {
            float* mine = p.partial + w * (BM * BN);
#pragma unroll
            for (int i = 0; i < 4; i++)
                *reinterpret_cast<float4*>(mine + (ty * 4 + i) * BN + tx * 4) =
                    make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            continue;
        }
        float* C = p.c + static_cast<long long>(bidx) * p.shape.M * p.shape.N;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int gm = m0 + ty * 4 + i;
            if (gm >= p.shape.M) continue;
            const int gn0 = n0 + tx * 4;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                v[j] = acc[i][j];
                if (p.epi.bias && gn0 + j < p.shape.N) v[j] += __ldg(p.epi.bias + gn0 + j);
                v[j] = act_apply(v[j], p.epi.act);
            }
            float* crow = C + static_cast<long long>(gm) * p.shape.N;
            if (p.c_vec_ok && gn0 + 3 < p.shape.N) {
                *reinterpret_cast<float4*>(crow + gn0) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (gn0 + j < p.shape.N) crow[gn0 + j] = v[j];
            }
        }
    }
}

// C = act(sum over splits (ascending) of the partial tiles + bias); one thread per 4 columns.
__global__ void __launch_bounds__(256)
generic_reduce_kernel(const float* __restrict__ partial, float* __restrict__ c, GemmShape shape,
                      Epilogue epi, int splits, int c_vec_ok)
{
    constexpr int PER_TILE = BM * BN / 4;
    const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long tiles = static_cast<long long>(shape.batch) * shape.tiles_m * shape.tiles_n;
    if (gid >= tiles * PER_TILE) return;
    const long long unit = gid / PER_TILE;
    const int e = static_cast<int>(gid - unit * PER_TILE);
    const int lr = e / (BN / 4), lc = (e % (BN / 4)) * 4;
    const int tiles_per_mat = shape.tiles_m * shape.tiles_n;
    const int bidx = static_cast<int>(unit / tiles_per_mat);
    const int t = static_cast<int>(unit - static_cast<long long>(bidx) * tiles_per_mat);
    const int r = (t / shape.tiles_n) * BM + lr, cidx = (t % shape.tiles_n) * BN + lc;
    if (r >= shape.M || cidx >= shape.N) return;
    const float* src = partial + unit * splits * (BM * BN) + lr * BN + lc;
    float4 sum = *reinterpret_cast<const float4*>(src);
    for (int sp = 1; sp < splits; sp++) {
        const float4 q = *reinterpret_cast<const float4*>(src + static_cast<long long>(sp) * (BM * BN));
        sum.x += q.x; sum.y += q.y; sum.z += q.z; sum.w += q.w;
    }
    float v[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (epi.bias && cidx + j < shape.N) v[j] += __ldg(epi.bias + cidx + j);
        v[j] = act_apply(v[j], epi.act);
    }
    float* crow = c + static_cast<long long>(bidx) * shape.M * shape.N + static_cast<long long>(r) * shape.N;
    if (c_vec_ok && cidx + 3 < shape.N) {
        *reinterpret_cast<float4*>(crow + cidx) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (cidx + j < shape.N) crow[cidx + j] = v[j];
    }
}

}  // namespace generic
}  // namespace tt
