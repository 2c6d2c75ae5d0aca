// Strict-FP32 SGEMM for sm_100a: SIMT FFMA tiles fed by TMA.
//
// One persistent CTA per SM walks a grouped raster of 128x128 output tiles.  A
// dedicated producer warp streams 128x32 (A) and 32x128 (B) float tiles into a
// shared-memory ring with TMA; eight consumer warps (8x8 accumulators per thread)
// read them with 128-bit shared loads and issue FFMAs only.  Stages are handed over
// with mbarriers (full: TMA transaction bytes; empty: one arrival per consumer
// warp), so the main loop has no CTA-wide barrier and the ring keeps filling across
// tile boundaries while the previous tile's epilogue stores.
//
// Operand layouts.  Each operand is either contiguous along K ("K-major") or along
// its M/N axis ("MN-major"); TMA copies tiles in their native order:
//   K-major : smem [128 rows][32 k], 128-byte rows, hardware 128B swizzle.  A thread
//             reads float4 = 4 consecutive k of one row; the 16-byte chunk index is
//             XORed with (row & 7), and thread->row assignment is interleaved so the
//             rows one warp instruction touches all differ in (row & 7): conflict-free.
//   MN-major: smem [32 k][128 cols], no swizzle.  A thread reads float4 = 4 adjacent
//             rows/cols of one k.
// Summation order over K is fixed (ascending k, one accumulator per output), so the
// result does not depend on the grid size or on which SM ran a tile.
#pragma once
#include "gemm_common.h"
#include "ptx.cuh"

namespace tt {
namespace simt {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr int STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 4;  // 16 KiB
constexpr int B_TILE_BYTES = BN * BK * 4;  // 16 KiB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int CONSUMER_WARPS = 8;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int RASTER_GROUP = 8;

struct Params {
    GemmShape shape;
    BatchDesc batch;
    Epilogue epi;
    float* c;
    unsigned int* status;  // device status word (bounded waits)
    int c_vec_ok;          // C base 16-byte aligned and N % 4 == 0
};

__device__ __forceinline__ float apply_act(float v, int act)
{
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return tanhf(v);
    return v;
}

template <bool A_KMAJ, bool B_KMAJ>
__global__ void __launch_bounds__(THREADS, 1)
sgemm_simt_kernel(const __grid_constant__ CUtensorMap map_a,
                  const __grid_constant__ CUtensorMap map_b, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    // 128B-swizzled tiles need 1024-byte alignment.
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023u));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    volatile uint32_t* cta_abort = reinterpret_cast<volatile uint32_t*>(empty_bar + STAGES);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], CONSUMER_WARPS);
        }
        *cta_abort = 0u;
        fence_mbar_init();
    }
    __syncthreads();

    const int k_tiles = (p.shape.K + BK - 1) / BK;
    const int tiles_per_mat = p.shape.tiles_m * p.shape.tiles_n;

    if (warp == CONSUMER_WARPS) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            prefetch_tensormap(&map_a);
            prefetch_tensormap(&map_b);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (long long w = blockIdx.x; ok && w < p.shape.work; w += gridDim.x) {
                const int bidx = static_cast<int>(w / tiles_per_mat);
                const int t = static_cast<int>(w - static_cast<long long>(bidx) * tiles_per_mat);
                int tm, tn;
                raster_tile(t, p.shape.tiles_m, p.shape.tiles_n, RASTER_GROUP, tm, tn);
                int ca[3] = {0, 0, 0}, cb[3] = {0, 0, 0};
                int br = bidx;
                for (int ax = p.batch.rank - 1; ax >= 0; ax--) {
                    const int d = p.batch.dims[ax];
                    const int bi = br % d;
                    br /= d;
                    if (p.batch.a_slot[ax] >= 0) ca[p.batch.a_slot[ax]] += bi * p.batch.a_mult[ax];
                    if (p.batch.b_slot[ax] >= 0) cb[p.batch.b_slot[ax]] += bi * p.batch.b_mult[ax];
                }
                const int m0 = tm * BM, n0 = tn * BN;
                for (int kt = 0; kt < k_tiles; kt++) {
                    if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, cta_abort, p.status,
                                           DEV_WAIT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * STAGE_BYTES;
                    uint8_t* sb = sa + A_TILE_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
                    const int k0 = kt * BK;
                    if (A_KMAJ) tma_load_5d(sa, &map_a, &full_bar[stage], k0, m0, ca[0], ca[1], ca[2]);
                    else        tma_load_5d(sa, &map_a, &full_bar[stage], m0, k0, ca[0], ca[1], ca[2]);
                    if (B_KMAJ) tma_load_5d(sb, &map_b, &full_bar[stage], k0, n0, cb[0], cb[1], cb[2]);
                    else        tma_load_5d(sb, &map_b, &full_bar[stage], n0, k0, cb[0], cb[1], cb[2]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int wm = warp >> 1;  // 0..3 -> 32 rows each
    const int wn = warp & 1;   // 0..1 -> 64 cols each
    const int ty = lane >> 3;  // 0..3
    const int tx = lane & 7;   // 0..7

    // Per-thread byte offsets inside a stage (see the layout notes at the top).
    int off_a[4];  // K-major A: index q = low two bits of the (compile-time part of the) chunk
    int off_b[8];  // K-major B: index = k chunk
    int off_am = 0, off_bm = 0;
    if (A_KMAJ) {
#pragma unroll
        for (int q = 0; q < 4; q++) off_a[q] = (wm * 32 + ty) * 128 + ((q ^ ty) << 4);
    } else {
        off_am = (wm * 32 + ty * 4) * 4;
    }
    if (B_KMAJ) {
#pragma unroll
        for (int c = 0; c < 8; c++) off_b[c] = A_TILE_BYTES + (wn * 64 + tx) * 128 + ((c ^ tx) << 4);
    } else {
        off_bm = A_TILE_BYTES + (wn * 64 + tx * 4) * 4;
    }

    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (long long w = blockIdx.x; ok && w < p.shape.work; w += gridDim.x) {
        const int bidx = static_cast<int>(w / tiles_per_mat);
        const int t = static_cast<int>(w - static_cast<long long>(bidx) * tiles_per_mat);
        int tm, tn;
        raster_tile(t, p.shape.tiles_m, p.shape.tiles_n, RASTER_GROUP, tm, tn);

        float acc[8][8];
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

        for (int kt = 0; kt < k_tiles; kt++) {
            if (!mbar_wait_bounded(&full_bar[stage], phase, cta_abort, p.status, DEV_WAIT_FULL)) {
                ok = false;
                break;
            }
            const uint8_t* st = smem + stage * STAGE_BYTES;

#pragma unroll
            for (int g = 0; g < BK / 4; g++) {  // 8 groups of 4 k
                float4 av[8], bv[8];            // K-major: [row] = 4 consecutive k
                float4 am[4][2], bm[4][2];      // MN-major: [k][half] = 4 adjacent rows/cols
                if (A_KMAJ) {
#pragma unroll
                    for (int ib = 0; ib < 2; ib++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int cc = g ^ ((i & 1) << 2);  // compile-time part of the chunk
                            av[ib * 4 + i] = *reinterpret_cast<const float4*>(
                                st + off_a[cc & 3] + (ib * 16 + i * 4) * 128 + (cc & 4) * 16);
                        }
                } else {
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
#pragma unroll
                        for (int ib = 0; ib < 2; ib++)
                            am[kk][ib] = *reinterpret_cast<const float4*>(
                                st + off_am + (g * 4 + kk) * (BM * 4) + ib * 64);
                }
                if (B_KMAJ) {
#pragma unroll
                    for (int jb = 0; jb < 2; jb++)
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            bv[jb * 4 + j] = *reinterpret_cast<const float4*>(
                                st + off_b[g] + (jb * 32 + j * 8) * 128);
                } else {
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
#pragma unroll
                        for (int jb = 0; jb < 2; jb++)
                            bm[kk][jb] = *reinterpret_cast<const float4*>(
                                st + off_bm + (g * 4 + kk) * (BN * 4) + jb * 128);
                }
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
                    float a[8], b[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        if (A_KMAJ) {
                            const float4 v = av[i];
                            a[i] = kk == 0 ? v.x : kk == 1 ? v.y : kk == 2 ? v.z : v.w;
                        } else {
                            const float4 v = am[kk][i >> 2];
                            a[i] = (i & 3) == 0 ? v.x : (i & 3) == 1 ? v.y : (i & 3) == 2 ? v.z : v.w;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        if (B_KMAJ) {
                            const float4 v = bv[j];
                            b[j] = kk == 0 ? v.x : kk == 1 ? v.y : kk == 2 ? v.z : v.w;
                        } else {
                            const float4 v = bm[kk][j >> 2];
                            b[j] = (j & 3) == 0 ? v.x : (j & 3) == 1 ? v.y : (j & 3) == 2 ? v.z : v.w;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++)
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;

        // ------------------------------ epilogue ------------------------------
        float* cmat = p.c + static_cast<long long>(bidx) * p.shape.M * p.shape.N;
        const int row_base = tm * BM + wm * 32;
        const int col_base = tn * BN + wn * 64;
        const float* bias = p.epi.bias;
        const int act = p.epi.act;
#pragma unroll
        for (int ib = 0; ib < 2; ib++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = row_base + ib * 16 + (A_KMAJ ? (i * 4 + ty) : (ty * 4 + i));
                if (r >= p.shape.M) continue;
                float* crow = cmat + static_cast<long long>(r) * p.shape.N;
#pragma unroll
                for (int jb = 0; jb < 2; jb++) {
                    if (B_KMAJ) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const int cidx = col_base + jb * 32 + j * 8 + tx;
                            if (cidx < p.shape.N) {
                                float v = acc[ib * 4 + i][jb * 4 + j];
                                if (bias) v += __ldg(bias + cidx);
                                crow[cidx] = apply_act(v, act);
                            }
                        }
                    } else {
                        const int cidx = col_base + jb * 32 + tx * 4;
                        float v[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            v[j] = acc[ib * 4 + i][jb * 4 + j];
                            if (bias && cidx + j < p.shape.N) v[j] += __ldg(bias + cidx + j);
                            v[j] = apply_act(v[j], act);
                        }
                        if (p.c_vec_ok && cidx + 3 < p.shape.N) {
                            *reinterpret_cast<float4*>(crow + cidx) = make_float4(v[0], v[1], v[2], v[3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                if (cidx + j < p.shape.N) crow[cidx + j] = v[j];
                        }
                    }
                }
            }
    }
}

}  // namespace simt
}  // namespace tt
