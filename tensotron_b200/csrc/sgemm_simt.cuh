// Strict-FP32 SGEMM for sm_100a: SIMT FMA tiles fed by TMA.
//
// One persistent CTA per SM walks a grouped raster of (16*TM)x128 output tiles, TM = 16
// (256x128 tile, 16x8 accumulators per thread) or TM = 8 (128x128, 8x8).  The CTA is three
// warpgroups: two of consumers (8 warps) and one producer warpgroup, of which a single thread
// works.  The producer streams (16*TM)x32 (A) and 32x128 (B) float tiles into a shared-memory
// ring with TMA, as far ahead of the consumers as the ring allows; the consumer warps read the
// tiles with 128-bit shared loads and issue packed two-wide FP32 FMAs (fma.rn.f32x2).  Stages
// are handed over with mbarriers (full: TMA transaction bytes; empty: one arrival per consumer
// warp), and the ring keeps filling across tile boundaries while the previous tile's epilogue
// stores.  The producer warpgroup gives its registers back (setmaxnreg.dec) and the consumers
// take them (setmaxnreg.inc), so the consumers keep the 232 registers their 128 accumulators
// plus fragments need.  (With the loads issued by thread 0 of consumer warp 0, that warp was
// the CTA's critical path: its producer work, serialised with its own FMAs, paced the ring and
// the other seven warps waited on the full barriers for about 4 % of their cycles.)
//
// Why 16x8 per thread and packed FMAs: on this SM the FP32 pipe retires 128 FMAs per
// clock, one warp instruction per scheduler per clock, and shared memory returns
// 128 B/clk.  With scalar FFMA every non-FMA instruction steals an FMA issue slot and an
// 8x8 register tile needs the whole shared-memory return bandwidth.  A 16x8 tile needs
// 75 % of it, and the two-wide FMA halves the FMA issue slots, leaving room for the
// loads.  128 accumulators plus fragments need > 170 registers, hence exactly 8 consumer
// warps (2 per scheduler partition).
//
// Operand layouts.  The main loop wants both operands "MN-major" in shared memory:
// [32 k][rows] with the M (or N) index contiguous, so that a float4 holds 4 adjacent
// rows/columns of one k and adjacent register pairs feed the packed FMA directly.
//   MN-major operand in global memory (A of a TN product, B of NN/TN): TMA lands the
//       tile in exactly that order; the main loop reads the TMA stage itself.
//   K-major operand (A of NN/NT, B of NT): TMA lands [rows][32 k] (128-byte rows,
//       hardware 128B swizzle).  While the FMAs of k-tile i run, the warps transpose
//       k-tile i+1 through registers (4 LDS.128 + 4 STS.128 per 4x4 block) into one of
//       two MN-major buffers whose rows are padded by 16 bytes; one CTA barrier per
//       k-tile (every 8192 FMA cycles) separates writers from readers.
// Summation order over K is fixed (ascending k, one accumulator per output, fused
// multiply-add), so the result does not depend on the tile shape, the grid size or the
// SM that ran a tile.
#pragma once
#include "gemm_common.h"
#include "ptx.cuh"

namespace tt {
namespace simt {

constexpr int BN = 128, BK = 32;
constexpr int WARPS = 8;                        // consumer warps (two warpgroups)
constexpr int CONSUMER_THREADS = WARPS * 32;
constexpr int THREADS = CONSUMER_THREADS + 128; // + the producer warpgroup
constexpr int PRODUCER_REGS = 24, CONSUMER_REGS = 240;   // 128 x 24 + 256 x 240 <= 64 K registers
constexpr int RASTER_GROUP = 8;
constexpr int KG = 4;        // k-steps whose fragments are loaded together
constexpr int G_UNROLL = 4;  // k groups unrolled in the main loop; bounds code size

// CTA barrier over the consumer warps only (the producer warpgroup never joins it).
__device__ __forceinline__ void consumer_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");
}

// NJ = tile width in units of 64 columns: 2 (128 columns, 8 per thread) or 3 (192 columns, 12 per
// thread; TM = 8 and MN-major B only -- a 192-column K-major tile has no transposition routine).
// The 192-wide tile exists for N = 192-like shapes, where 128-wide tiles are a quarter padding.
template <int TM, bool A_KMAJ, bool B_KMAJ, int NJ = 2>
struct Cfg {
    static_assert(NJ == 2 || (NJ == 3 && TM == 8 && !B_KMAJ), "tile width");
    static constexpr int BM = 16 * TM;
    static constexpr int BN = 64 * NJ;
    static constexpr int RAW_A = BM * BK * 4;
    static constexpr int RAW_B = BN * BK * 4;
    static constexpr int STAGE_BYTES = RAW_A + RAW_B;
    // Row pitch (bytes) of the MN-major tile the main loop reads: the TMA stage itself,
    // or the padded transposed copy of a K-major tile.
    static constexpr int ROWB_A = A_KMAJ ? BM * 4 + 16 : BM * 4;
    static constexpr int ROWB_B = B_KMAJ ? BN * 4 + 16 : BN * 4;
    static constexpr int TA_BYTES = A_KMAJ ? BK * ROWB_A : 0;
    static constexpr int TB_BYTES = B_KMAJ ? BK * ROWB_B : 0;
    static constexpr bool HAS_T = A_KMAJ || B_KMAJ;
    static constexpr bool ALL_T = A_KMAJ && B_KMAJ;
    static constexpr int BUDGET = 227 * 1024 - 1024 /*align slack*/ - 512 /*barriers, cursor*/;
    static constexpr int FIT = (BUDGET - 2 * (TA_BYTES + TB_BYTES)) / STAGE_BYTES;
    static constexpr int STAGES = FIT > 4 ? 4 : FIT;
    static constexpr int OFF_TA = STAGES * STAGE_BYTES;
    static constexpr int OFF_TB = OFF_TA + 2 * TA_BYTES;
    static constexpr int OFF_BAR = (OFF_TB + 2 * TB_BYTES + 127) & ~127;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;  // barriers @0, cursor @128, stream-K scratch @256
    static_assert(STAGES >= 2, "shared-memory budget");
};

struct Params {
    GemmShape shape;
    BatchDesc batch;
    Epilogue epi;
    float* c;
    unsigned int* status;  // device status word (bounded waits)
    int c_vec_ok;          // C base 16-byte aligned and N % 4 == 0
    // split-K: every output tile is cut into `splits` k-ranges of `kps` k-tiles; work item
    // w = tile * splits + split.  Partial tiles go to `partial` ([tile][split][BM][BN]);
    // splitk_reduce_kernel adds them in split order and runs the epilogue.
    int splits, kps;
    float* partial;
    // stream-K: one "partial tile stored" flag per CTA (zero outside a launch; set by the CTA
    // whose range starts inside a tile, cleared by the CTA that adds that partial tile)
    unsigned int* sk_flags;
    // stream-K: the first `sk_first` tiles (whole waves of the grid) are computed as whole tiles,
    // round-robin like MODE_TILES; only the tiles behind them are dealt out as k-tile units
    // (shape.work counts those units)
    long long sk_first;
    // stream-K, aligned form (sk_split >= 2, for a remainder of at most half a wave): every
    // remaining tile is cut into sk_split equal k ranges, CTA j takes tile j / sk_split, range
    // j % sk_split.  The CTAs that work on the same range index then walk k together, which keeps
    // the L2 sharing of a whole-tile wave; contiguous unit ranges (sk_split == 0) do not.
    int sk_split;
};

__device__ __forceinline__ float apply_act(float v, int act)
{
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return tanhf(v);
    return v;
}

// Bias and activation of four adjacent outputs (columns c0 .. c0 + 3, those < ncols).  Kept out of
// line on purpose: inlined into the fully unrolled store loops (up to 128 outputs per thread, each
// with its own copy of tanhf) it made the epilogue tens of kilobytes of code that every tile had to
// pull through the instruction cache, which showed as `no_instruction` stalls on short-K shapes
// even when no bias or activation was asked for.  The store loops call it only when there is one.
__device__ __noinline__ void bias_act4(float* v, const float* __restrict__ bias, int c0, int ncols, int act)
{
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (bias && c0 + j < ncols) v[j] += __ldg(bias + c0 + j);
        v[j] = apply_act(v[j], act);
    }
}

// Batch coordinates (TMA coordinate slots 0..2 per operand) of batch entry bidx.
struct BatchCoords {
    int a[3], b[3];
};

__device__ __forceinline__ BatchCoords batch_coords(const BatchDesc& batch, int bidx)
{
    BatchCoords c;
    c.a[0] = c.a[1] = c.a[2] = 0;
    c.b[0] = c.b[1] = c.b[2] = 0;
    int br = bidx;
    for (int ax = batch.rank - 1; ax >= 0; ax--) {
        const int d = batch.dims[ax];
        const int bi = br % d;
        br /= d;
        const int sa = batch.a_slot[ax], sb = batch.b_slot[ax];
        if (sa == 0) c.a[0] += bi * batch.a_mult[ax];
        else if (sa == 1) c.a[1] += bi * batch.a_mult[ax];
        else if (sa == 2) c.a[2] += bi * batch.a_mult[ax];
        if (sb == 0) c.b[0] += bi * batch.b_mult[ax];
        else if (sb == 1) c.b[1] += bi * batch.b_mult[ax];
        else if (sb == 2) c.b[2] += bi * batch.b_mult[ax];
    }
    return c;
}

// Transposes one K-major TMA tile ([ROWS][32 k], 128B-swizzled) into an MN-major tile
// ([32 k][ROWS], row pitch ROWB bytes).  Each thread moves 4x4 blocks: block (R, c) =
// rows 4R..4R+3, k 4c..4c+3.  A quarter warp covers 4 chunks x 2 row groups, which
// makes the swizzled reads conflict-free and the padded writes 2-way.
template <int ROWS, int ROWB>
__device__ __forceinline__ void transpose_tile(const uint8_t* raw, uint8_t* dst, int warp, int lane)
{
    constexpr int ITER = ROWS / 128;  // blocks per thread
#pragma unroll
    for (int u = 0; u < ITER; u++) {
        const int R = (ROWS == 256 ? warp * 8 : (warp & 3) * 8) + (lane >> 2);
        const int c = (ROWS == 256 ? u * 4 : (warp >> 2) * 4) + (lane & 3);
        const int rsw = (R & 1) << 2;  // (4R + i) & 7 == rsw + i
        float4 r[4];
#pragma unroll
        for (int i = 0; i < 4; i++)
            r[i] = *reinterpret_cast<const float4*>(raw + (4 * R + i) * 128 + ((c ^ (rsw + i)) << 4));
        uint8_t* out = dst + (4 * c) * ROWB + R * 16;
        *reinterpret_cast<float4*>(out) = make_float4(r[0].x, r[1].x, r[2].x, r[3].x);
        *reinterpret_cast<float4*>(out + ROWB) = make_float4(r[0].y, r[1].y, r[2].y, r[3].y);
        *reinterpret_cast<float4*>(out + 2 * ROWB) = make_float4(r[0].z, r[1].z, r[2].z, r[3].z);
        *reinterpret_cast<float4*>(out + 3 * ROWB) = make_float4(r[0].w, r[1].w, r[2].w, r[3].w);
    }
}

// How a CTA's work is cut (compile-time, because a second epilogue body in the kernel cost
// the main loop 14 % through register allocation; the three modes share one store loop):
//   MODE_TILES   whole output tiles, round-robin over the CTAs;
//   MODE_SPLITK  every tile cut into `splits` equal k ranges (small M x N);
//   MODE_STREAMK whole waves of tiles first (round-robin, so the CTAs in flight share A and B
//                panels in L2 exactly as in MODE_TILES); the tiles x k-tiles units of the rest
//                are dealt to the CTAs as equal contiguous ranges,
//                so no SM idles in a partial last wave.  A CTA whose range starts inside a tile
//                computes that segment first, stores it as a partial tile and raises its flag;
//                the CTA that holds the head of the tile (k from 0, the last segment of its
//                range) adds the partial tiles of the following CTAs to its accumulators in
//                ascending k and stores the finished tile.  The partial tiles it needs were
//                stored about a tile's time earlier, so the wait is normally over before it
//                starts (it is bounded like every other wait).
constexpr int MODE_TILES = 0, MODE_SPLITK = 1, MODE_STREAMK = 2;

template <int TM, bool A_KMAJ, bool B_KMAJ, int MODE, int NJ = 2>
__global__ void __launch_bounds__(THREADS, 1)
sgemm_simt_kernel(const __grid_constant__ CUtensorMap map_a,
                  const __grid_constant__ CUtensorMap map_b, const Params p)
{
    using C = Cfg<TM, A_KMAJ, B_KMAJ, NJ>;
    constexpr int STAGES = C::STAGES;
    constexpr int BN = C::BN;      // this instantiation's tile width (shadows the 128-column default)
    constexpr int HALVES = TM / 8;  // 8-row halves of the thread tile
    extern __shared__ uint8_t smem_raw[];
    // 128B-swizzled tiles need 1024-byte alignment.
    // (pointer arithmetic on the shared array itself, so the compiler keeps emitting
    // shared-space loads rather than generic ones)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty_bar = full_bar + STAGES;
    volatile uint32_t* cta_abort = reinterpret_cast<volatile uint32_t*>(empty_bar + STAGES);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    const int k_tiles = (p.shape.K + BK - 1) / BK;
    const int tiles_per_mat = p.shape.tiles_m * p.shape.tiles_n;
    // This CTA's work: items blockIdx.x, +gridDim.x, ... (< work), or for MODE_STREAMK the
    // contiguous unit range [w_begin, w_end) of the work = tiles x k-tiles units.
    // (both the producer and the consumers walk it with the cursor pair below: `ca` over the
    // round-robin items, then `cw` over the unit range)
    const long long a_end = MODE == 2 ? p.sk_first : p.shape.work;
    // (the unit part is at most a tile and a half per CTA: its unit count fits 32 bits, the host
    // checks)
    int w_begin = 0, w_end = 0;
    if (MODE == 2) {
        if (p.sk_split >= 2) {
            const int kps = (k_tiles + p.sk_split - 1) / p.sk_split;
            const int tile = blockIdx.x / p.sk_split, part = blockIdx.x - tile * p.sk_split;
            if (static_cast<long long>(tile) * k_tiles < p.shape.work) {      // (CTAs beyond the last tile idle here)
                w_begin = tile * k_tiles + min(k_tiles, part * kps);
                w_end = tile * k_tiles + min(k_tiles, (part + 1) * kps);
            }
        } else {
            w_begin = static_cast<int>((p.shape.work * blockIdx.x) / gridDim.x);
            w_end = static_cast<int>((p.shape.work * (blockIdx.x + 1)) / gridDim.x);
        }
    }

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], WARPS);
        }
        *cta_abort = 0u;
        fence_mbar_init();
    }
    __syncthreads();

    if (warp >= WARPS) {
        // ------------------------- producer warpgroup -------------------------
        // Walks the same (work item, reduced-axis entry, k-tile) sequence as the consumers and
        // fills the ring as far ahead as the empty barriers allow.  One thread; its cursor
        // lives in registers.
        setmaxnreg_dec<PRODUCER_REGS>();
        if (warp != WARPS || lane != 0) return;
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        uint32_t ps = 0, use = 0;   // stage to fill next; how many times the ring has wrapped
        bool ok = true;
        const int sra = p.batch.red_a_slot, srb = p.batch.red_b_slot;
        long long ca = blockIdx.x;
        int cw = w_begin;
        while (ok) {
            long long unit;
            int kb, ke;
            if (ca < a_end) {
                unit = ca / p.splits;
                const int split = static_cast<int>(ca - unit * p.splits);
                kb = split * p.kps;
                ke = min(k_tiles, kb + p.kps);
                ca += gridDim.x;
            } else if (MODE == 2 && cw < w_end) {
                const int tu = cw / k_tiles;
                unit = p.sk_first + tu;
                kb = cw - tu * k_tiles;
                ke = min(k_tiles, kb + (w_end - cw));
                cw += ke - kb;
            } else {
                break;
            }
            const int bidx = static_cast<int>(unit / tiles_per_mat);
            const int t = static_cast<int>(unit - static_cast<long long>(bidx) * tiles_per_mat);
            int tm, tn;
            raster_tile(t, p.shape.tiles_m, p.shape.tiles_n, RASTER_GROUP, tm, tn);
            const int m0 = tm * C::BM, n0 = tn * BN;
            const BatchCoords bc = batch_coords(p.batch, bidx);
            for (int r = 0; ok && r < p.batch.red_count; r++) {
                // the reduced batch axis has a coordinate slot of its own (or none when the
                // operand is broadcast along it)
                const int ca0 = bc.a[0] + (sra == 0 ? r : 0), ca1 = bc.a[1] + (sra == 1 ? r : 0),
                          ca2 = bc.a[2] + (sra == 2 ? r : 0);
                const int cb0 = bc.b[0] + (srb == 0 ? r : 0), cb1 = bc.b[1] + (srb == 1 ? r : 0),
                          cb2 = bc.b[2] + (srb == 2 ? r : 0);
                for (int kt = kb; kt < ke; kt++) {
                    if (use > 0) {
                        // the stage was used before: wait until all warps released that use
                        if (!mbar_wait_bounded(&empty_bar[ps], (use - 1) & 1u, cta_abort, p.status, DEV_WAIT_EMPTY)) {
                            ok = false;
                            break;
                        }
                    }
                    uint8_t* sa = smem + ps * C::STAGE_BYTES;
                    uint8_t* sb = sa + C::RAW_A;
                    mbar_arrive_expect_tx(&full_bar[ps], C::STAGE_BYTES);
                    const int k0 = kt * BK;
                    if (A_KMAJ) tma_load_5d(sa, &map_a, &full_bar[ps], k0, m0, ca0, ca1, ca2);
                    else        tma_load_5d(sa, &map_a, &full_bar[ps], m0, k0, ca0, ca1, ca2);
                    if (B_KMAJ) tma_load_5d(sb, &map_b, &full_bar[ps], k0, n0, cb0, cb1, cb2);
                    else        tma_load_5d(sb, &map_b, &full_bar[ps], n0, k0, cb0, cb1, cb2);
                    if (++ps == STAGES) { ps = 0; use++; }
                }
            }
        }
        if (!ok) {
            // A wait gave up: before this thread leaves (and the CTA's shared memory can go), wait,
            // again with a limit, for the loads it issued itself -- the last arming of every stage.
            uint32_t s = ps, u = use;
            for (int i = 0; i < STAGES; i++) {
                if (s == 0) {
                    if (u == 0) break;      // fewer than STAGES loads were ever issued
                    s = STAGES;
                    u--;
                }
                s--;
                mbar_wait_drain(&full_bar[s], u & 1u);
            }
        }
        return;
    }
    // ------------------------------ consumer warps ------------------------------
    setmaxnreg_inc<CONSUMER_REGS>();

    // Transposes the K-major tiles of TMA stage `s` into transposed buffer `tb`.
    auto transpose_stage = [&](uint32_t s, uint32_t tb) {
        const uint8_t* raw = smem + s * C::STAGE_BYTES;
        if constexpr (A_KMAJ)
            transpose_tile<C::BM, C::ROWB_A>(raw, smem + C::OFF_TA + tb * C::TA_BYTES, warp, lane);
        if constexpr (B_KMAJ)
            transpose_tile<BN, C::ROWB_B>(raw + C::RAW_A, smem + C::OFF_TB + tb * C::TB_BYTES, warp, lane);
    };

    uint32_t stage = 0, phase = 0, tb = 0;
    if (C::HAS_T) {
        // prologue: k-tile 0 of the first tile
        if (mbar_wait_bounded(&full_bar[0], 0u, cta_abort, p.status, DEV_WAIT_FULL)) {
            transpose_stage(0, 0);
            if (C::ALL_T) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[0]);
            }
        }
        consumer_sync();
        if (*cta_abort) return;
    }

    // ---- consumer mapping: warp grid 4 (m) x 2 (n), lane grid 4 (ty) x 8 (tx) ----
    const int wm = warp >> 1;
    const int wn = warp & 1;
    const int ty = lane >> 3;
    const int tx = lane & 7;
    constexpr int WROWS = C::BM / 4;  // rows per warp: 32 (TM=8) or 64 (TM=16)
    const int off_am = (wm * WROWS + ty * 4) * 4;
    const int off_bm = (wn * (32 * NJ) + tx * 4) * 4;

    long long ca = blockIdx.x;
    int cw = w_begin;
    for (;;) {
        long long unit;
        long long w = 0;      // MODE_SPLITK: this item's index (its workspace slot)
        int kb, ke;
        if (ca < a_end) {
            w = ca;
            unit = ca / p.splits;
            const int split = static_cast<int>(ca - unit * p.splits);
            kb = split * p.kps;
            ke = min(k_tiles, kb + p.kps);
            ca += gridDim.x;
        } else if (MODE == 2 && cw < w_end) {
            const int tu = cw / k_tiles;
            unit = p.sk_first + tu;
            kb = cw - tu * k_tiles;
            ke = min(k_tiles, kb + (w_end - cw));
            cw += ke - kb;
        } else {
            break;
        }
        const int bidx = static_cast<int>(unit / tiles_per_mat);
        const int t = static_cast<int>(unit - static_cast<long long>(bidx) * tiles_per_mat);
        int tm, tn;
        raster_tile(t, p.shape.tiles_m, p.shape.tiles_n, RASTER_GROUP, tm, tn);
        const bool last_tile = ca >= a_end && cw >= w_end;

        // Accumulators are packed float2 for the two-wide FP32 FMA.  For a row pair
        // (i, i+1) and a column pair (j, j+1):
        //   d0 = (C[i][j],   C[i+1][j+1]) += (a_i, a_i+1) * (b_j,   b_j+1)
        //   d1 = (C[i][j+1], C[i+1][j])   += (a_i, a_i+1) * (b_j+1, b_j)
        // so neither operand has to be broadcast into both halves of a register pair;
        // only the swapped column pair is built.  Each lane is an independent IEEE fma
        // in ascending k, so the bits equal the scalar-FMA formulation.
        float2 d0[TM / 2][2 * NJ], d1[TM / 2][2 * NJ];
#pragma unroll
        for (int i = 0; i < TM / 2; i++)
#pragma unroll
            for (int j = 0; j < 2 * NJ; j++) d0[i][j] = d1[i][j] = make_float2(0.f, 0.f);

        const int iters = (ke - kb) * p.batch.red_count;  // k-tiles x entries of the reduced axis
#pragma unroll 1
        for (int it = 0; it < iters; it++) {
            bool ok = true;
            if (!C::HAS_T)
                ok = mbar_wait_bounded(&full_bar[stage], phase, cta_abort, p.status, DEV_WAIT_FULL);
            if (!C::HAS_T && !ok) return;  // no CTA barriers on this path: leaving is safe

            const uint8_t* st = smem + stage * C::STAGE_BYTES;
            const uint8_t* sa = (A_KMAJ ? smem + C::OFF_TA + tb * C::TA_BYTES : st) + off_am;
            const uint8_t* sb = (B_KMAJ ? smem + C::OFF_TB + tb * C::TB_BYTES : st + C::RAW_A) + off_bm;

            const auto k_group = [&](int g) {  // one group of KG k-steps
                const uint8_t* sag = sa + g * KG * C::ROWB_A;
                const uint8_t* sbg = sb + g * KG * C::ROWB_B;
                float4 bm[KG][NJ];  // [k][32-column block] = 4 adjacent cols
#pragma unroll
                for (int kk = 0; kk < KG; kk++)
#pragma unroll
                    for (int jb = 0; jb < NJ; jb++)
                        bm[kk][jb] = *reinterpret_cast<const float4*>(sbg + kk * C::ROWB_B + jb * 128);
#pragma unroll
                for (int h = 0; h < HALVES; h++) {
                    float4 am[KG][2];  // [k][ib] = 4 adjacent rows
#pragma unroll
                    for (int kk = 0; kk < KG; kk++)
#pragma unroll
                        for (int ib = 0; ib < 2; ib++)
                            am[kk][ib] = *reinterpret_cast<const float4*>(
                                sag + kk * C::ROWB_A + (h * 32 + ib * 16) * 4);
#pragma unroll
                    for (int kk = 0; kk < KG; kk++) {
                        float2 a2[4], b2[2 * NJ], b2s[2 * NJ];
#pragma unroll
                        for (int pr = 0; pr < 4; pr++) {  // row pairs of this half
                            const float4 v = am[kk][pr >> 1];
                            a2[pr] = (pr & 1) ? make_float2(v.z, v.w) : make_float2(v.x, v.y);
                        }
#pragma unroll
                        for (int q = 0; q < 2 * NJ; q++) {  // column pairs
                            const float4 v = bm[kk][q >> 1];
                            b2[q] = (q & 1) ? make_float2(v.z, v.w) : make_float2(v.x, v.y);
                            b2s[q] = make_float2(b2[q].y, b2[q].x);
                        }
#pragma unroll
                        for (int pr = 0; pr < 4; pr++)
#pragma unroll
                            for (int q = 0; q < 2 * NJ; q++) {
                                d0[h * 4 + pr][q] = __ffma2_rn(a2[pr], b2[q], d0[h * 4 + pr][q]);
                                d1[h * 4 + pr][q] = __ffma2_rn(a2[pr], b2s[q], d1[h * 4 + pr][q]);
                            }
                    }
                }
            };
#pragma unroll G_UNROLL
            for (int g = 0; g < BK / KG; g++) k_group(g);

            // advance to the next k-tile's stage
            uint32_t nstage = stage + 1, nphase = phase;
            if (nstage == STAGES) { nstage = 0; nphase ^= 1u; }
            if (!C::ALL_T) {
                // this k-tile's TMA stage was read by the main loop: release it
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[stage]);
            }
            if (C::HAS_T) {
                if (!(last_tile && it == iters - 1)) {  // a next k-tile exists
                    if (mbar_wait_bounded(&full_bar[nstage], nphase, cta_abort, p.status, DEV_WAIT_FULL)) {
                        transpose_stage(nstage, tb ^ 1u);
                        if (C::ALL_T) {
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&empty_bar[nstage]);
                        }
                    }
                }
                // writers of buffer tb^1 | readers of buffer tb: one barrier orders both
                consumer_sync();
                if (*cta_abort) return;  // uniform: every thread sees the flag after the barrier
                tb ^= 1u;
            }
            stage = nstage;
            phase = nphase;
        }

        // ------------------------------ epilogue ------------------------------
        // Unpacked view of the accumulators: element (r, c) of the thread tile.
        const auto acc_at = [&](int r, int c) -> float {
            const float2 v = ((r & 1) == (c & 1)) ? d0[r >> 1][c >> 1] : d1[r >> 1][c >> 1];
            return (r & 1) ? v.y : v.x;
        };
        const auto acc_ref = [&](int r, int c) -> float& {
            float2& v = ((r & 1) == (c & 1)) ? d0[r >> 1][c >> 1] : d1[r >> 1][c >> 1];
            return (r & 1) ? v.y : v.x;
        };
        (void)acc_ref;
        if constexpr (MODE == MODE_TILES) {
            // whole tiles only: store straight to C
            float* cmat = p.c + static_cast<long long>(bidx) * p.shape.M * p.shape.N;
            const float* bias = p.epi.bias;
            const int act = p.epi.act;
            const bool plain = bias == nullptr && act == 0;
#pragma unroll
            for (int h = 0; h < HALVES; h++)
#pragma unroll
                for (int ib = 0; ib < 2; ib++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int lr = wm * WROWS + h * 32 + ib * 16 + ty * 4 + i;
                        const int r = tm * C::BM + lr;
                        if (r >= p.shape.M) continue;
                        float* crow = cmat + static_cast<long long>(r) * p.shape.N;
                        const int ai = h * 8 + ib * 4 + i;
#pragma unroll
                        for (int jb = 0; jb < NJ; jb++) {
                            const int lc = wn * (32 * NJ) + jb * 32 + tx * 4;
                            const int cidx = tn * BN + lc;
                            float v[4];
#pragma unroll
                            for (int j = 0; j < 4; j++) v[j] = acc_at(ai, jb * 4 + j);
                            if (!plain) bias_act4(v, bias, cidx, p.shape.N, act);
                            if (p.c_vec_ok && cidx + 3 < p.shape.N) {
                                *reinterpret_cast<float4*>(crow + cidx) = make_float4(v[0], v[1], v[2], v[3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; j++)
                                    if (cidx + j < p.shape.N) crow[cidx + j] = v[j];
                            }
                        }
                    }
        } else {
            // One store loop for all modes.  A finished tile goes to C (bounds, bias, activation);
            // a partial one (split-K range, or a stream-K range that covers only part of the
            // tile's k) goes densely ([BM][BN]) to a workspace slot.
            bool partial_tile = false, head_tile = false;
            long long slot = 0;
            if (MODE == 1) {
                partial_tile = p.splits > 1;
                slot = w;
            } else if (MODE == 2) {
                // range starts inside the tile: hand the segment over (slot = this CTA); head of a tile
                // that the following CTAs finish: stored the same way (slot = grid + this CTA) and
                // added up from memory below
                partial_tile = kb != 0;
                head_tile = kb == 0 && ke != k_tiles;
                slot = head_tile ? gridDim.x + blockIdx.x : blockIdx.x;
            }
            const bool raw = partial_tile || head_tile;
            float* base;
            int ld, row_lim, col_lim, vec_ok;
            const float* bias = nullptr;
            int act = 0;
            if (raw) {
                base = p.partial + slot * (C::BM * BN);
                ld = BN; row_lim = C::BM; col_lim = BN; vec_ok = 1;
            } else {
                base = scatter_base(p.epi, p.c, tm * C::BM) + static_cast<long long>(bidx) * p.shape.M * p.shape.N +
                       static_cast<long long>(tm) * C::BM * p.shape.N + tn * BN;
                ld = p.shape.N; row_lim = p.shape.M - tm * C::BM; col_lim = p.shape.N - tn * BN;
                vec_ok = p.c_vec_ok;
                bias = p.epi.bias ? p.epi.bias + tn * BN : nullptr;
                act = p.epi.act;
            }
    #pragma unroll
            for (int h = 0; h < HALVES; h++)
    #pragma unroll
                for (int ib = 0; ib < 2; ib++)
    #pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int lr = wm * WROWS + h * 32 + ib * 16 + ty * 4 + i;
                        if (lr >= row_lim) continue;
                        float* crow = base + static_cast<long long>(lr) * ld;
                        const int ai = h * 8 + ib * 4 + i;
    #pragma unroll
                        for (int jb = 0; jb < NJ; jb++) {
                            const int lc = wn * (32 * NJ) + jb * 32 + tx * 4;
                            float v[4];
    #pragma unroll
                            for (int j = 0; j < 4; j++) v[j] = acc_at(ai, jb * 4 + j);
                            if (bias != nullptr || act != 0) bias_act4(v, bias, lc, col_lim, act);
                            if (vec_ok && lc + 3 < col_lim) {
                                *reinterpret_cast<float4*>(crow + lc) = make_float4(v[0], v[1], v[2], v[3]);
                            } else {
    #pragma unroll
                                for (int j = 0; j < 4; j++)
                                    if (lc + j < col_lim) crow[lc + j] = v[j];
                            }
                        }
                    }
            if (MODE == 2 && partial_tile) {
                // the partial tile is stored: fence, CTA barrier, flag (release)
                __threadfence();
                consumer_sync();
                if (tid == 0) {
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + blockIdx.x), "r"(1u) : "memory");
                }
            }
            if (MODE == 2 && head_tile) {
                // Head of a tile that the following CTAs finish.  The accumulators are in memory
                // now; the tile is put together from memory: this CTA's segment (k from 0) plus
                // the partial tiles of the following CTAs in ascending CTA = ascending k, then the
                // epilogue.  (Adding the partial tiles to the accumulators instead would give the
                // kernel a second loop over all 128 of them, which costs the main loop registers.)
                volatile int& s_hi = *reinterpret_cast<volatile int*>(smem + C::OFF_BAR + 256);
                if (tid == 0) {
                    int hi = blockIdx.x;
                    if (p.sk_split >= 2) {
                        // the non-empty ranges of this tile: parts 1 .. ceil(k_tiles / kps) - 1
                        const int kps = (k_tiles + p.sk_split - 1) / p.sk_split;
                        hi = blockIdx.x + (k_tiles + kps - 1) / kps - 1;
                    } else {
                        const long long u_hi = (unit - p.sk_first + 1) * k_tiles;   // end of this tile in the unit range
                        while (hi + 1 < static_cast<int>(gridDim.x) && (p.shape.work * (hi + 1)) / gridDim.x < u_hi) hi++;
                    }
                    s_hi = hi;
                    for (int cta = blockIdx.x + 1; cta <= hi; cta++) {
                        const unsigned long long t0 = global_timer_ns();
                        unsigned int spins = 0, v;
                        for (;;) {
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.sk_flags + cta) : "memory");
                            if (v != 0u) break;
                            if ((++spins & 63u) == 0 && global_timer_ns() - t0 > WAIT_LIMIT_NS) {
                                *cta_abort = 1u;
                                if (p.status) atomicCAS(p.status, 0u, static_cast<unsigned int>(DEV_WAIT_STREAMK));
                                break;
                            }
                        }
                        p.sk_flags[cta] = 0u;   // consumed: the next launch starts from zero again
                    }
                }
                consumer_sync();                // this CTA's segment is stored; the others' flags were seen
                if (*cta_abort) return;
                const int hi = s_hi;
                const float* mine = p.partial + slot * (C::BM * BN);
                float* ctile = scatter_base(p.epi, p.c, tm * C::BM) + static_cast<long long>(bidx) * p.shape.M * p.shape.N +
                               static_cast<long long>(tm) * C::BM * p.shape.N + tn * BN;
                const int rows_here = p.shape.M - tm * C::BM, cols_here = p.shape.N - tn * BN;
                const float* tbias = p.epi.bias ? p.epi.bias + tn * BN : nullptr;
                // Eight float4 per thread at a time: all loads of a group are issued before the first
                // is used (the stores to C may alias the workspace as far as the compiler knows, so it
                // would not move loads across them by itself).
                constexpr int UF = 8;
                constexpr int TOTAL4 = C::BM * BN / 4;
                for (int e0 = tid; e0 < TOTAL4; e0 += WARPS * 32 * UF) {
                    float4 sum[UF];
    #pragma unroll
                    for (int u = 0; u < UF; u++) {
                        const int e = e0 + u * WARPS * 32;
                        sum[u] = e < TOTAL4 ? __ldcg(reinterpret_cast<const float4*>(mine) + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    for (int cta = blockIdx.x + 1; cta <= hi; cta++) {
                        const float4* part = reinterpret_cast<const float4*>(p.partial + static_cast<long long>(cta) * (C::BM * BN));
                        float4 q[UF];
    #pragma unroll
                        for (int u = 0; u < UF; u++) {
                            const int e = e0 + u * WARPS * 32;
                            q[u] = e < TOTAL4 ? __ldcg(part + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
    #pragma unroll
                        for (int u = 0; u < UF; u++) {
                            sum[u].x += q[u].x; sum[u].y += q[u].y; sum[u].z += q[u].z; sum[u].w += q[u].w;
                        }
                    }
    #pragma unroll
                    for (int u = 0; u < UF; u++) {
                        const int e = e0 + u * WARPS * 32;
                        const int lr = e / (BN / 4), lc = (e % (BN / 4)) * 4;
                        if (e >= TOTAL4 || lr >= rows_here || lc >= cols_here) continue;
                        float v[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
                        if (tbias != nullptr || p.epi.act != 0) bias_act4(v, tbias, lc, cols_here, p.epi.act);
                        float* crow = ctile + static_cast<long long>(lr) * p.shape.N;
                        if (p.c_vec_ok && lc + 3 < cols_here) {
                            *reinterpret_cast<float4*>(crow + lc) = make_float4(v[0], v[1], v[2], v[3]);
                        } else {
    #pragma unroll
                            for (int j = 0; j < 4; j++)
                                if (lc + j < cols_here) crow[lc + j] = v[j];
                        }
                    }
                }
            }
        }
    }
}

// C = act(sum over splits (ascending) of the partial tiles + bias).  One thread per 4
// consecutive columns of one tile row; grid covers tiles x (BM * BN / 4) threads.
template <int BM>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ c, GemmShape shape,
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
    int tm, tn;
    raster_tile(t, shape.tiles_m, shape.tiles_n, RASTER_GROUP, tm, tn);
    const int r = tm * BM + lr, cidx = tn * BN + lc;
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
        v[j] = apply_act(v[j], epi.act);
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

}  // namespace simt
}  // namespace tt
