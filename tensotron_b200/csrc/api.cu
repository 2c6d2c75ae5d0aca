// C ABI of libtensotron_gemm.so: argument checks, layout classification, variant
// choice, TMA descriptor construction and kernel launches.  Nothing here allocates,
// synchronises or copies from pageable memory after tt_create, so every compute call
// can be recorded into a CUDA graph.
#include "../../include/tensotron_gemm.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdio.h>
#include <string.h>

#include "conv.cuh"
#include "elementwise.cuh"
#include "gemm_common.h"
#include "gemm_generic.cuh"
#include "linear_small.cuh"
#include "mlp_step.h"
#include "peer.cuh"
#include "sgemm_simt.cuh"
#include "skinny.cuh"
#include "tensor_map.h"
#include "tf32_launch.h"

using namespace tt;

struct tt_handle_s {
    CUcontext ctx;   // the CUDA context the handle's memory and kernels live in (see tt_create)
    int device;
    int num_sms;
    int max_cluster;   // largest thread-block cluster the any-stride kernel may use (16, else the portable 8)
    int math_mode;
    int variant;  // 0 auto, 1 generic, 2 simt-tma 256x128, 3 simt-tma 128x128, 4/5 tcgen05 tile height 128/256
    uint8_t* workspace;
    size_t workspace_bytes;
    unsigned int* status;  // device status word
    tt_stats stats;
    long long map_hits0, map_misses0;   // descriptor-cache totals at the last tt_reset_stats
    char err[256];
};

namespace {

constexpr size_t DEFAULT_WORKSPACE = 256ull << 20;
// Device words owned by the handle: word 0 = status of the bounded waits; from word 64 on, one
// stream-K flag per CTA (zero between launches).
constexpr int STREAMK_FLAGS_WORD = 64, HANDLE_WORDS = 1024;
constexpr long long TMA_MIN_FLOP_ELEMS = 1ll << 21;  // M*N*K below this -> any-stride kernel
constexpr long long SMALL_3XTF32_MAX_ELEMS = 1ll << 28;  // M x N x K up to which 3xTF32 runs on the strict-FP32 kernels
constexpr long long LINEAR_SMALL_MAX_ELEMS = 1ll << 21;  // M x N x K up to which a Linear backward is ONE launch (linear_small.cuh)
constexpr long long SMALL_MAX_FLOP_ELEMS = 1ll << 27;  // ... and up to this when the output is a few tiles only

int fail(tt_handle_t h, int code, const char* fmt, const char* detail = "")
{
    if (h) snprintf(h->err, sizeof(h->err), fmt, detail);
    return code;
}

int cuda_fail(tt_handle_t h, cudaError_t e, const char* what)
{
    if (h) snprintf(h->err, sizeof(h->err), "%s: %s", what, cudaGetErrorString(e));
    return TT_ERR_CUDA;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- batch handling -------------------------------------------------------------

struct HostBatch {
    int rank = 0;
    int dims[MAX_BATCH_RANK];
    int as[MAX_BATCH_RANK];
    int bs[MAX_BATCH_RANK];
    // one merged batch axis that is summed into the output (1 = none)
    int red_count = 1;
    int red_as = 0, red_bs = 0;
};

// Drops size-1 axes and merges adjacent axes that are jointly contiguous for both
// operands (broadcast merges with broadcast).  Returns false when more than
// MAX_BATCH_RANK axes remain.
bool collapse_batch(int rank, const int* dims, const int* as, const int* bs, HostBatch& out)
{
    out.rank = 0;
    for (int ax = 0; ax < rank; ax++) {
        if (dims[ax] == 1) continue;
        if (out.rank > 0) {
            const int o = out.rank - 1;
            // previous (outer) axis o, this (inner) axis ax: mergeable when
            // stride_outer == dim_inner * stride_inner for both operands
            if (static_cast<long long>(out.as[o]) == static_cast<long long>(dims[ax]) * as[ax] &&
                static_cast<long long>(out.bs[o]) == static_cast<long long>(dims[ax]) * bs[ax]) {
                out.dims[o] *= dims[ax];
                out.as[o] = as[ax];
                out.bs[o] = bs[ax];
                continue;
            }
        }
        if (out.rank == MAX_BATCH_RANK) return false;
        out.dims[out.rank] = dims[ax];
        out.as[out.rank] = as[ax];
        out.bs[out.rank] = bs[ax];
        out.rank++;
    }
    return true;
}

// Per-operand TMA batch dims: walks the axes innermost-first, skipping broadcast
// axes, merging an axis into the open slot when it continues it contiguously.
// Fills slot/mult for the kernel and appends (extent, stride) to the view.
bool plan_tma_batch(const HostBatch& hb, const int* strides, signed char* slot, int* mult,
                    OperandView& view, int red_stride, signed char* red_slot)
{
    int nslots = 0;
    long long cur_extent = 0, cur_stride = 0;
    int slot_extent[3] = {1, 1, 1};
    long long slot_stride[3] = {0, 0, 0};
    for (int ax = hb.rank - 1; ax >= 0; ax--) {
        if (strides[ax] == 0) { slot[ax] = -1; mult[ax] = 0; continue; }
        if (nslots > 0 && static_cast<long long>(strides[ax]) == cur_extent * cur_stride) {
            slot[ax] = static_cast<signed char>(nslots - 1);
            mult[ax] = static_cast<int>(cur_extent);
            cur_extent *= hb.dims[ax];
            slot_extent[nslots - 1] = static_cast<int>(cur_extent);
            continue;
        }
        if (nslots == 3) return false;
        slot[ax] = static_cast<signed char>(nslots);
        mult[ax] = 1;
        cur_extent = hb.dims[ax];
        cur_stride = strides[ax];
        slot_extent[nslots] = hb.dims[ax];
        slot_stride[nslots] = strides[ax];
        nslots++;
    }
    *red_slot = -1;
    if (hb.red_count > 1 && red_stride != 0) {
        // the reduced axis gets a coordinate slot of its own
        if (nslots == 3) return false;
        *red_slot = static_cast<signed char>(nslots);
        slot_extent[nslots] = hb.red_count;
        slot_stride[nslots] = red_stride;
        nslots++;
    }
    for (int s = 0; s < nslots; s++) {
        if (slot_stride[s] < 0) return false;
        view.dim[view.rank] = static_cast<uint64_t>(slot_extent[s]);
        view.stride_elems[view.rank] = static_cast<uint64_t>(slot_stride[s]);
        view.rank++;
    }
    return true;
}

void fill_batch_desc(const HostBatch& hb, BatchDesc& bd)
{
    memset(&bd, 0, sizeof(bd));
    bd.rank = hb.rank;
    for (int i = 0; i < hb.rank; i++) {
        bd.dims[i] = hb.dims[i];
        bd.a_stride[i] = hb.as[i];
        bd.b_stride[i] = hb.bs[i];
        bd.a_slot[i] = bd.b_slot[i] = -1;
    }
    bd.red_count = hb.red_count;
    bd.red_a_stride = hb.red_as;
    bd.red_b_stride = hb.red_bs;
    bd.red_a_slot = bd.red_b_slot = -1;
}

// ---- operand classification -----------------------------------------------------

// Builds the 2-D part of a TMA view for one operand.  `rows` is the M (or N) extent,
// row_stride / k_stride the element strides of that axis and of K.  Returns 1 for a
// K-major view, 0 for an MN-major view, -1 when neither axis is contiguous.
int operand_view(const float* base, int rows, int K, int row_stride, int k_stride,
                 OperandView& v)
{
    v.base = base;
    v.rank = 2;
    v.stride_elems[0] = 1;
    // A size-1 axis has no meaningful stride: give it the next legal one.
    const auto legal = [](long long extent) {
        return static_cast<uint64_t>(((extent + 3) / 4) * 4);
    };
    if (k_stride == 1 || K == 1) {
        if (rows > 1 && row_stride <= 0) return -1;
        v.dim[0] = K; v.dim[1] = rows;
        v.stride_elems[1] = rows == 1 ? legal(K) : static_cast<uint64_t>(row_stride);
        return 1;
    }
    if (row_stride == 1 || rows == 1) {
        if (k_stride <= 0) return -1;
        v.dim[0] = rows; v.dim[1] = K;
        v.stride_elems[1] = static_cast<uint64_t>(k_stride);
        return 0;
    }
    return -1;
}

struct GemmCall {
    const float* a;
    const float* b;
    float* c;
    int M, N, K, aMs, aKs, bKs, bNs;
    HostBatch batch;
    int batch_count;
    Epilogue epi;
    size_t ws_off = 0;  // first free byte of the handle workspace for this call
};

int launch_generic(tt_handle_t h, cudaStream_t st, const GemmCall& g)
{
    generic::Params p;
    p.a = g.a; p.b = g.b; p.c = g.c;
    p.shape.M = g.M; p.shape.N = g.N; p.shape.K = g.K;
    p.shape.tiles_m = (g.M + generic::BM - 1) / generic::BM;
    p.shape.tiles_n = (g.N + generic::BN - 1) / generic::BN;
    p.shape.batch = g.batch_count;
    const long long tiles = static_cast<long long>(g.batch_count) * p.shape.tiles_m * p.shape.tiles_n;
    // Split K when the tiles alone leave most of the machine idle: aim at about two CTAs per
    // SM and at least 64 k per range.  Up to 16 ranges (a power of two) run as one thread-block
    // cluster per tile that adds its partial tiles through distributed shared memory (one
    // launch, no workspace); beyond that the partial tiles go to the workspace and a second
    // kernel adds them.  Both forms add the ranges in ascending k, so they give the same bits.
    int splits = 1, kspan = g.K > 0 ? g.K : 1;
    bool cluster = false;
    const size_t ws_avail = h->workspace_bytes > g.ws_off ? h->workspace_bytes - g.ws_off : 0;
    if (tiles < h->num_sms && g.K >= 128 && g.batch.red_count == 1) {
        long long want = (2ll * h->num_sms + tiles - 1) / tiles;
        const long long max_by_k = g.K / 64;
        if (want > max_by_k) want = max_by_k;
        if (want > 64) want = 64;
        bool chosen = false;
        if (want >= 2 && want <= 2 * h->max_cluster) {
            int sp = 2;
            while (sp * 2 <= want && sp * 2 <= h->max_cluster) sp *= 2;
            const int ks = ((g.K + sp - 1) / sp + generic::BK - 1) / generic::BK * generic::BK;
            const size_t need = static_cast<size_t>(tiles) * sp * generic::BM * generic::BN * sizeof(float);
            if ((g.K + ks - 1) / ks == sp && (h->variant != 8 || need <= ws_avail)) {   // no empty range
                splits = sp;
                kspan = ks;
                cluster = h->variant != 8;     // variant 8: the same ranges, added through the workspace
                chosen = true;
            }
        }
        if (!chosen) {
            kspan = g.K;
            const size_t per_split = static_cast<size_t>(tiles) * generic::BM * generic::BN * sizeof(float);
            if (per_split > 0 && want * per_split > ws_avail) want = static_cast<long long>(ws_avail / per_split);
            if (want >= 2 && g.K >= 512) {
                kspan = static_cast<int>((g.K + want - 1) / want);
                kspan = ((kspan + generic::BK - 1) / generic::BK) * generic::BK;
                splits = (g.K + kspan - 1) / kspan;
            }
        }
    }
    p.splits = splits;
    p.kspan = kspan;
    p.partial = reinterpret_cast<float*>(h->workspace + g.ws_off);
    p.c_vec_ok = aligned16(g.c) && (g.N % 4 == 0);
    p.shape.work = tiles * splits;
    fill_batch_desc(g.batch, p.batch);
    p.epi = g.epi;
    p.aMs = g.aMs; p.aKs = g.aKs; p.bKs = g.bKs; p.bNs = g.bNs;
    if (cluster) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(static_cast<unsigned int>(p.shape.work), 1, 1);
        cfg.blockDim = dim3(generic::THREADS, 1, 1);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned int>(splits);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t le = cudaLaunchKernelEx(&cfg, generic::gemm_generic_kernel<true>, p);
        if (le != cudaSuccess) return cuda_fail(h, le, "generic gemm cluster launch");
        h->stats.launches++;
        h->stats.splitk++;
        h->stats.generic++;
        return TT_OK;
    }
    const long long max_grid = static_cast<long long>(h->num_sms) * 8;
    const int grid = static_cast<int>(p.shape.work < max_grid ? p.shape.work : max_grid);
    generic::gemm_generic_kernel<false><<<grid, generic::THREADS, 0, st>>>(p);
    h->stats.launches++;
    if (splits > 1) {
        const long long threads = tiles * (generic::BM * generic::BN / 4);
        generic::generic_reduce_kernel<<<static_cast<unsigned int>((threads + 255) / 256), 256, 0, st>>>(
            p.partial, g.c, p.shape, g.epi, splits, p.c_vec_ok);
        h->stats.launches++;
        h->stats.splitk++;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "generic gemm launch");
    h->stats.generic++;
    return TT_OK;
}

template <int TM, bool AK, bool BK_, int NJ = 2>
int launch_simt_t(tt_handle_t h, cudaStream_t st, const CUtensorMap& ma, const CUtensorMap& mb,
                  const simt::Params& p, int grid, int mode)
{
    constexpr int smem = simt::Cfg<TM, AK, BK_, NJ>::SMEM_BYTES;
    if (mode == simt::MODE_STREAMK)
        simt::sgemm_simt_kernel<TM, AK, BK_, simt::MODE_STREAMK, NJ><<<grid, simt::THREADS, smem, st>>>(ma, mb, p);
    else if (TM == 8 && NJ == 2 && mode == simt::MODE_SPLITK)   // split-K exists for the 128x128 tile only
        simt::sgemm_simt_kernel<8, AK, BK_, simt::MODE_SPLITK><<<grid, simt::THREADS, smem, st>>>(ma, mb, p);
    else
        simt::sgemm_simt_kernel<TM, AK, BK_, simt::MODE_TILES, NJ><<<grid, simt::THREADS, smem, st>>>(ma, mb, p);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "simt gemm launch");
    return TT_OK;
}

// Tile and split-K choice for the FMA kernel.  256x128 tiles (16x8 per thread) run at
// about 76 % of the FMA peak, 128x128 tiles (8x8 per thread) at about 70 %, but small
// grids quantise badly on 148 SMs; cutting K into `splits` ranges (partials reduced in a
// fixed order by the last CTA of each tile) fills the machine for small M x N.  The model
// is time ~ waves x (k-tiles per split + fixed per-item overhead) x per-tile cost, and the
// choice depends on the shape and the SM count only.
struct SimtPlan {
    int tm;
    int splits;
    int kps;
    bool streamk = false;   // deal tiles x k-tiles units evenly to the CTAs (partial last wave)
    int nj = 2;             // tile width / 64: 2 = 128 columns, 3 = 192 columns (128-row tiles, MN-major B)
};

SimtPlan plan_simt(const tt_handle_t h, int M, int N, int K, int batch, size_t ws_avail, int red_count, bool b_kmajor)
{
    const int k_tiles = (K + simt::BK - 1) / simt::BK;
    if (red_count > 1) ws_avail = 0;  // a reduced batch axis already lengthens the k loop: no split-K
    SimtPlan best{16, 1, k_tiles};
    double best_t = 1e300;
    // (rows per thread, tile width / 64): cost per tile relative to a 128x128 tile at full FMA rate,
    // over the fraction of that rate the shape reaches (16x8 per thread 0.80, 8x12 0.76, 8x8 0.73)
    struct Shape { int tm, nj; double cost; };
    const Shape shapes[3] = {{16, 2, 2.0 / 0.80}, {8, 2, 1.0 / 0.73}, {8, 3, 1.5 / 0.76}};
    for (const Shape& sh : shapes) {
        const int tm = sh.tm, bm = 16 * tm, bn = 64 * sh.nj;
        if (sh.nj == 3 && b_kmajor) continue;          // the 192-column tile reads MN-major B only
        const long long tiles = static_cast<long long>(batch) * ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
        const double tile_cost = sh.cost;
        for (int splits = 1; splits <= 32; splits++) {
            const int kps = (k_tiles + splits - 1) / splits;
            const int real = (k_tiles + kps - 1) / kps;
            if (real != splits) continue;              // skip counts that leave empty ranges
            if (splits > 1) {
                if (tm != 8 || sh.nj != 2) break;      // split-K exists for the 128x128 tile only
                if (kps < 1) break;
                const size_t need = static_cast<size_t>(tiles) * splits * bm * bn * sizeof(float);
                if (need > ws_avail) break;
            }
            const long long work = tiles * splits;
            const long long waves = (work + h->num_sms - 1) / h->num_sms;
            // per work item: kps k-tiles + ~2 k-tiles worth of pipeline fill / epilogue; the
            // reduction kernel costs about as much as two more k-tiles of a 128x128 tile
            const double t = static_cast<double>(waves) * (static_cast<double>(kps) * red_count + 2.0) * tile_cost +
                             (splits > 1 ? 2.0 / 0.70 : 0.0);
            if (t < best_t) { best_t = t; best = SimtPlan{tm, splits, kps, false, sh.nj}; }
        }
        // stream-K: no wave quantisation (work / SMs tile-times); needs one partial-tile slot
        // per CTA and enough k-tiles for the ranges to be worth cutting.  Less than one wave of
        // 128x128 tiles may be cut over up to four CTAs per tile (a partial tile of that shape
        // is half the traffic of a 256x128 one).
        const bool sub_wave = tm == 8 && sh.nj == 2 && tiles < h->num_sms;
        if (red_count == 1 && k_tiles >= 8 && tiles >= h->num_sms / (sub_wave ? 4 : 2)) {
            const size_t need = 2 * static_cast<size_t>(h->num_sms) * bm * bn * sizeof(float);   // two partial-tile slots per CTA
            const long long waves = (tiles + h->num_sms - 1) / h->num_sms;
            const double fill = static_cast<double>(tiles) / (static_cast<double>(waves) * h->num_sms);
            // A remainder of at most half a wave behind whole waves is cut into k-aligned equal
            // ranges (try_launch_simt_tm): whole + 1 / split waves, locality of a whole-tile wave.
            const long long whole = tiles / h->num_sms, rest = tiles - whole * h->num_sms;
            if (need <= ws_avail && whole >= 1 && rest > 0 && rest * 2 <= h->num_sms && k_tiles >= 2 * (h->num_sms / rest)) {
                const double split = static_cast<double>(h->num_sms / rest);
                // (the cost of the partial tiles scales with their size: 11 units for 256 x 128)
                const double t = (static_cast<double>(whole) + 1.0 / split) * (k_tiles + 2.0) * tile_cost +
                                 11.0 * (bm * bn) / (256.0 * 128.0);
                if (t < best_t) { best_t = t; best = SimtPlan{tm, 1, k_tiles, true, sh.nj}; }
            } else if (need <= ws_avail && fill < 0.97) {
                // measured: storing and re-reading the partial tiles costs about 20 us (11 units of a
                // 128x128 k-tile) whatever the shape, and the stream-K form of the kernel runs its
                // main loop about 4 % slower than the whole-tile form (16384^3: 145.1 ms against
                // 141.1 ms although it saves 0.65 of a wave; 4096^3, 3.46 waves: 2.30 against 2.55 ms).
                // Below one wave of 128x128 tiles: 2.5 units plus 1.5 per CTA that shares a tile
                // (1024^3: 50 us against 54 with two split-K ranges, 1024 x 1024 x 4096: 155 against
                // 175, 768^3: 31 against 27).
                const double body = (static_cast<double>(tiles) / h->num_sms) * (k_tiles + 2.0) * tile_cost;
                const double t = sub_wave ? body + 2.5 + 1.5 * h->num_sms / static_cast<double>(tiles)
                                          : (body + 11.0) * 1.05;
                if (t < best_t) { best_t = t; best = SimtPlan{tm, 1, k_tiles, true, sh.nj}; }
            }
        }
    }
    return best;
}

// Returns TT_ERR_UNSUPPORTED (without touching h->err) when the operands cannot be
// expressed as TMA descriptors; the caller then uses the any-stride kernel.
template <int TM, int NJ = 2>
int try_launch_simt_tm(tt_handle_t h, cudaStream_t st, const GemmCall& g, const SimtPlan& plan)
{
    constexpr int BM = 16 * TM, BN = 64 * NJ;
    OperandView va, vb;
    const int ak = operand_view(g.a, g.M, g.K, g.aMs, g.aKs, va);
    const int bk = operand_view(g.b, g.N, g.K, g.bNs, g.bKs, vb);
    if (ak < 0 || bk < 0) return TT_ERR_UNSUPPORTED;
    simt::Params p;
    memset(&p, 0, sizeof(p));
    fill_batch_desc(g.batch, p.batch);
    if (!plan_tma_batch(g.batch, g.batch.as, p.batch.a_slot, p.batch.a_mult, va, g.batch.red_as, &p.batch.red_a_slot)) return TT_ERR_UNSUPPORTED;
    if (!plan_tma_batch(g.batch, g.batch.bs, p.batch.b_slot, p.batch.b_mult, vb, g.batch.red_bs, &p.batch.red_b_slot)) return TT_ERR_UNSUPPORTED;
    if (!tma_compatible(va) || !tma_compatible(vb)) return TT_ERR_UNSUPPORTED;

    CUtensorMap ma, mb;
    int r = ak ? encode_tensor_map(&ma, va, simt::BK, BM, Swizzle::B128)
               : encode_tensor_map(&ma, va, BM, simt::BK, Swizzle::None);
    if (r != 0) return TT_ERR_UNSUPPORTED;
    r = bk ? encode_tensor_map(&mb, vb, simt::BK, BN, Swizzle::B128)
           : encode_tensor_map(&mb, vb, BN, simt::BK, Swizzle::None);
    if (r != 0) return TT_ERR_UNSUPPORTED;

    p.shape.M = g.M; p.shape.N = g.N; p.shape.K = g.K;
    p.shape.tiles_m = (g.M + BM - 1) / BM;
    p.shape.tiles_n = (g.N + BN - 1) / BN;
    p.shape.batch = g.batch_count;
    p.splits = plan.splits;
    p.kps = plan.kps;
    p.partial = reinterpret_cast<float*>(h->workspace + g.ws_off);
    const long long tiles = static_cast<long long>(g.batch_count) * p.shape.tiles_m * p.shape.tiles_n;
    const int k_tiles = (g.K + simt::BK - 1) / simt::BK;
    const int mode = plan.streamk ? simt::MODE_STREAMK : plan.splits > 1 ? simt::MODE_SPLITK : simt::MODE_TILES;
    // work = what the CTAs share out: tiles x splits items, or for stream-K the k-tile units of the
    // tiles behind the whole waves.  The whole waves stop one wave early when the remainder is
    // less than half a wave, so the unit part holds between half a tile and a tile and a half per
    // CTA (an output tile is then shared by three CTAs at most).
    p.sk_first = 0;
    p.sk_split = 0;
    if (plan.streamk && tiles >= h->num_sms) {
        long long whole = tiles / h->num_sms;
        const long long rest = tiles - whole * h->num_sms;
        if (rest > 0 && rest * 2 <= h->num_sms && k_tiles >= 2 * (h->num_sms / rest)) {
            // at most half a wave left: every remaining tile is cut into equal k ranges, one per
            // CTA, so the CTAs stay aligned in k (and share operand panels in L2 like a whole wave)
            p.sk_split = static_cast<int>(h->num_sms / rest);
        } else if (rest < h->num_sms / 2) {
            whole -= 1;
        }
        p.sk_first = whole * h->num_sms;
    }
    p.shape.work = plan.streamk ? (tiles - p.sk_first) * k_tiles : tiles * plan.splits;
    if (plan.streamk && p.shape.work >= (1ll << 31)) return TT_ERR_UNSUPPORTED;   // the kernel's unit cursor is 32 bits
    p.epi = g.epi;
    p.c = g.c;
    p.status = h->status;
    p.sk_flags = h->status + STREAMK_FLAGS_WORD;
    p.c_vec_ok = aligned16(g.c) && (g.N % 4 == 0);
    const int grid = static_cast<int>(p.shape.work < h->num_sms && p.sk_first == 0 ? p.shape.work : h->num_sms);
    if (plan.splits > 1 || plan.streamk) h->stats.splitk++;
    int rc;
    if constexpr (NJ == 3) {
        if (bk) return TT_ERR_UNSUPPORTED;             // planned for MN-major B only
        if (ak) rc = launch_simt_t<8, true, false, 3>(h, st, ma, mb, p, grid, mode);
        else rc = launch_simt_t<8, false, false, 3>(h, st, ma, mb, p, grid, mode);
    } else {
        if (ak && bk) rc = launch_simt_t<TM, true, true>(h, st, ma, mb, p, grid, mode);
        else if (ak && !bk) rc = launch_simt_t<TM, true, false>(h, st, ma, mb, p, grid, mode);
        else if (!ak && !bk) rc = launch_simt_t<TM, false, false>(h, st, ma, mb, p, grid, mode);
        else rc = launch_simt_t<TM, false, true>(h, st, ma, mb, p, grid, mode);
    }
    if (rc != TT_OK) return rc;
    h->stats.launches++;
    h->stats.simt_tma++;
    if (plan.splits > 1) {
        const long long threads = static_cast<long long>(g.batch_count) * p.shape.tiles_m * p.shape.tiles_n * (BM * BN / 4);
        simt::splitk_reduce_kernel<BM><<<static_cast<unsigned int>((threads + 255) / 256), 256, 0, st>>>(
            p.partial, g.c, p.shape, g.epi, plan.splits, p.c_vec_ok);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(h, e, "split-K reduce launch");
        h->stats.launches++;
    }
    return TT_OK;
}

// Pre-transposition of large K-major operands.  The FMA kernel reads MN-major tiles straight
// from the TMA stage but has to transpose K-major tiles through shared memory on every k-tile:
// that costs a CTA barrier per k-tile and the shared memory of a ring stage (3 stages instead of
// 4), 5 to 18 % of the run time depending on the shape (1024 x 4096 x 4096 with K-major B: 669 us
// against 566 us with MN-major B).  One streaming transposition into the workspace costs 8 bytes
// of traffic per operand element, which is far less once the other dimension reaches a few
// hundred: gain / cost is about N / 440 for A (M x K) and M / 440 for B (N x K).  The sums are the
// same sums in the same order, so the bits of C do not change.
constexpr int PRE_T_MIN_N_FOR_A = 512, PRE_T_MIN_M_FOR_B = 512;
constexpr long long PRE_T_MIN_ELEMS = 1ll << 19;
constexpr size_t PRE_T_RESERVE = 64ull << 20;   // kept free behind the copies (stream-K partial tiles)

bool pre_transpose(tt_handle_t h, cudaStream_t st, const float*& base, int rows, int K, int& row_stride,
                   int& k_stride, size_t& ws_off)
{
    if (k_stride != 1 || rows < 2 || K < 2 || rows % 4 != 0 || K % 4 != 0 || row_stride % 4 != 0 ||
        row_stride < K || !aligned16(base) || static_cast<long long>(rows) * K < PRE_T_MIN_ELEMS)
        return false;
    const size_t bytes = (sizeof(float) * static_cast<size_t>(rows) * K + 255) & ~static_cast<size_t>(255);
    if (ws_off + bytes + PRE_T_RESERVE > h->workspace_bytes) return false;
    float* dst = reinterpret_cast<float*>(h->workspace + ws_off);
    const dim3 grid((K + 63) / 64, (rows + 63) / 64);
    ew::transpose_kernel<<<grid, 256, 0, st>>>(base, dst, rows, K, row_stride, rows);
    h->stats.launches++;
    base = dst;
    row_stride = 1;
    k_stride = rows;
    ws_off += bytes;
    return true;
}

int try_launch_simt(tt_handle_t h, cudaStream_t st, const GemmCall& g_in)
{
    GemmCall g = g_in;
    if (h->variant == 0 && g.batch_count == 1 && g.batch.red_count == 1) {
        if (g.N >= PRE_T_MIN_N_FOR_A) pre_transpose(h, st, g.a, g.M, g.K, g.aMs, g.aKs, g.ws_off);
        if (g.M >= PRE_T_MIN_M_FOR_B) pre_transpose(h, st, g.b, g.N, g.K, g.bNs, g.bKs, g.ws_off);
    } else if (h->variant == 0 && g.batch.red_count == 1) {
        // Batched: an operand whose batch entries lie one after the other as ONE dense K-major
        // matrix (a single non-broadcast batch axis of stride rows x K) is transposed as that
        // matrix; its entries then sit side by side along the row axis of the copy.  What the
        // copy is weighed against is the number of columns (rows) every operand entry meets
        // over the whole call, i.e. N (M) times the entries of the other operand it is
        // broadcast against.
        const auto stacked = [&](const float*& base, int rows, int& row_stride, int& k_stride, int* bstride,
                                 int other_extent, int min_other) {
            int ax = -1;
            for (int i = 0; i < g.batch.rank; i++) {
                if (bstride[i] == 0) continue;
                if (ax >= 0) return;                   // more than one batch axis: leave it
                ax = i;
            }
            if (ax < 0 || k_stride != 1 || row_stride != g.K || rows % 4 != 0 ||
                static_cast<long long>(bstride[ax]) != static_cast<long long>(rows) * g.K)
                return;
            const long long total_rows = static_cast<long long>(rows) * g.batch.dims[ax];
            const long long other_total = static_cast<long long>(other_extent) * (g.batch_count / g.batch.dims[ax]);
            if (total_rows > (1ll << 30) || other_total < min_other) return;
            if (pre_transpose(h, st, base, static_cast<int>(total_rows), g.K, row_stride, k_stride, g.ws_off))
                bstride[ax] = rows;                    // entries are `rows` columns apart in the [K][total rows] copy
        };
        stacked(g.a, g.M, g.aMs, g.aKs, g.batch.as, g.N, PRE_T_MIN_N_FOR_A);
        stacked(g.b, g.N, g.bNs, g.bKs, g.batch.bs, g.M, PRE_T_MIN_M_FOR_B);
    }
    const size_t ws_avail = h->workspace_bytes > g.ws_off ? h->workspace_bytes - g.ws_off : 0;
    const bool b_kmajor = g.bKs == 1 || g.K == 1;      // as operand_view classifies it
    SimtPlan plan = plan_simt(h, g.M, g.N, g.K, g.batch_count, ws_avail, g.batch.red_count, b_kmajor);
    if (h->variant == 2 || h->variant == 3 || h->variant == 7) {
        // pinned tile shape (A/B measurements and tests): no split-K
        plan.tm = h->variant == 2 ? 16 : 8;
        plan.nj = h->variant == 7 ? 3 : 2;
        plan.splits = 1;
        plan.kps = (g.K + simt::BK - 1) / simt::BK;
        plan.streamk = false;
        if (plan.nj == 3 && b_kmajor) return TT_ERR_UNSUPPORTED;
    }
    if (h->variant == 6 || g.epi.scatter_rows > 0) {
        // pinned: 256x128 tiles with stream-K (measurements; the scatter epilogue lives in this form)
        plan.tm = 16; plan.nj = 2; plan.splits = 1; plan.kps = (g.K + simt::BK - 1) / simt::BK; plan.streamk = true;
        if (2 * static_cast<size_t>(h->num_sms) * 256 * simt::BN * sizeof(float) > ws_avail) return TT_ERR_UNSUPPORTED;
    }
    if (h->variant == 9) {
        // pinned: 128x128 tiles with stream-K (measurements)
        plan.tm = 8; plan.nj = 2; plan.splits = 1; plan.kps = (g.K + simt::BK - 1) / simt::BK; plan.streamk = true;
        if (2 * static_cast<size_t>(h->num_sms) * 128 * simt::BN * sizeof(float) > ws_avail) return TT_ERR_UNSUPPORTED;
    }
    if (plan.nj == 3) return try_launch_simt_tm<8, 3>(h, st, g, plan);
    return plan.tm == 16 ? try_launch_simt_tm<16>(h, st, g, plan) : try_launch_simt_tm<8>(h, st, g, plan);
}

// Products with one tiny dimension: HBM-bound streaming kernels (skinny.cuh).  Returns
// TT_ERR_UNSUPPORTED when the call is not one of the handled forms.
int try_launch_skinny(tt_handle_t h, cudaStream_t st, const GemmCall& g)
{
    if (g.batch_count != 1 || g.batch.red_count != 1 || g.K <= 0) return TT_ERR_UNSUPPORTED;
    const bool bias_ok = !g.epi.bias || aligned16(g.epi.bias);
    const size_t ws_avail = h->workspace_bytes > g.ws_off ? h->workspace_bytes - g.ws_off : 0;
    // (in every math mode: the tensor-core kernel takes 52 us for 8192 x 10 x 4096 and 40 us for
    // 1024 x 10 x 4096, these forms 41 and 17 us, in strict FP32 arithmetic)
    if (g.N <= skinny::MAXD && g.M >= 64 && g.K >= 128 && g.aKs == 1 && g.bKs == 1 && g.K % 4 == 0 &&
        g.aMs % 4 == 0 && (g.N == 1 || g.bNs % 4 == 0) && aligned16(g.a) && aligned16(g.b)) {
        // 8 rows per CTA while the accumulators fit comfortably; 4 rows for N > 8 (8 x 12 and
        // 8 x 16 accumulators run slower: 105 vs 88 us at 8192 x 10 x 4096)
        // Tall products (half a wave of 56-row units or more): the TMA-fed stream, a persistent CTA
        // per SM.  Variant 10 keeps the K-cut form below for comparison.
        const int units = (g.M + skinny::stream::RB - 1) / skinny::stream::RB;
        if (h->variant != 10 && units >= h->num_sms / 2) {
            OperandView va, vb;
            CUtensorMap ma, mb;
            const int nt = g.N <= 4 ? 4 : g.N <= 8 ? 8 : g.N <= 12 ? 12 : 16;
            if (operand_view(g.a, g.M, g.K, g.aMs, 1, va) == 1 && operand_view(g.b, g.N, g.K, g.bNs, 1, vb) == 1 &&
                tma_compatible(va) && tma_compatible(vb) &&
                encode_tensor_map(&ma, va, skinny::stream::KC, skinny::stream::RB, Swizzle::None) == 0 &&
                encode_tensor_map(&mb, vb, skinny::stream::KC, nt, Swizzle::None) == 0) {
                const int grid = units < h->num_sms ? units : h->num_sms;
                const unsigned int th = skinny::stream::THREADS;
                if (nt == 4)       skinny::skinny_n_stream_kernel<4><<<grid, th, skinny::stream::Cfg<4>::SMEM_BYTES, st>>>(ma, mb, g.c, g.M, g.N, g.K, g.epi, h->status);
                else if (nt == 8)  skinny::skinny_n_stream_kernel<8><<<grid, th, skinny::stream::Cfg<8>::SMEM_BYTES, st>>>(ma, mb, g.c, g.M, g.N, g.K, g.epi, h->status);
                else if (nt == 12) skinny::skinny_n_stream_kernel<12><<<grid, th, skinny::stream::Cfg<12>::SMEM_BYTES, st>>>(ma, mb, g.c, g.M, g.N, g.K, g.epi, h->status);
                else               skinny::skinny_n_stream_kernel<16><<<grid, th, skinny::stream::Cfg<16>::SMEM_BYTES, st>>>(ma, mb, g.c, g.M, g.N, g.K, g.epi, h->status);
                h->stats.launches++;
                const cudaError_t e = cudaGetLastError();
                if (e != cudaSuccess) return cuda_fail(h, e, "skinny stream launch");
                h->stats.skinny++;
                return TT_OK;
            }
        }
        const int rows = g.N <= 8 ? 8 : 4;
        const unsigned int blocks = static_cast<unsigned int>((g.M + rows - 1) / rows);   // one CTA per row group
        if (g.N <= 4)
            skinny::skinny_n_kernel<8, 4><<<blocks, 256, 0, st>>>(g.a, g.b, g.c, g.M, g.N, g.K, g.aMs, g.bNs, g.epi);
        else if (g.N <= 8)
            skinny::skinny_n_kernel<8, 8><<<blocks, 256, 0, st>>>(g.a, g.b, g.c, g.M, g.N, g.K, g.aMs, g.bNs, g.epi);
        else
            skinny::skinny_n_kernel<4, 16><<<blocks, 256, 0, st>>>(g.a, g.b, g.c, g.M, g.N, g.K, g.aMs, g.bNs, g.epi);
        h->stats.launches++;
    } else if (g.M <= skinny::MAXD && g.N >= 256 && g.K >= 256 && g.bNs == 1 && g.N % 4 == 0 &&
               g.bKs % 4 == 0 && aligned16(g.b) && aligned16(g.c) && bias_ok) {
        const int gx = (g.N / 4 + 63) / 64;
        if (h->variant != 10) {
            // TMA-fed form: one CTA per SM (its ring and operand slice fill the shared memory), so
            // the k ranges are sized for a single wave, and capped by what the slice buffer holds
            namespace ms = skinny::mstream;
            OperandView vb;
            CUtensorMap mb;
            const long long r0 = h->num_sms / gx > 0 ? h->num_sms / gx : 1;
            int kspan = static_cast<int>((g.K + r0 - 1) / r0);
            kspan = (kspan + ms::KT - 1) / ms::KT * ms::KT;
            const int mt = g.M <= 4 ? 4 : g.M <= 8 ? 8 : g.M <= 12 ? 12 : 16;
            const int ks_max = ms::A_FLOATS / mt / ms::KT * ms::KT;
            if (kspan > ks_max) kspan = ks_max;
            const int n_ranges = (g.K + kspan - 1) / kspan;
            const size_t need = n_ranges > 1 ? sizeof(float) * static_cast<size_t>(n_ranges) * g.M * g.N : 0;
            if (need <= ws_avail && operand_view(g.b, g.K, g.N, g.bKs, 1, vb) == 1 && tma_compatible(vb) &&
                encode_tensor_map(&mb, vb, ms::NW, ms::KT, Swizzle::None) == 0) {
                float* partial = reinterpret_cast<float*>(h->workspace + g.ws_off);
                float* dst = n_ranges == 1 ? g.c : partial;
                const int direct = n_ranges == 1 ? 1 : 0;
                const dim3 grid(gx, n_ranges);
                if (mt == 4)       skinny::skinny_m_stream_kernel<4><<<grid, ms::THREADS, ms::SMEM_BYTES, st>>>(mb, g.a, dst, g.M, g.N, g.K, g.aMs, g.aKs, kspan, g.epi, direct, h->status);
                else if (mt == 8)  skinny::skinny_m_stream_kernel<8><<<grid, ms::THREADS, ms::SMEM_BYTES, st>>>(mb, g.a, dst, g.M, g.N, g.K, g.aMs, g.aKs, kspan, g.epi, direct, h->status);
                else if (mt == 12) skinny::skinny_m_stream_kernel<12><<<grid, ms::THREADS, ms::SMEM_BYTES, st>>>(mb, g.a, dst, g.M, g.N, g.K, g.aMs, g.aKs, kspan, g.epi, direct, h->status);
                else               skinny::skinny_m_stream_kernel<16><<<grid, ms::THREADS, ms::SMEM_BYTES, st>>>(mb, g.a, dst, g.M, g.N, g.K, g.aMs, g.aKs, kspan, g.epi, direct, h->status);
                h->stats.launches++;
                if (n_ranges > 1) {
                    const long long count4 = static_cast<long long>(g.M) * g.N / 4;
                    skinny::skinny_reduce_kernel<<<static_cast<unsigned int>((count4 + 255) / 256), 256, 0, st>>>(
                        partial, g.c, count4, g.N, n_ranges, static_cast<long long>(g.M) * g.N, g.epi);
                    h->stats.launches++;
                    h->stats.splitk++;
                }
                const cudaError_t e = cudaGetLastError();
                if (e != cudaSuccess) return cuda_fail(h, e, "skinny stream launch");
                h->stats.skinny++;
                return TT_OK;
            }
        }
        long long ranges = (4ll * h->num_sms + gx - 1) / gx;
        if (ranges > g.K / 64) ranges = g.K / 64;
        const size_t per_range = sizeof(float) * static_cast<size_t>(g.M) * g.N;
        if (ranges > 1 && ranges * per_range > ws_avail) ranges = static_cast<long long>(ws_avail / per_range);
        if (ranges < 1) ranges = 1;
        int kspan = static_cast<int>((g.K + ranges - 1) / ranges);
        kspan = (kspan + 3) & ~3;
        const int n_ranges = (g.K + kspan - 1) / kspan;
        float* partial = reinterpret_cast<float*>(h->workspace + g.ws_off);
        skinny::skinny_m_kernel<<<dim3(gx, n_ranges), 256, 0, st>>>(
            g.a, g.b, n_ranges == 1 ? g.c : partial, g.M, g.N, g.K, g.aMs, g.aKs, g.bKs, kspan, g.epi,
            n_ranges == 1 ? 1 : 0);
        h->stats.launches++;
        if (n_ranges > 1) {
            const long long count4 = static_cast<long long>(g.M) * g.N / 4;
            skinny::skinny_reduce_kernel<<<static_cast<unsigned int>((count4 + 255) / 256), 256, 0, st>>>(
                partial, g.c, count4, g.N, n_ranges, static_cast<long long>(g.M) * g.N, g.epi);
            h->stats.launches++;
            h->stats.splitk++;
        }
    } else if (h->variant != 10 && g.K <= skinny::MAXD && g.M >= 64 && g.N >= 256 && g.bNs == 1 && g.N % 4 == 0 &&
               g.bKs % 4 == 0 && aligned16(g.b) && aligned16(g.c) && bias_ok) {
        // tiny K (the dX of a narrow layer): bound by the write of C
        const dim3 grid((g.N + skinny::SK_COLS - 1) / skinny::SK_COLS, (g.M + skinny::SK_ROWS - 1) / skinny::SK_ROWS);
        if (grid.y > 65535u) return TT_ERR_UNSUPPORTED;
        if (g.K <= 4)       skinny::skinny_k_kernel<1><<<grid, 256, 0, st>>>(g.a, g.b, g.c, g.M, g.N, g.K, g.aMs, g.aKs, g.bKs, g.epi);
        else if (g.K <= 8)  skinny::skinny_k_kernel<2><<<grid, 256, 0, st>>>(g.a, g.b, g.c, g.M, g.N, g.K, g.aMs, g.aKs, g.bKs, g.epi);
        else if (g.K <= 12) skinny::skinny_k_kernel<3><<<grid, 256, 0, st>>>(g.a, g.b, g.c, g.M, g.N, g.K, g.aMs, g.aKs, g.bKs, g.epi);
        else                skinny::skinny_k_kernel<4><<<grid, 256, 0, st>>>(g.a, g.b, g.c, g.M, g.N, g.K, g.aMs, g.aKs, g.bKs, g.epi);
        h->stats.launches++;
    } else {
        return TT_ERR_UNSUPPORTED;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "skinny gemm launch");
    h->stats.skinny++;
    return TT_OK;
}

int run_gemm(tt_handle_t h, cudaStream_t st, const GemmCall& g)
{
    if (g.M == 0 || g.N == 0 || g.batch_count == 0) return TT_OK;
    if (g.K == 0 && !g.epi.bias && g.epi.act == TT_ACT_NONE) {
        const cudaError_t e = cudaMemsetAsync(
            g.c, 0, sizeof(float) * static_cast<size_t>(g.batch_count) * g.M * g.N, st);
        if (e != cudaSuccess) return cuda_fail(h, e, "memset C");
        return TT_OK;
    }
    if (g.epi.scatter_rows > 0) {
        // Row-block scatter: only the tensor-core kernel and the stream-K FMA kernel store
        // through the scatter table; anything else is the caller's fallback (local + copy).
        if (g.K == 0 || g.batch_count != 1 || g.batch.red_count != 1 || h->variant == 1 || h->variant == 8 ||
            g.epi.scatter_rows % 256 != 0)
            return TT_ERR_UNSUPPORTED;
        if (h->math_mode != TT_MATH_FP32) {
            int n_launch = 0;
            const int rc = tf32::try_launch(h->math_mode, st, g.a, g.b, g.c, g.M, g.N, g.K, g.aMs,
                                            g.aKs, g.bKs, g.bNs, g.batch_count, g.batch.rank,
                                            g.batch.dims, g.batch.as, g.batch.bs, g.epi, h->num_sms,
                                            h->status, h->workspace + g.ws_off,
                                            h->workspace_bytes > g.ws_off ? h->workspace_bytes - g.ws_off : 0, &n_launch,
                                            h->variant == 4 ? 1 : h->variant == 5 ? 2 : 0);
            if (rc == TT_OK) { h->stats.launches += n_launch; h->stats.tcgen05++; return TT_OK; }
            if (rc != TT_ERR_UNSUPPORTED) return fail(h, rc, "tcgen05 gemm launch failed");
        }
        return try_launch_simt(h, st, g);
    }
    const long long vol = static_cast<long long>(g.M) * g.N * (g.K > 0 ? g.K : 1);
    if (g.K > 0 && (h->variant == 0 || h->variant == 10)) {
        // one tiny dimension: stream the large operand once, in every math mode (strict FP32
        // arithmetic, so at least as accurate as the mode asks for)
        const int rc = try_launch_skinny(h, st, g);
        if (rc != TT_ERR_UNSUPPORTED) return rc;
    }
    if (g.K > 0 && h->variant != 1 && h->variant != 8) {
        // 3xTF32 on a small single product: its two operand-split launches in front of the GEMM cost
        // more than the strict-FP32 kernels need for the whole product (512^3: 22.6 us against
        // 18.5 us), and strict FP32 is at least as accurate as the mode asks for.
        const bool small_3x = h->math_mode == TT_MATH_3XTF32 && h->variant == 0 && g.batch_count == 1 &&
                              vol <= SMALL_3XTF32_MAX_ELEMS;
        if (h->math_mode != TT_MATH_FP32 && g.batch.red_count == 1 && !small_3x) {  // the tensor-core kernel has no reduced axis
            int n_launch = 0;
            const int rc = tf32::try_launch(h->math_mode, st, g.a, g.b, g.c, g.M, g.N, g.K, g.aMs,
                                            g.aKs, g.bKs, g.bNs, g.batch_count, g.batch.rank,
                                            g.batch.dims, g.batch.as, g.batch.bs, g.epi, h->num_sms,
                                            h->status, h->workspace + g.ws_off,
                                            h->workspace_bytes > g.ws_off ? h->workspace_bytes - g.ws_off : 0, &n_launch,
                                            h->variant == 4 ? 1 : h->variant == 5 ? 2 : 0);
            if (rc == TT_OK) { h->stats.launches += n_launch; h->stats.tcgen05++; return TT_OK; }
            if (rc != TT_ERR_UNSUPPORTED) return fail(h, rc, "tcgen05 gemm launch failed");
        }
        // A small output with little work in total (benchmark config 1, the GEMMs of the small
        // networks) is latency-bound: the any-stride kernel serves it in ONE launch, K cut across
        // the CTAs of a cluster, where the TMA-fed kernel would need a second launch to add its
        // partial tiles.
        const long long tiles64 = static_cast<long long>(g.batch_count) * ((g.M + 63) / 64) * ((g.N + 63) / 64);
        const bool small_output = h->variant == 0 && g.batch.red_count == 1 && tiles64 <= h->num_sms / 2 &&
                                  vol <= SMALL_MAX_FLOP_ELEMS;
        if (!small_output &&
            (h->variant == 2 || h->variant == 3 || h->variant == 6 || h->variant == 7 || h->variant == 9 ||
             vol >= TMA_MIN_FLOP_ELEMS)) {
            const int rc = try_launch_simt(h, st, g);
            if (rc != TT_ERR_UNSUPPORTED) return rc;
        }
    }
    return launch_generic(h, st, g);
}

bool g_generic_cluster16 = false;

// Per-device kernel attributes, set once at handle creation so that no compute call
// does lazy set-up work (which could not be captured into a graph).
template <int TM, bool AK, bool BK_>
cudaError_t init_simt_one()
{
    const int bytes = simt::Cfg<TM, AK, BK_>::SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(simt::sgemm_simt_kernel<TM, AK, BK_, simt::MODE_TILES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(simt::sgemm_simt_kernel<TM, AK, BK_, simt::MODE_STREAMK>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess || TM != 8) return e;
    return cudaFuncSetAttribute(simt::sgemm_simt_kernel<8, AK, BK_, simt::MODE_SPLITK>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <int TM>
cudaError_t init_simt_tm()
{
    cudaError_t e;
    if ((e = init_simt_one<TM, true, true>()) != cudaSuccess) return e;
    if ((e = init_simt_one<TM, true, false>()) != cudaSuccess) return e;
    if ((e = init_simt_one<TM, false, true>()) != cudaSuccess) return e;
    return init_simt_one<TM, false, false>();
}

template <bool AK>
cudaError_t init_simt_wide()
{
    const int bytes = simt::Cfg<8, AK, false, 3>::SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(simt::sgemm_simt_kernel<8, AK, false, simt::MODE_TILES, 3>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(simt::sgemm_simt_kernel<8, AK, false, simt::MODE_STREAMK, 3>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

cudaError_t init_kernels()
{
    cudaError_t e = init_simt_tm<8>();
    if (e != cudaSuccess) return e;
    e = init_simt_tm<16>();
    if (e != cudaSuccess) return e;
    if ((e = init_simt_wide<true>()) != cudaSuccess) return e;
    if ((e = init_simt_wide<false>()) != cudaSuccess) return e;
    // clusters of 16 CTAs need this attribute; without it the any-stride kernel stays at 8
    g_generic_cluster16 = cudaFuncSetAttribute(generic::gemm_generic_kernel<true>,
                                               cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    if (!g_generic_cluster16) cudaGetLastError();
    if (mlp_step::init_device() != 0) return cudaErrorUnknown;
    if ((e = cudaFuncSetAttribute(skinny::skinny_n_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::stream::Cfg<4>::SMEM_BYTES)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(skinny::skinny_n_stream_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::stream::Cfg<8>::SMEM_BYTES)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(skinny::skinny_n_stream_kernel<12>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::stream::Cfg<12>::SMEM_BYTES)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(skinny::skinny_n_stream_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::stream::Cfg<16>::SMEM_BYTES)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(skinny::skinny_m_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::mstream::SMEM_BYTES)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(skinny::skinny_m_stream_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::mstream::SMEM_BYTES)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(skinny::skinny_m_stream_kernel<12>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::mstream::SMEM_BYTES)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(skinny::skinny_m_stream_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  skinny::mstream::SMEM_BYTES)) != cudaSuccess) return e;
    return tf32::init_device() == 0 ? cudaSuccess : cudaErrorUnknown;
}

int check_common(tt_handle_t h, const void* a, const void* b, const void* c, int M, int N, int K)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (M < 0 || N < 0 || K < 0) return fail(h, TT_ERR_INVALID_ARG, "negative dimension");
    if ((static_cast<long long>(M) * N > 0) && (!c || (K > 0 && (!a || !b))))
        return fail(h, TT_ERR_INVALID_ARG, "null device pointer");
    return TT_OK;
}

// Driver entry points, resolved through the runtime so the library does not link libcuda.
struct DriverApi {
    PFN_cuCtxGetCurrent_v4000 get_current = nullptr;
    PFN_cuCtxPushCurrent_v4000 push_current = nullptr;
    PFN_cuCtxPopCurrent_v4000 pop_current = nullptr;
    PFN_cuCtxGetDevice_v2000 get_device = nullptr;
    bool ok = false;
};

const DriverApi& driver_api()
{
    static DriverApi api = [] {
        DriverApi d;
        const auto get = [](const char* name) -> void* {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
                return nullptr;
            return fn;
        };
        d.get_current = reinterpret_cast<PFN_cuCtxGetCurrent_v4000>(get("cuCtxGetCurrent"));
        d.push_current = reinterpret_cast<PFN_cuCtxPushCurrent_v4000>(get("cuCtxPushCurrent"));
        d.pop_current = reinterpret_cast<PFN_cuCtxPopCurrent_v4000>(get("cuCtxPopCurrent"));
        d.get_device = reinterpret_cast<PFN_cuCtxGetDevice_v2000>(get("cuCtxGetDevice"));
        d.ok = d.get_current && d.push_current && d.pop_current && d.get_device;
        return d;
    }();
    return api;
}

// Every entry runs in the handle's context.  Normally that context is already current on the
// calling thread (the host made it current before tt_create and keeps it so) and the scope does
// nothing.  When another context, or none, is current, the handle's context is pushed for the
// duration of the call and popped again: the caller's current context is never replaced.
struct CtxScope {
    bool pushed = false;
    int rc = TT_OK;
    explicit CtxScope(tt_handle_t h)
    {
        const DriverApi& d = driver_api();
        CUcontext cur = nullptr;
        if (!d.ok || d.get_current(&cur) != CUDA_SUCCESS) { rc = cuda_fail(h, cudaErrorUnknown, "cuCtxGetCurrent"); return; }
        if (cur == h->ctx) return;
        if (d.push_current(h->ctx) != CUDA_SUCCESS) { rc = cuda_fail(h, cudaErrorUnknown, "cuCtxPushCurrent"); return; }
        pushed = true;
    }
    ~CtxScope()
    {
        if (pushed) { CUcontext out = nullptr; driver_api().pop_current(&out); }
    }
    CtxScope(const CtxScope&) = delete;
    CtxScope& operator=(const CtxScope&) = delete;
};

// First statement of every entry after its argument checks: declares the scope object for the rest of the function.
#define TT_BIND(h)                  \
    CtxScope tt_ctx_scope_(h);      \
    if (tt_ctx_scope_.rc) return tt_ctx_scope_.rc

// Linear backward (activation backward + bias gradient, dX, dW).  With `scatter` the weight
// gradient is first offered to the kernels whose epilogue stores through the scatter table;
// *fused tells the caller whether one of them took it (otherwise dw holds the whole gradient).
int linear_bwd_impl(tt_handle_t h, cudaStream_t st, const float* x, const float* w, const float* y,
                    const float* dy, float* dx, float* dw, float* dbias, int M, int N, int K, int act,
                    const Epilogue* scatter, int* fused)
{
    if (fused) *fused = 0;
    if (!h) return TT_ERR_INVALID_ARG;
    if (M < 0 || N < 0 || K < 0) return fail(h, TT_ERR_INVALID_ARG, "negative dimension");
    if (act < TT_ACT_NONE || act > TT_ACT_TANH) return fail(h, TT_ERR_INVALID_ARG, "unknown activation");
    if (!dy || !x || !w || !dw || (act != TT_ACT_NONE && !y))
        return fail(h, TT_ERR_INVALID_ARG, "null device pointer");
    TT_BIND(h);
    int rc = TT_OK;
    h->stats.calls++;

    // Small layers (the latency-bound shapes of small networks): everything in one launch.
    if (h->variant == 0 && !(scatter && scatter->scatter_rows > 0) && M > 0 && N > 0 && K > 0 &&
        static_cast<long long>(M) * N * K <= LINEAR_SMALL_MAX_ELEMS) {
        lin_small::Params lp;
        lp.x = x; lp.w = w; lp.y = y; lp.dy = dy; lp.dx = dx; lp.dw = dw; lp.db = dbias;
        lp.M = M; lp.N = N; lp.K = K; lp.act = act;
        lp.tiles_k = (K + lin_small::T - 1) / lin_small::T;
        lp.tiles_dx = dx ? ((M + lin_small::T - 1) / lin_small::T) * lp.tiles_k : 0;
        const int tiles_dw = ((N + lin_small::T - 1) / lin_small::T) * lp.tiles_k;
        lin_small::linear_bwd_small_kernel<<<lp.tiles_dx + tiles_dw, lin_small::THREADS, 0, st>>>(lp);
        h->stats.launches++;
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(h, e, "small linear backward launch");
        return TT_OK;
    }

    const float* g = dy;
    size_t ws_used = 0;  // the masked gradient and the column-sum partials stay live during the GEMMs
    if (static_cast<long long>(M) * N > 0 && (act != TT_ACT_NONE || dbias)) {
        const int chunks = ew::colsum_chunks(M);
        const size_t g_bytes = act != TT_ACT_NONE ? sizeof(float) * static_cast<size_t>(M) * N : 0;
        const size_t g_bytes_al = (g_bytes + 255) & ~static_cast<size_t>(255);
        const size_t part_bytes = dbias ? sizeof(float) * static_cast<size_t>(chunks) * N : 0;
        if (g_bytes_al + part_bytes > h->workspace_bytes)
            return fail(h, TT_ERR_WORKSPACE, "workspace too small for linear backward");
        float* gbuf = act != TT_ACT_NONE ? reinterpret_cast<float*>(h->workspace) : nullptr;
        // one chunk of rows (M < 128): the column sums are final, they go straight to dbias
        float* partial = !dbias ? nullptr : chunks == 1 ? dbias : reinterpret_cast<float*>(h->workspace + g_bytes_al);
        const bool vec = (N % 4 == 0) && aligned16(dy) && (!act || aligned16(y));
        const dim3 grid((N + ew::COLSUM_COLS - 1) / ew::COLSUM_COLS, chunks);
        if (vec) ew::act_bwd_colsum_kernel<true><<<grid, 256, 0, st>>>(y, dy, gbuf, partial, M, N, act, chunks);
        else     ew::act_bwd_colsum_kernel<false><<<grid, 256, 0, st>>>(y, dy, gbuf, partial, M, N, act, chunks);
        h->stats.launches++;
        if (dbias && chunks > 1) {
            ew::colsum_finish_kernel<<<(N + 255) / 256, 256, 0, st>>>(partial, dbias, N, chunks);
            h->stats.launches++;
        }
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(h, e, "linear backward elementwise launch");
        if (gbuf) g = gbuf;
        ws_used = (g_bytes_al + part_bytes + 255) & ~static_cast<size_t>(255);
    } else if (dbias && N > 0) {
        const cudaError_t e = cudaMemsetAsync(dbias, 0, sizeof(float) * N, st);
        if (e != cudaSuccess) return cuda_fail(h, e, "memset dbias");
    }
    if (dx) {
        // dx[m,k] = sum_n g[m*N + n] * w[n*K + k]   (src/Tensotron/TensorOps.LinearNT.cs:36)
        GemmCall gx{g, w, dx, M, K, N, N, 1, K, 1, HostBatch(), 1, Epilogue{nullptr, TT_ACT_NONE}};
        gx.ws_off = ws_used;
        if ((rc = run_gemm(h, st, gx))) return rc;
    }
    // dw[n,k] = sum_m g[m*N + n] * x[m*K + k]       (src/Tensotron/TensorOps.LinearNT.cs:44)
    GemmCall gw{g, x, dw, N, K, M, 1, N, K, 1, HostBatch(), 1, Epilogue{nullptr, TT_ACT_NONE}};
    gw.ws_off = ws_used;
    if (scatter && scatter->scatter_rows > 0) {
        gw.epi.scatter_rows = scatter->scatter_rows;
        for (int o = 0; o < MAX_PEERS; o++) gw.epi.scatter[o] = scatter->scatter[o];
        rc = run_gemm(h, st, gw);
        if (rc == TT_OK) {
            if (fused) *fused = 1;
            return TT_OK;
        }
        if (rc != TT_ERR_UNSUPPORTED) return rc;
        gw.epi.scatter_rows = 0;
    }
    return run_gemm(h, st, gw);
}


}  // namespace

extern "C" {

TT_API const char* tt_version(void) { return "tensotron-gemm-b200 0.1 (sm_100a)"; }

TT_API int tt_create(int device, size_t workspace_bytes, tt_handle_t* out_handle)
{
    if (!out_handle) return TT_ERR_INVALID_ARG;
    *out_handle = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return TT_ERR_CUDA;
    // Context: the one that is current on the calling thread when it belongs to `device` (a host
    // with a driver-API context of its own makes it current before this call, the way it does
    // for its cuBLAS handle); only when none is current, or the current one is on another
    // device, the device's primary context is made current (cudaSetDevice).
    const DriverApi& d = driver_api();
    if (!d.ok) return TT_ERR_CUDA;
    CUcontext ctx = nullptr;
    CUdevice ctx_dev = -1;
    if (d.get_current(&ctx) != CUDA_SUCCESS) return TT_ERR_CUDA;
    if (ctx && (d.get_device(&ctx_dev) != CUDA_SUCCESS || static_cast<int>(ctx_dev) != device)) ctx = nullptr;
    if (!ctx) {
        if (cudaSetDevice(device) != cudaSuccess) return TT_ERR_CUDA;
        if (cudaFree(nullptr) != cudaSuccess) return TT_ERR_CUDA;   // brings the primary context up
        if (d.get_current(&ctx) != CUDA_SUCCESS || !ctx) return TT_ERR_CUDA;
    }
    tt_handle_s* h = new tt_handle_s();
    memset(h, 0, sizeof(*h));
    h->ctx = ctx;
    h->device = device;
    h->math_mode = TT_MATH_FP32;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete h; return TT_ERR_CUDA; }
    if (prop.major != 10) { delete h; return TT_ERR_UNSUPPORTED; }  // sm_100a code only
    h->num_sms = prop.multiProcessorCount;
    h->workspace_bytes = workspace_bytes ? workspace_bytes : DEFAULT_WORKSPACE;
    if (cudaMalloc(&h->workspace, h->workspace_bytes) != cudaSuccess) { delete h; return TT_ERR_CUDA; }
    if (cudaMalloc(&h->status, HANDLE_WORDS * sizeof(unsigned int)) != cudaSuccess) { cudaFree(h->workspace); delete h; return TT_ERR_CUDA; }
    cudaMemset(h->status, 0, HANDLE_WORDS * sizeof(unsigned int));
    // kernel attributes are per context: set them in this one
    if (init_kernels() != cudaSuccess) { cudaFree(h->workspace); cudaFree(h->status); delete h; return TT_ERR_CUDA; }
    h->max_cluster = g_generic_cluster16 ? 16 : 8;
    h->stats.workspace_bytes = static_cast<long long>(h->workspace_bytes);
    h->err[0] = 0;
    *out_handle = h;
    return TT_OK;
}

TT_API int tt_destroy(tt_handle_t h)
{
    if (!h) return TT_ERR_INVALID_ARG;
    {
        CtxScope scope(h);
        if (scope.rc == TT_OK) {
            cudaFree(h->workspace);
            cudaFree(h->status);
        }
    }
    delete h;
    return TT_OK;
}

TT_API const char* tt_last_error(tt_handle_t h) { return h ? h->err : "null handle"; }

TT_API int tt_set_math_mode(tt_handle_t h, int mode)
{
    if (!h) return TT_ERR_INVALID_ARG;
    // 1 is cuBLAS's legacy tensor-op math, which SetCuBlasMathMode also accepts
    // (src/Tensotron/TensorRuntime.cs:332-338): served by the TF32 kernel, the nearest mode here
    // (and more accurate than the FP16-class arithmetic that value selects in cuBLAS).
    if (mode == 1) mode = TT_MATH_TF32;
    if (mode != TT_MATH_FP32 && mode != TT_MATH_TF32 && mode != TT_MATH_3XTF32)
        return fail(h, TT_ERR_INVALID_ARG, "unknown math mode");
    h->math_mode = mode;
    return TT_OK;
}

TT_API int tt_get_math_mode(tt_handle_t h, int* mode)
{
    if (!h || !mode) return TT_ERR_INVALID_ARG;
    *mode = h->math_mode;
    return TT_OK;
}

TT_API int tt_set_variant(tt_handle_t h, int variant)
{
    if (!h || variant < 0 || variant > 10) return TT_ERR_INVALID_ARG;
    h->variant = variant;
    return TT_OK;
}

TT_API int tt_matmul(tt_handle_t h, void* stream, const float* a, const float* b, float* c, int M, int N,
              int K, int aMs, int aKs, int bKs, int bNs)
{
    int rc = check_common(h, a, b, c, M, N, K);
    if (rc) return rc;
    TT_BIND(h);
    h->stats.calls++;
    GemmCall g{a, b, c, M, N, K, aMs, aKs, bKs, bNs, HostBatch(), 1, Epilogue{nullptr, TT_ACT_NONE}};
    return run_gemm(h, static_cast<cudaStream_t>(stream), g);
}

TT_API int tt_matmul_batched(tt_handle_t h, void* stream, const float* a, const float* b, float* c,
                      int batchCount, int M, int N, int K, int aMs, int aKs, int bKs, int bNs,
                      int batchRank, const int* batchDims, const int* aBatchStrides,
                      const int* bBatchStrides)
{
    int rc = check_common(h, a, b, c, M, N, K);
    if (rc) return rc;
    if (batchCount < 0 || batchRank < 0) return fail(h, TT_ERR_INVALID_ARG, "negative batch");
    if (batchRank > 0 && (!batchDims || !aBatchStrides || !bBatchStrides))
        return fail(h, TT_ERR_INVALID_ARG, "null batch arrays");
    long long prod = 1;
    for (int i = 0; i < batchRank; i++) {
        if (batchDims[i] < 0) return fail(h, TT_ERR_INVALID_ARG, "negative batch dim");
        prod *= batchDims[i];
    }
    if (prod != batchCount) return fail(h, TT_ERR_INVALID_ARG, "batchCount != product(batchDims)");
    TT_BIND(h);
    h->stats.calls++;
    GemmCall g{a, b, c, M, N, K, aMs, aKs, bKs, bNs, HostBatch(), batchCount,
               Epilogue{nullptr, TT_ACT_NONE}};
    if (batchCount == 0) return TT_OK;
    if (!collapse_batch(batchRank, batchDims, aBatchStrides, bBatchStrides, g.batch))
        return fail(h, TT_ERR_UNSUPPORTED, "more than 8 non-mergeable batch axes");
    return run_gemm(h, static_cast<cudaStream_t>(stream), g);
}

TT_API int tt_matmul_batched_reduce(tt_handle_t h, void* stream, const float* a, const float* b, float* c,
                                    int M, int N, int K, int aMs, int aKs, int bKs, int bNs, int batchRank,
                                    const int* batchDims, const int* aBatchStrides,
                                    const int* bBatchStrides, const int* reduceAxis)
{
    int rc = check_common(h, a, b, c, M, N, K);
    if (rc) return rc;
    if (batchRank < 0 || batchRank > 32) return fail(h, TT_ERR_INVALID_ARG, "bad batch rank");
    if (batchRank > 0 && (!batchDims || !aBatchStrides || !bBatchStrides || !reduceAxis))
        return fail(h, TT_ERR_INVALID_ARG, "null batch arrays");
    int kd[32], ka[32], kb[32], nk = 0;
    HostBatch hb;
    bool have_red = false;
    long long kept = 1;
    for (int ax = 0; ax < batchRank; ax++) {
        if (batchDims[ax] < 0) return fail(h, TT_ERR_INVALID_ARG, "negative batch dim");
        if (batchDims[ax] == 0) return TT_OK;  // empty batch: nothing to compute (C is empty or stays as is)
        if (reduceAxis[ax] && batchDims[ax] > 1) {
            if (!have_red) {
                hb.red_count = batchDims[ax]; hb.red_as = aBatchStrides[ax]; hb.red_bs = bBatchStrides[ax];
                have_red = true;
            } else if (static_cast<long long>(hb.red_as) == static_cast<long long>(batchDims[ax]) * aBatchStrides[ax] &&
                       static_cast<long long>(hb.red_bs) == static_cast<long long>(batchDims[ax]) * bBatchStrides[ax]) {
                hb.red_count *= batchDims[ax]; hb.red_as = aBatchStrides[ax]; hb.red_bs = bBatchStrides[ax];
            } else {
                return fail(h, TT_ERR_UNSUPPORTED, "reduced batch axes do not merge into one");
            }
        } else if (!reduceAxis[ax]) {
            kd[nk] = batchDims[ax]; ka[nk] = aBatchStrides[ax]; kb[nk] = bBatchStrides[ax];
            kept *= batchDims[ax];
            nk++;
        }
    }
    TT_BIND(h);
    h->stats.calls++;
    const int rc_n = hb.red_count, rc_a = hb.red_as, rc_b = hb.red_bs;
    if (!collapse_batch(nk, kd, ka, kb, hb))
        return fail(h, TT_ERR_UNSUPPORTED, "more than 8 non-mergeable batch axes");
    hb.red_count = rc_n; hb.red_as = rc_a; hb.red_bs = rc_b;
    GemmCall g{a, b, c, M, N, K, aMs, aKs, bKs, bNs, hb, static_cast<int>(kept), Epilogue{nullptr, TT_ACT_NONE}};
    return run_gemm(h, static_cast<cudaStream_t>(stream), g);
}

TT_API int tt_reduce_sum_axes(tt_handle_t h, void* stream, const float* src, float* dst, int rank,
                              const int* dims, const int* reduceAxis)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (rank < 0 || rank > 8 || (rank > 0 && (!dims || !reduceAxis))) return fail(h, TT_ERR_INVALID_ARG, "bad reduction rank");
    ew::ReduceAxes ax;
    memset(&ax, 0, sizeof(ax));
    long long n_out = 1, n_red = 1, stride = 1;
    long long strides[8];
    for (int i = rank - 1; i >= 0; i--) {
        if (dims[i] < 0) return fail(h, TT_ERR_INVALID_ARG, "negative dimension");
        strides[i] = stride;
        stride *= dims[i];
    }
    for (int i = 0; i < rank; i++) {
        if (reduceAxis[i]) {
            ax.red_dim[ax.n_red] = dims[i]; ax.red_stride[ax.n_red] = strides[i]; ax.n_red++;
            n_red *= dims[i];
        } else {
            ax.kept_dim[ax.n_kept] = dims[i]; ax.kept_stride[ax.n_kept] = strides[i]; ax.n_kept++;
            n_out *= dims[i];
        }
    }
    if (n_out > 0 && (!dst || (n_red > 0 && !src))) return fail(h, TT_ERR_INVALID_ARG, "null device pointer");
    TT_BIND(h);
    h->stats.calls++;
    if (n_out == 0) return TT_OK;
    ew::reduce_axes_kernel<<<static_cast<unsigned int>((n_out + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, dst, ax, n_out, n_red);
    h->stats.launches++;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "reduction launch");
    return TT_OK;
}

TT_API int tt_linear_fwd(tt_handle_t h, void* stream, const float* x, const float* w, const float* bias,
                  float* y, int M, int N, int K, int act)
{
    int rc = check_common(h, x, w, y, M, N, K);
    if (rc) return rc;
    if (act < TT_ACT_NONE || act > TT_ACT_TANH) return fail(h, TT_ERR_INVALID_ARG, "unknown activation");
    TT_BIND(h);
    h->stats.calls++;
    // y[m,n] = sum_k x[m*K + k] * w[n*K + k]   (src/Tensotron/TensorOps.LinearNT.cs:24)
    GemmCall g{x, w, y, M, N, K, K, 1, 1, K, HostBatch(), 1, Epilogue{bias, act}};
    return run_gemm(h, static_cast<cudaStream_t>(stream), g);
}

TT_API int tt_linear_bwd(tt_handle_t h, void* stream, const float* x, const float* w, const float* y,
                  const float* dy, float* dx, float* dw, float* dbias, int M, int N, int K, int act)
{
    return linear_bwd_impl(h, static_cast<cudaStream_t>(stream), x, w, y, dy, dx, dw, dbias, M, N, K, act,
                           nullptr, nullptr);
}

namespace {
// Fills the derived sizes; false when the description is not a valid convolution.
bool conv_shape(const tt_conv2d_desc* d, conv::Shape& s)
{
    if (!d || d->n < 0 || d->c <= 0 || d->h <= 0 || d->w <= 0 || d->o <= 0 || d->kh <= 0 || d->kw <= 0 ||
        d->stride <= 0 || d->dilation <= 0 || d->padding < 0)
        return false;
    s.n = d->n; s.c = d->c; s.h = d->h; s.w = d->w; s.o = d->o; s.kh = d->kh; s.kw = d->kw;
    s.stride = d->stride; s.pad = d->padding; s.dil = d->dilation;
    // ConvOutSize (src/Tensotron/TensorOps.Conv.cs:5-6)
    s.ho = (d->h + 2 * d->padding - d->dilation * (d->kh - 1) - 1) / d->stride + 1;
    s.wo = (d->w + 2 * d->padding - d->dilation * (d->kw - 1) - 1) / d->stride + 1;
    if (s.ho <= 0 || s.wo <= 0) return false;
    const long long K = static_cast<long long>(d->c) * d->kh * d->kw, L = static_cast<long long>(s.ho) * s.wo;
    if (K + 4 > 0x7fffffffll || L > 0x7fffffffll || static_cast<long long>(d->n) * (K + 4) * L > 0x7fffffffll ||
        static_cast<long long>(d->n) * d->o * L > 0x7fffffffll)
        return false;     // element offsets fit int32, like every buffer of the reference
    s.K = static_cast<int>(K);
    s.L = static_cast<int>(L);
    s.Kp = (s.K + 1 + 3) & ~3;
    return true;
}

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct ConvWorkspace {
    size_t col, wp, dcol, end;   // byte offsets into the handle workspace
};

ConvWorkspace conv_workspace(const conv::Shape& s, bool backward)
{
    ConvWorkspace w;
    w.col = 0;
    w.wp = align256(sizeof(float) * static_cast<size_t>(s.n) * s.Kp * s.L);
    w.dcol = w.wp + align256(sizeof(float) * static_cast<size_t>(s.o) * s.Kp);
    w.end = w.dcol + (backward ? align256(sizeof(float) * static_cast<size_t>(s.n) * s.K * s.L) : 0);
    return w;
}

int conv_im2col(tt_handle_t h, cudaStream_t st, const conv::Shape& s, const float* x, float* col)
{
    const long long total = static_cast<long long>(s.n) * s.Kp * s.L;
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(h->num_sms) * 32;
    if (blocks > cap) blocks = cap;
    conv::im2col_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(x, col, s);
    h->stats.launches++;
    return TT_OK;
}
}  // namespace

TT_API size_t tt_conv2d_workspace(const tt_conv2d_desc* d, int backward)
{
    conv::Shape s;
    if (!conv_shape(d, s)) return 0;
    // + room for what the GEMMs themselves may take (split-K partial tiles, 3xTF32 operand planes)
    return conv_workspace(s, backward != 0).end + (64ull << 20);
}

TT_API int tt_conv2d_fwd(tt_handle_t h, void* stream, const tt_conv2d_desc* d, const float* x, const float* w,
                         const float* bias, float* y)
{
    if (!h) return TT_ERR_INVALID_ARG;
    conv::Shape s;
    if (!conv_shape(d, s)) return fail(h, TT_ERR_INVALID_ARG, "bad convolution description");
    if (s.n > 0 && (!x || !w || !y)) return fail(h, TT_ERR_INVALID_ARG, "null device pointer");
    TT_BIND(h);
    h->stats.calls++;
    if (s.n == 0) return TT_OK;
    const ConvWorkspace ws = conv_workspace(s, false);
    if (ws.end > h->workspace_bytes) return fail(h, TT_ERR_WORKSPACE, "workspace too small for the convolution's columns");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* col = reinterpret_cast<float*>(h->workspace + ws.col);
    float* wp = reinterpret_cast<float*>(h->workspace + ws.wp);
    conv_im2col(h, st, s, x, col);
    conv::pack_weight_kernel<<<(s.o * s.Kp + 255) / 256, 256, 0, st>>>(w, bias, wp, s.o, s.K, s.Kp);
    h->stats.launches++;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "im2col launch");
    // y[n][o][l] = sum_k wp[o][k] * col[n][k][l]   (the k = K term is bias[o] * 1)
    GemmCall g{wp, col, y, s.o, s.L, s.Kp, s.Kp, 1, s.L, 1, HostBatch(), s.n, Epilogue{nullptr, TT_ACT_NONE}};
    const int bd[1] = {s.n}, as[1] = {0}, bs[1] = {s.Kp * s.L};
    if (!collapse_batch(1, bd, as, bs, g.batch)) return fail(h, TT_ERR_UNSUPPORTED, "batch");
    g.ws_off = ws.end;
    return run_gemm(h, st, g);
}

TT_API int tt_conv2d_bwd(tt_handle_t h, void* stream, const tt_conv2d_desc* d, const float* x, const float* w,
                         const float* dy, float* dx, float* dw, float* dbias)
{
    if (!h) return TT_ERR_INVALID_ARG;
    conv::Shape s;
    if (!conv_shape(d, s)) return fail(h, TT_ERR_INVALID_ARG, "bad convolution description");
    if (!x || !w || !dy || !dw) return fail(h, TT_ERR_INVALID_ARG, "null device pointer");
    TT_BIND(h);
    h->stats.calls++;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (s.n == 0) {
        cudaMemsetAsync(dw, 0, sizeof(float) * static_cast<size_t>(s.o) * s.K, st);
        if (dbias) cudaMemsetAsync(dbias, 0, sizeof(float) * s.o, st);
        return TT_OK;
    }
    const ConvWorkspace ws = conv_workspace(s, dx != nullptr);
    if (ws.end > h->workspace_bytes) return fail(h, TT_ERR_WORKSPACE, "workspace too small for the convolution's columns");
    float* col = reinterpret_cast<float*>(h->workspace + ws.col);
    conv_im2col(h, st, s, x, col);
    if (dbias) {
        conv::bias_grad_kernel<<<s.o, 256, 0, st>>>(dy, dbias, s.n, s.o, s.L);
        h->stats.launches++;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "convolution backward launch");
    int rc;
    {
        // dw[o][k] = sum_n sum_l dy[n][o][l] * col[n][k][l]: the batch axis is summed inside the k loop
        GemmCall g{dy, col, dw, s.o, s.K, s.L, s.L, 1, 1, s.L, HostBatch(), 1, Epilogue{nullptr, TT_ACT_NONE}};
        g.batch.red_count = s.n;
        g.batch.red_as = s.o * s.L;
        g.batch.red_bs = s.Kp * s.L;
        g.ws_off = ws.end;
        if ((rc = run_gemm(h, st, g))) return rc;
    }
    if (dx) {
        // dcol[n][k][l] = sum_o w[o][k] * dy[n][o][l]
        float* dcol = reinterpret_cast<float*>(h->workspace + ws.dcol);
        GemmCall g{w, dy, dcol, s.K, s.L, s.o, 1, s.K, s.L, 1, HostBatch(), s.n, Epilogue{nullptr, TT_ACT_NONE}};
        const int bd[1] = {s.n}, as[1] = {0}, bs[1] = {s.o * s.L};
        if (!collapse_batch(1, bd, as, bs, g.batch)) return fail(h, TT_ERR_UNSUPPORTED, "batch");
        g.ws_off = ws.end;
        if ((rc = run_gemm(h, st, g))) return rc;
        const long long total = static_cast<long long>(s.n) * s.c * s.h * s.w;
        long long blocks = (total + 255) / 256;
        const long long cap = static_cast<long long>(h->num_sms) * 32;
        if (blocks > cap) blocks = cap;
        conv::col2im_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(dcol, dx, s);
        h->stats.launches++;
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(h, e, "col2im launch");
    }
    return TT_OK;
}

TT_API int tt_softmax_cross_entropy(tt_handle_t h, void* stream, const float* logits, const int* labels,
                             float* dlogits, float* loss, int rows, int classes, float scale)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (rows < 0 || classes <= 0 || !logits || !labels) return fail(h, TT_ERR_INVALID_ARG, "bad cross-entropy arguments");
    TT_BIND(h);
    h->stats.calls++;
    if (rows == 0) return TT_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (sizeof(float) * static_cast<size_t>(rows) > h->workspace_bytes)
        return fail(h, TT_ERR_WORKSPACE, "workspace too small for cross-entropy");
    float* row_loss = loss ? reinterpret_cast<float*>(h->workspace) : nullptr;
    const int warps_per_block = 8;
    ew::softmax_ce_rows_kernel<<<(rows + warps_per_block - 1) / warps_per_block, 256, 0, st>>>(
        logits, labels, dlogits, row_loss, rows, classes, scale, h->status);
    h->stats.launches++;
    if (loss) {
        ew::sum_fixed_kernel<<<1, 1024, 0, st>>>(row_loss, loss, rows, scale);
        h->stats.launches++;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "cross-entropy launch");
    return TT_OK;
}

TT_API int tt_mse_loss(tt_handle_t h, void* stream, const float* input, const float* target, float* dinput,
                       float* loss, long long count)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (count < 0 || (count > 0 && (!input || !target))) return fail(h, TT_ERR_INVALID_ARG, "bad MSE arguments");
    TT_BIND(h);
    h->stats.calls++;
    if (count == 0) return TT_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int blocks = ew::reduce_blocks(count);
    if (sizeof(float) * 1024 > h->workspace_bytes) return fail(h, TT_ERR_WORKSPACE, "workspace too small for the loss");
    float* partial = reinterpret_cast<float*>(h->workspace);
    ew::reduce_partial_kernel<0><<<blocks, 256, 0, st>>>(input, target, dinput, partial, count,
                                                        2.f / static_cast<float>(count));
    h->stats.launches++;
    if (loss) {
        ew::sum_fixed_kernel<<<1, 1024, 0, st>>>(partial, loss, blocks, 1.f / static_cast<float>(count));
        h->stats.launches++;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "MSE launch");
    return TT_OK;
}

TT_API int tt_clip_grad_norm(tt_handle_t h, void* stream, float* grads, long long n, float max_norm, float eps,
                             float* norm_out)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (n < 0 || (n > 0 && !grads)) return fail(h, TT_ERR_INVALID_ARG, "bad clip arguments");
    TT_BIND(h);
    h->stats.calls++;
    if (n == 0) return TT_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int blocks = ew::reduce_blocks(n);
    if (sizeof(float) * 1028 > h->workspace_bytes) return fail(h, TT_ERR_WORKSPACE, "workspace too small for the clip");
    float* partial = reinterpret_cast<float*>(h->workspace);
    float* sumsq = partial + 1024;
    ew::reduce_partial_kernel<1><<<blocks, 256, 0, st>>>(grads, nullptr, nullptr, partial, n, 0.f);
    ew::sum_fixed_kernel<<<1, 1024, 0, st>>>(partial, sumsq, blocks, 1.f);
    long long sblocks = (n + 255) / 256;
    const long long cap = static_cast<long long>(h->num_sms) * 16;
    if (sblocks > cap) sblocks = cap;
    ew::clip_scale_kernel<<<static_cast<int>(sblocks), 256, 0, st>>>(grads, sumsq, n, max_norm, eps, norm_out);
    h->stats.launches += 3;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "clip launch");
    return TT_OK;
}

TT_API int tt_adam_step(tt_handle_t h, void* stream, float* p, const float* g, float* m, float* v,
                 float* adv, long long n, float beta1, float beta2, float lr, float eps,
                 float coupled_wd, float decoupled_factor, int advance)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (n < 0 || !adv || (n > 0 && (!p || !g || !m || !v))) return fail(h, TT_ERR_INVALID_ARG, "bad Adam arguments");
    TT_BIND(h);
    h->stats.calls++;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (advance) {
        ew::adam_advance_kernel<<<1, 1, 0, st>>>(adv, beta1, beta2);
        h->stats.launches++;
    }
    if (n > 0) {
        const bool vec = aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v);
        const long long work = vec ? (n + 3) / 4 : n;
        long long blocks = (work + 255) / 256;
        const long long cap = static_cast<long long>(h->num_sms) * 16;
        if (blocks > cap) blocks = cap;
        if (vec) ew::adam_step_kernel<true><<<static_cast<int>(blocks), 256, 0, st>>>(p, g, m, v, adv, n, beta1, beta2, lr, eps, coupled_wd, decoupled_factor);
        else     ew::adam_step_kernel<false><<<static_cast<int>(blocks), 256, 0, st>>>(p, g, m, v, adv, n, beta1, beta2, lr, eps, coupled_wd, decoupled_factor);
        h->stats.launches++;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "Adam launch");
    return TT_OK;
}

TT_API int tt_mlp_train_step(tt_handle_t h, void* stream, const tt_mlp_desc* net, float* params, float* m,
                             float* v, float* adv, float* grads_out, const float* x, const void* target,
                             float* loss_out, int batch, float lr, float beta1, float beta2, float eps,
                             float max_grad_norm, float clip_eps)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (!net || !params || !m || !v || !adv || !x || !target || batch < 1)
        return fail(h, TT_ERR_INVALID_ARG, "bad MLP step arguments");
    if (net->act < TT_ACT_NONE || net->act > TT_ACT_TANH || (net->loss != TT_LOSS_MSE && net->loss != TT_LOSS_CE))
        return fail(h, TT_ERR_INVALID_ARG, "unknown activation or loss");
    if (!aligned16(params) || !aligned16(m) || !aligned16(v) || (grads_out && !aligned16(grads_out)))
        return fail(h, TT_ERR_INVALID_ARG, "flat parameter buffers must be 16-byte aligned");
    TT_BIND(h);
    h->stats.calls++;
    int ctas = 0;
    const int rc = mlp_step::launch(static_cast<cudaStream_t>(stream), net, params, m, v, adv, grads_out, x, target,
                                    loss_out, h->status, batch, lr, beta1, beta2, eps, max_grad_norm, clip_eps, 1, &ctas);
    if (rc == TT_ERR_UNSUPPORTED) return fail(h, rc, "network or batch outside what the one-launch MLP step holds");
    if (rc != TT_OK) return fail(h, rc, "MLP step launch failed");
    h->stats.launches++;
    return TT_OK;
}

TT_API int tt_add_into(tt_handle_t h, void* stream, float* target, const float* source, long long n)
{
    if (!h) return TT_ERR_INVALID_ARG;
    if (n < 0 || (n > 0 && (!target || !source))) return fail(h, TT_ERR_INVALID_ARG, "bad AddInto arguments");
    TT_BIND(h);
    h->stats.calls++;
    if (n == 0) return TT_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = aligned16(target) && aligned16(source);
    const long long work = vec ? (n + 3) / 4 : n;
    long long blocks = (work + 255) / 256;
    const long long cap = static_cast<long long>(h->num_sms) * 16;
    if (blocks > cap) blocks = cap;
    if (vec) ew::add_into_kernel<true><<<static_cast<int>(blocks), 256, 0, st>>>(target, source, n);
    else     ew::add_into_kernel<false><<<static_cast<int>(blocks), 256, 0, st>>>(target, source, n);
    h->stats.launches++;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "AddInto launch");
    return TT_OK;
}

TT_API int tt_broadcast_batch(int ra, const int* a_dims, const int* a_strides, int rb, const int* b_dims,
                       const int* b_strides, int* rank, int* dims, int* a_bs, int* b_bs)
{
    if (ra < 0 || rb < 0 || !rank) return TT_ERR_INVALID_ARG;
    const int r = ra > rb ? ra : rb;
    *rank = r;
    for (int j = 0; j < r; j++) {
        const int axa = j - (r - ra), axb = j - (r - rb);
        const int da = axa >= 0 ? a_dims[axa] : 1;
        const int db = axb >= 0 ? b_dims[axb] : 1;
        if (da != db && da != 1 && db != 1) return TT_ERR_INVALID_ARG;
        const int od = da > db ? da : db;
        dims[j] = od;
        a_bs[j] = (axa >= 0 && da == od) ? a_strides[axa] : 0;
        b_bs[j] = (axb >= 0 && db == od) ? b_strides[axb] : 0;
    }
    return TT_OK;
}

TT_API int tt_shard_range(long long total, int world, int rank, long long* start, long long* count)
{
    if (total < 0 || world < 1 || rank < 0 || rank >= world || !start || !count) return TT_ERR_INVALID_ARG;
    const long long per = (total + world - 1) / world;
    const long long s0 = per * rank < total ? per * rank : total;
    const long long s1 = s0 + per < total ? s0 + per : total;
    *start = s0;
    *count = s1 - s0;
    return TT_OK;
}

TT_API int tt_get_stats(tt_handle_t h, tt_stats* out)
{
    if (!h || !out) return TT_ERR_INVALID_ARG;
    *out = h->stats;
    // the descriptor cache belongs to the calling thread, not to the handle: totals since the
    // thread's first call minus what tt_reset_stats recorded
    unsigned long long hits = 0, misses = 0;
    tensor_map_cache_stats(&hits, &misses);
    out->tensor_map_hits = static_cast<long long>(hits) - h->map_hits0;
    out->tensor_map_misses = static_cast<long long>(misses) - h->map_misses0;
    return TT_OK;
}

TT_API int tt_reset_stats(tt_handle_t h)
{
    if (!h) return TT_ERR_INVALID_ARG;
    const long long ws = h->stats.workspace_bytes;
    memset(&h->stats, 0, sizeof(h->stats));
    h->stats.workspace_bytes = ws;
    unsigned long long hits = 0, misses = 0;
    tensor_map_cache_stats(&hits, &misses);
    h->map_hits0 = static_cast<long long>(hits);
    h->map_misses0 = static_cast<long long>(misses);
    return TT_OK;
}

TT_API int tt_check(tt_handle_t h, void* stream)
{
    if (!h) return TT_ERR_INVALID_ARG;
    TT_BIND(h);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(h, e, "stream synchronize");
    unsigned int word = 0;
    e = cudaMemcpy(&word, h->status, sizeof(word), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(h, e, "status read");
    if (word != 0) {
        cudaMemset(h->status, 0, HANDLE_WORDS * sizeof(unsigned int));   // the status word and any flag left raised
        if (word == DEV_BAD_LABEL) {
            snprintf(h->err, sizeof(h->err), "cross-entropy label outside [0, classes): that row's loss is NaN");
            return TT_ERR_BAD_LABEL;
        }
        snprintf(h->err, sizeof(h->err), "device-side bounded wait gave up (code %u)", word);
        return TT_ERR_DEVICE_WAIT;
    }
    return TT_OK;
}

// ---- gradient exchange over peer memory --------------------------------------------------

struct tt_peer_group_s {
    tt_handle_t h;
    int world, rank;
    long long n;
    float* stage[MAX_PEERS];
    float* params[MAX_PEERS];
    unsigned int* flags[MAX_PEERS];
    unsigned long long wait_limit_ns;
};

static_assert(sizeof(cudaIpcMemHandle_t) == TT_IPC_HANDLE_BYTES, "IPC handle size");
static_assert(TT_MAX_PEERS == MAX_PEERS && TT_MAX_SEGMENTS == peer::MAX_SEGS && TT_PEER_CHANNELS == peer::CHANNELS &&
                  TT_PEER_FLAG_WORDS == peer::FLAG_WORDS && peer::STEP_COUNTER_WORD < peer::FLAG_WORDS,
              "header constants");

TT_API int tt_peer_alloc(tt_handle_t h, size_t bytes, void** out_ptr)
{
    if (!h || !out_ptr || bytes == 0) return TT_ERR_INVALID_ARG;
    TT_BIND(h);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return cuda_fail(h, e, "peer buffer allocation");
    e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) { cudaFree(p); return cuda_fail(h, e, "peer buffer clear"); }
    *out_ptr = p;
    return TT_OK;
}

TT_API int tt_peer_free(tt_handle_t h, void* ptr)
{
    if (!h) return TT_ERR_INVALID_ARG;
    TT_BIND(h);
    const cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) return cuda_fail(h, e, "peer buffer free");
    return TT_OK;
}

TT_API int tt_peer_export(tt_handle_t h, void* ptr, unsigned char* handle_out)
{
    if (!h || !ptr || !handle_out) return TT_ERR_INVALID_ARG;
    TT_BIND(h);
    cudaIpcMemHandle_t hd;
    const cudaError_t e = cudaIpcGetMemHandle(&hd, ptr);
    if (e != cudaSuccess) return cuda_fail(h, e, "cudaIpcGetMemHandle");
    memcpy(handle_out, &hd, sizeof(hd));
    return TT_OK;
}

TT_API int tt_peer_open(tt_handle_t h, const unsigned char* handle, void** out_ptr)
{
    if (!h || !handle || !out_ptr) return TT_ERR_INVALID_ARG;
    TT_BIND(h);
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle, sizeof(hd));
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(h, e, "cudaIpcOpenMemHandle");
    *out_ptr = p;
    return TT_OK;
}

TT_API int tt_peer_close(tt_handle_t h, void* ptr)
{
    if (!h || !ptr) return TT_ERR_INVALID_ARG;
    TT_BIND(h);
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) return cuda_fail(h, e, "cudaIpcCloseMemHandle");
    return TT_OK;
}

TT_API int tt_peer_group_create(tt_handle_t h, int world, int rank, long long n, void* const* stage,
                                void* const* params, void* const* flags, tt_peer_group_t* out)
{
    if (!h || !out) return TT_ERR_INVALID_ARG;
    *out = nullptr;
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || n <= 0 || n % 4 != 0 || !stage || !params || !flags)
        return fail(h, TT_ERR_INVALID_ARG, "bad peer group arguments");
    tt_peer_group_s* g = new tt_peer_group_s();
    memset(g, 0, sizeof(*g));
    g->h = h; g->world = world; g->rank = rank; g->n = n;
    g->wait_limit_ns = peer::PEER_WAIT_LIMIT_NS;
    for (int r = 0; r < world; r++) {
        if (!stage[r] || !params[r] || !flags[r] || !aligned16(stage[r]) || !aligned16(params[r])) {
            delete g;
            return fail(h, TT_ERR_INVALID_ARG, "null or unaligned peer buffer");
        }
        g->stage[r] = static_cast<float*>(stage[r]);
        g->params[r] = static_cast<float*>(params[r]);
        g->flags[r] = static_cast<unsigned int*>(flags[r]);
    }
    *out = g;
    return TT_OK;
}

TT_API int tt_peer_set_wait_limit(tt_peer_group_t g, int milliseconds)
{
    if (!g || milliseconds < 1 || milliseconds > 600000) return TT_ERR_INVALID_ARG;
    g->wait_limit_ns = 1000000ull * static_cast<unsigned long long>(milliseconds);
    return TT_OK;
}

TT_API int tt_peer_group_destroy(tt_peer_group_t g)
{
    if (!g) return TT_ERR_INVALID_ARG;
    delete g;
    return TT_OK;
}

TT_API int tt_peer_linear_bwd(tt_handle_t h, void* stream, tt_peer_group_t g, const float* x, const float* w,
                              const float* y, const float* dy, float* dx, long long w_off, long long b_off,
                              int M, int N, int K, int act, int own_rows, int* fused)
{
    if (fused) *fused = 0;
    if (!h || !g) return TT_ERR_INVALID_ARG;
    if (N < 0 || K < 0 || w_off < 0 || w_off % 4 != 0 || w_off + static_cast<long long>(N) * K > g->n ||
        (b_off >= 0 && b_off + N > g->n))
        return fail(h, TT_ERR_INVALID_ARG, "gradient range outside the flat buffer");
    if (own_rows < 0 || own_rows % 256 != 0 || (own_rows > 0 && (N + own_rows - 1) / own_rows > g->world))
        return fail(h, TT_ERR_INVALID_ARG, "own_rows must be a multiple of 256 that covers N with at most world blocks");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* local = g->stage[g->rank] + static_cast<long long>(g->rank) * g->n;
    const bool exchange = own_rows > 0;
    Epilogue sc{nullptr, TT_ACT_NONE};
    if (exchange) {
        sc.scatter_rows = own_rows;
        for (int o = 0; o < g->world; o++) sc.scatter[o] = g->stage[o] + static_cast<long long>(g->rank) * g->n + w_off;
    }
    int did_fuse = 0;
    int rc = linear_bwd_impl(h, st, x, w, y, dy, dx, local + w_off, b_off >= 0 ? local + b_off : nullptr, M, N, K,
                             act, exchange ? &sc : nullptr, &did_fuse);
    if (rc) return rc;
    if (fused) *fused = did_fuse;
    if (exchange && !did_fuse) {
        // the whole gradient is in the local slot: copy every other owner's row block to it
        for (int o = 0; o < g->world; o++) {
            if (o == g->rank) continue;
            const long long r0 = static_cast<long long>(o) * own_rows;
            if (r0 >= N) break;
            const long long rows = (N - r0) < own_rows ? (N - r0) : own_rows;
            const long long count = rows * K, at = w_off + r0 * K;
            if (count % 4 != 0 || at % 4 != 0)
                return fail(h, TT_ERR_UNSUPPORTED, "row blocks of the weight gradient are not 16-byte aligned");
            long long blocks = (count / 4 + 255) / 256;
            const long long cap = static_cast<long long>(h->num_sms) * 8;
            if (blocks > cap) blocks = cap;
            peer::copy_to_peer_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
                local + at, g->stage[o] + static_cast<long long>(g->rank) * g->n + at, count / 4);
            h->stats.launches++;
        }
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(h, e, "peer copy launch");
    }
    return TT_OK;
}

namespace {
int fill_segments(tt_handle_t h, tt_peer_group_t g, int n, const long long* off, const long long* len,
                  peer::SegList& out, long long& total4)
{
    total4 = 0;
    out.n = 0;
    if (n < 0 || n > peer::MAX_SEGS || (n > 0 && (!off || !len)))
        return fail(h, TT_ERR_INVALID_ARG, "bad segment list");
    for (int i = 0; i < n; i++) {
        if (off[i] < 0 || len[i] < 0 || off[i] % 4 != 0 || len[i] % 4 != 0 || off[i] + len[i] > g->n)
            return fail(h, TT_ERR_INVALID_ARG, "segment not a multiple of 4 floats or outside the flat buffer");
        out.off[i] = off[i];
        out.len[i] = len[i];
        total4 += len[i] / 4;
    }
    out.n = n;
    return TT_OK;
}
}  // namespace

TT_API int tt_peer_push(tt_handle_t h, void* stream, tt_peer_group_t g, int channel, int new_step, int n_segments,
                        const long long* offsets, const long long* lengths)
{
    if (!h || !g) return TT_ERR_INVALID_ARG;
    if (channel < 0 || channel >= peer::CHANNELS) return fail(h, TT_ERR_INVALID_ARG, "bad exchange channel");
    TT_BIND(h);
    int rc = TT_OK;
    h->stats.calls++;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    peer::SegList segs;
    long long total4 = 0;
    if ((rc = fill_segments(h, g, n_segments, offsets, lengths, segs, total4))) return rc;
    peer::PeerPtrs dst;
    for (int o = 0; o < MAX_PEERS; o++)
        dst.p[o] = (o < g->world && o != g->rank) ? g->stage[o] + static_cast<long long>(g->rank) * g->n : nullptr;
    peer::FlagPtrs f;
    for (int o = 0; o < MAX_PEERS; o++)
        f.p[o] = o < g->world ? g->flags[o] + channel * peer::CHANNEL_WORDS + g->rank : nullptr;
    unsigned int* step_counter = g->flags[g->rank] + peer::STEP_COUNTER_WORD;
    const float* local = g->stage[g->rank] + static_cast<long long>(g->rank) * g->n;
    if (g->world == 1) total4 = 0;   // nobody to copy to
    if (total4 <= peer::PUSH_SINGLE_BLOCK_MAX4) {
        peer::push_signal_kernel<<<1, 1024, 0, st>>>(local, dst, g->world, segs, total4, f, step_counter, new_step ? 1 : 0);
        h->stats.launches++;
    } else {
        long long blocks = (total4 + 255) / 256;
        const long long cap = static_cast<long long>(h->num_sms) * 8;
        if (blocks > cap) blocks = cap;
        peer::push_segments_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(local, dst, g->world, segs, total4);
        peer::signal_kernel<<<1, 32, 0, st>>>(f, g->world, step_counter, new_step ? 1 : 0);
        h->stats.launches += 2;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "peer push launch");
    return TT_OK;
}

TT_API int tt_peer_adam_step(tt_handle_t h, void* stream, tt_peer_group_t g, int channel, int n_owned,
                             const long long* owned_off, const long long* owned_len, int n_repl,
                             const long long* repl_off, const long long* repl_len, float* m, float* v, float* adv,
                             float beta1, float beta2, float lr, float eps, float coupled_wd,
                             float decoupled_factor, int advance)
{
    if (!h || !g) return TT_ERR_INVALID_ARG;
    if (channel < 0 || channel >= peer::CHANNELS) return fail(h, TT_ERR_INVALID_ARG, "bad exchange channel");
    if (!m || !v || !adv || !aligned16(m) || !aligned16(v)) return fail(h, TT_ERR_INVALID_ARG, "bad Adam arguments");
    TT_BIND(h);
    int rc = TT_OK;
    h->stats.calls++;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    peer::SegList owned, repl;
    long long owned4 = 0, repl4 = 0;
    if ((rc = fill_segments(h, g, n_owned, owned_off, owned_len, owned, owned4))) return rc;
    if ((rc = fill_segments(h, g, n_repl, repl_off, repl_len, repl, repl4))) return rc;
    unsigned int* step_counter = g->flags[g->rank] + peer::STEP_COUNTER_WORD;
    peer::PeerPtrs pp;
    for (int o = 0; o < MAX_PEERS; o++) pp.p[o] = o < g->world ? g->params[o] : nullptr;
    // tell every rank that this rank's rows are in its parameter buffer (last block of the kernel)
    peer::FlagPtrs f;
    for (int o = 0; o < MAX_PEERS; o++)
        f.p[o] = o < g->world ? g->flags[o] + channel * peer::CHANNEL_WORDS + MAX_PEERS + g->rank : nullptr;
    long long blocks = (owned4 + repl4 + 255) / 256;
    const long long cap = static_cast<long long>(h->num_sms) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    peer::reduce_adam_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
        g->stage[g->rank], g->n, g->world, g->rank, pp, m, v, adv, advance ? 1 : 0, owned, owned4, repl, repl4, beta1,
        beta2, lr, eps, coupled_wd, decoupled_factor, g->flags[g->rank] + channel * peer::CHANNEL_WORDS, step_counter,
        h->status, g->wait_limit_ns, f, g->flags[g->rank] + peer::DONE_COUNTER_WORD + channel);
    h->stats.launches++;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "peer Adam launch");
    return TT_OK;
}

TT_API int tt_peer_sync(tt_handle_t h, void* stream, tt_peer_group_t g, int n_channels)
{
    if (!h || !g) return TT_ERR_INVALID_ARG;
    if (n_channels < 1 || n_channels > peer::CHANNELS) return fail(h, TT_ERR_INVALID_ARG, "bad channel count");
    TT_BIND(h);
    h->stats.calls++;
    peer::wait_kernel<<<1, 32 * n_channels, 0, static_cast<cudaStream_t>(stream)>>>(
        g->flags[g->rank] + MAX_PEERS, g->world, g->flags[g->rank] + peer::STEP_COUNTER_WORD, h->status,
        g->wait_limit_ns);
    h->stats.launches++;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(h, e, "peer sync launch");
    return TT_OK;
}

}  // extern "C"
