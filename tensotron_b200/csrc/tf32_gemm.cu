// TF32 / 3xTF32 GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
// Persistent, warp-specialised CTA (one per SM, 320 threads):
//   warp 0     TMA producer: streams A (MT x 128 rows x 32 k) and B (256 cols x 32 k)
//              float tiles into a shared-memory ring (mbarrier full/empty hand-over);
//   warp 1     MMA issuer: one elected thread issues tcgen05.mma.kind::tf32 (M = 128,
//              N = 256, K = 8 per instruction) with shared-memory operand descriptors and
//              FP32 accumulators in tensor memory; tcgen05.commit releases ring stages
//              and signals finished accumulators.  The same warp owns the TMEM allocation;
//   warps 2-9  epilogue: tcgen05.ld the accumulator (a warp reads the 32-lane TMEM
//              sub-partition warp % 4; the two warps of a sub-partition take one half of the
//              columns each), add bias / apply the activation, store C.  The load of the next
//              32-column chunk is in flight while the current one is stored.
// MT = 1: 128x256 tiles with two accumulator buffers (the epilogue of tile i overlaps
// the MMAs of tile i+1).  MT = 2: 256x256 tiles (two M = 128 MMAs share every B tile,
// halving L2->SM traffic per flop) with a single accumulator set.
// The tile WIDTH is a launch parameter (bn = 64, 128, 192 or 256: the N of the MMA instruction,
// the rows of the B box, the columns the epilogue reads out), so that e.g. N = 192 is one
// 192-wide tile and no MMA, operand byte or TMEM read-out is spent on padding columns.
//
// Operands keep their global layout: a K-major tile is one TMA box of [rows][32 k]
// (128-byte rows, 128B swizzle, K-major UMMA descriptor); an MN-major tile is a row of
// [32 k][32 cols] boxes (32-byte-chunk 128B swizzle, MN-major UMMA descriptor, 4096 bytes
// between boxes).
//
// 3xTF32: A and B are split beforehand (one streaming pass) into hi = tf32(x) and
// lo = tf32(x - hi); each k-step issues lo*hi, hi*lo, hi*hi into the same FP32
// accumulator, which recovers close to FP32 accuracy at a third of the TF32 rate.
//
// Every wait is bounded; a wait that gives up raises a CTA-wide flag, all roles leave
// their loops, tensor memory is freed and the host can read the status word.
#include "tf32_launch.h"

#include <string.h>

#include "ptx.cuh"
#include "tensor_map.h"

namespace tt {
namespace tf32 {

constexpr int BN = 256, BK = 32, UMMA_K = 8;
constexpr int THREADS = 320;
constexpr int EPI_WARPS = 8;
constexpr int TMEM_COLS = 512;
constexpr int RASTER_GROUP = 8;

template <int MT, bool SPLIT>
struct Cfg {
    static constexpr int BM = 128 * MT;
    static constexpr int A_BYTES = BM * BK * 4;
    static constexpr int B_BYTES = BN * BK * 4;   // room for the widest tile; bn * BK * 4 bytes are filled
    static constexpr int PLANES = SPLIT ? 2 : 1;  // hi (+ lo)
    static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES) * PLANES;
    static constexpr int ACC_BUFS = MT == 1 ? 2 : 1;
    // epilogue staging: per epilogue warp EPI_BUFS blocks of 32 rows x 32 columns (128-byte rows,
    // the 16-byte chunks of row r stored at chunk index c ^ (r & 7), so both the row-wise writes
    // and the 4-rows-at-a-time reads are free of bank conflicts).  Two blocks per warp where the
    // ring can spare the room (128-row tiles, one operand plane): the TMA store of one block is
    // still reading it while the next block is staged, so a warp keeps two stores in flight.
    // With one block a warp's read-out is a chain of store latencies, which is what bounds
    // short-K products (their epilogue is longer than their MMAs).
    static constexpr int EPI_BUFS = (MT == 1 && !SPLIT) ? 2 : 1;
    static constexpr int OUT_BLOCK_BYTES = 32 * 128;
    static constexpr int OUT_WARP_BYTES = EPI_BUFS * OUT_BLOCK_BYTES;
    static constexpr int OUT_BYTES = EPI_WARPS * OUT_WARP_BYTES;
    static constexpr int BUDGET = 227 * 1024 - 1024 /*alignment slack*/ - 1024 /*barriers*/ - OUT_BYTES;
    static constexpr int STAGES = BUDGET / STAGE_BYTES;
    static constexpr int OFF_BAR = STAGES * STAGE_BYTES;
    static constexpr int OFF_OUT = OFF_BAR + 1024;   // 1024-byte aligned: the blocks are TMA-store sources
    static constexpr int SMEM_BYTES = OFF_OUT + OUT_BYTES + 1024;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared-memory budget");
    static_assert(STAGES >= 2, "shared-memory budget");
};

struct Params {
    GemmShape shape;
    BatchDesc batch;
    Epilogue epi;
    float* c;
    unsigned int* status;
    int c_vec_ok;
    // MN-major operand whose rows are a multiple of 32: the tensor map splits the row axis into
    // (32, rows / 32), so one TMA instruction brings all 32-column boxes of a k-tile
    // (coordinates {0, k, row / 32, batch...}) instead of one instruction per box.
    int a_grouped, b_grouped;
    // C is written with TMA stores from the staging blocks (map_c: {N, M, batch}, box 32 x 32,
    // 128-byte swizzle = the staging blocks' layout); 0: plain stores (scatter, N % 4 != 0).
    int c_tma;
    // tile width: 64, 128, 192 or 256 columns (tiles_n = ceil(N / bn))
    int bn;
};

// ---- tcgen05 wrappers -----------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], tf32 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrival once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns of this warp's TMEM sub-partition.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, with the loaded registers as in/out operands: the compiler then sees every
// later use of r as depending on the wait and cannot schedule arithmetic on r ahead of it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// Shared-memory operand descriptor (sm_100 format): start address, leading / stride byte
// offsets in 16-byte units, version 1, layout type (2 = 128-byte swizzle of 16-byte
// chunks, 1 = 128-byte swizzle of 32-byte chunks).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;   // descriptor version
    d |= static_cast<uint64_t>(layout_type) << 61;
    return d;
}

// Instruction descriptor: D = F32, A = B = TF32, M = 128, N = n (a multiple of 16, at most 256),
// per-operand major-ness.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int n)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

__device__ __forceinline__ float act_apply(float v, int act)
{
    if (act == 1) return v > 0.f ? v : 0.f;
    if (act == 2) return tanhf(v);
    return v;
}

struct TileCoord {
    int bidx, tm, tn;
};

__device__ __forceinline__ TileCoord decode_tile(long long w, const GemmShape& s)
{
    const int tiles_per_mat = s.tiles_m * s.tiles_n;
    TileCoord t;
    t.bidx = static_cast<int>(w / tiles_per_mat);
    const int r = static_cast<int>(w - static_cast<long long>(t.bidx) * tiles_per_mat);
    raster_tile(r, s.tiles_m, s.tiles_n, RASTER_GROUP, t.tm, t.tn);
    return t;
}

// map order: A hi, B hi, A lo, B lo (the lo maps are unused unless SPLIT).
template <int MT, bool A_KMAJ, bool B_KMAJ, bool SPLIT>
__global__ void __launch_bounds__(THREADS, 1)
tf32_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_alo,
                 const __grid_constant__ CUtensorMap map_blo, const __grid_constant__ CUtensorMap map_c,
                 const Params p)
{
    using C = Cfg<MT, SPLIT>;
    constexpr int STAGES = C::STAGES;
    constexpr int ACC_BUFS = C::ACC_BUFS;
    extern __shared__ uint8_t smem_raw[];
    // (pointer arithmetic on the shared array itself, so the compiler keeps emitting
    // shared-space loads rather than generic ones)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;
    uint64_t* acc_empty = acc_full + ACC_BUFS;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_BUFS);
    volatile uint32_t* cta_abort = tmem_slot + 1;
    uint64_t* drain_bar = reinterpret_cast<uint64_t*>(tmem_slot + 2);   // only used on the way out after a wait gave up

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_tiles = (p.shape.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < ACC_BUFS; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], EPI_WARPS);
        }
        mbar_init(drain_bar, 1);
        *cta_abort = 0u;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            prefetch_tensormap(&map_a);
            prefetch_tensormap(&map_b);
            if (SPLIT) {
                prefetch_tensormap(&map_alo);
                prefetch_tensormap(&map_blo);
            }
            uint32_t stage = 0, phase = 0, armed = 0;   // armed: stages armed so far, counted up to STAGES
            bool ok = true;
            for (long long w = blockIdx.x; ok && w < p.shape.work; w += gridDim.x) {
                const TileCoord tc = decode_tile(w, p.shape);
                int ca[3] = {0, 0, 0}, cb[3] = {0, 0, 0};
                int br = tc.bidx;
                for (int ax = p.batch.rank - 1; ax >= 0; ax--) {
                    const int d = p.batch.dims[ax];
                    const int bi = br % d;
                    br /= d;
                    if (p.batch.a_slot[ax] >= 0) ca[p.batch.a_slot[ax]] += bi * p.batch.a_mult[ax];
                    if (p.batch.b_slot[ax] >= 0) cb[p.batch.b_slot[ax]] += bi * p.batch.b_mult[ax];
                }
                const int m0 = tc.tm * C::BM, n0 = tc.tn * p.bn;
                for (int kt = 0; kt < k_tiles; kt++) {
                    if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, cta_abort, p.status, DEV_WAIT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = smem + stage * C::STAGE_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], (C::A_BYTES + p.bn * BK * 4) * C::PLANES);
                    const int k0 = kt * BK;
#pragma unroll
                    for (int pl = 0; pl < C::PLANES; pl++) {
                        const CUtensorMap* ma = pl == 0 ? &map_a : &map_alo;
                        const CUtensorMap* mb = pl == 0 ? &map_b : &map_blo;
                        uint8_t* sa = st + pl * (C::A_BYTES + C::B_BYTES);
                        uint8_t* sb = sa + C::A_BYTES;
                        if (A_KMAJ) {
                            tma_load_5d(sa, ma, &full_bar[stage], k0, m0, ca[0], ca[1], ca[2]);
                        } else if (p.a_grouped) {
                            tma_load_5d(sa, ma, &full_bar[stage], 0, k0, m0 >> 5, ca[0], ca[1]);
                        } else {
#pragma unroll
                            for (int i = 0; i < C::BM / 32; i++)
                                tma_load_5d(sa + i * 4096, ma, &full_bar[stage], m0 + i * 32, k0, ca[0], ca[1], ca[2]);
                        }
                        if (B_KMAJ) {
                            tma_load_5d(sb, mb, &full_bar[stage], k0, n0, cb[0], cb[1], cb[2]);
                        } else if (p.b_grouped) {
                            tma_load_5d(sb, mb, &full_bar[stage], 0, k0, n0 >> 5, cb[0], cb[1]);
                        } else {
                            for (int i = 0; i < p.bn / 32; i++)
                                tma_load_5d(sb + i * 4096, mb, &full_bar[stage], n0 + i * 32, k0, cb[0], cb[1], cb[2]);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    if (armed < STAGES) armed++;
                }
            }
            if (!ok || *cta_abort) {
                // A wait gave up somewhere in this CTA: before the teardown, wait (again with a limit)
                // for the loads this thread issued itself -- the last arming of every stage.
                uint32_t st = stage, ph = phase;
                for (uint32_t i = 0; i < armed; i++) {
                    if (st == 0) { st = STAGES; ph ^= 1u; }
                    st--;
                    mbar_wait_drain(&full_bar[st], ph);
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------- MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(!A_KMAJ, !B_KMAJ, p.bn);
            // K-major: 16-byte-chunk swizzle, 8-row groups 1024 bytes apart.  MN-major (32-bit
            // operands): 32-byte-chunk swizzle, 4-k groups 512 bytes apart inside a box of
            // 32 columns, boxes 4096 bytes apart.
            constexpr uint32_t A_LBO = A_KMAJ ? 16 : 4096, B_LBO = B_KMAJ ? 16 : 4096;
            constexpr uint32_t A_SBO = A_KMAJ ? 1024 : 512, B_SBO = B_KMAJ ? 1024 : 512;
            constexpr uint32_t A_LT = A_KMAJ ? 2 : 1, B_LT = B_KMAJ ? 2 : 1;
            constexpr uint32_t A_KSTEP = A_KMAJ ? UMMA_K * 4 : 1024, B_KSTEP = B_KMAJ ? UMMA_K * 4 : 1024;
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (long long w = blockIdx.x; ok && w < p.shape.work; w += gridDim.x) {
                if (!mbar_wait_bounded(&acc_empty[acc], acc_phase ^ 1u, cta_abort, p.status, DEV_WAIT_TMEM)) break;
                tc_fence_after();
                const uint32_t d_base = tmem_base + acc * (MT * BN);
                for (int kt = 0; kt < k_tiles; kt++) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase, cta_abort, p.status, DEV_WAIT_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + stage * C::STAGE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; kk++) {
                        const uint32_t accumulate = (kt > 0 || kk > 0) ? 1u : 0u;
#pragma unroll
                        for (int j = 0; j < MT; j++) {
                            const uint32_t a_hi = st + j * (128 * BK * 4) + kk * A_KSTEP;
                            const uint32_t b_hi = st + C::A_BYTES + kk * B_KSTEP;
                            const uint64_t da = make_desc(a_hi, A_LBO, A_SBO, A_LT);
                            const uint64_t db = make_desc(b_hi, B_LBO, B_SBO, B_LT);
                            const uint32_t d = d_base + j * BN;
                            if (SPLIT) {
                                const uint32_t plane = C::A_BYTES + C::B_BYTES;
                                const uint64_t dal = make_desc(a_hi + plane, A_LBO, A_SBO, A_LT);
                                const uint64_t dbl = make_desc(b_hi + plane, B_LBO, B_SBO, B_LT);
                                umma_tf32(d, dal, db, idesc, accumulate);   // lo * hi
                                umma_tf32(d, da, dbl, idesc, 1u);           // hi * lo
                                umma_tf32(d, da, db, idesc, 1u);            // hi * hi
                            } else {
                                umma_tf32(d, da, db, idesc, accumulate);
                            }
                        }
                    }
                    umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs retire
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&acc_full[acc]);  // accumulator complete
                if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
            }
            if (*cta_abort) {
                // leaving after a wait gave up: the MMAs issued so far must have retired before the
                // TMEM they write is freed (commit to a barrier of its own, bounded wait)
                umma_commit(drain_bar);
                mbar_wait_drain(drain_bar, 0u);
            }
        }
    } else {
        // --------------------------------- epilogue ---------------------------------
        const int ew = warp - 2;   // 0 .. 7
        const int q = warp & 3;    // TMEM sub-partition a warp may read: lanes 32q .. 32q+31
        const int cbeg = (ew >> 2) * (p.bn / 2), cend = cbeg + p.bn / 2;   // this warp's half of the tile's columns
        uint32_t acc = 0, acc_phase = 0;
        const float* bias = p.epi.bias;
        const int act = p.epi.act;
        const bool plain = bias == nullptr && act == 0;
        const bool bias_vec = (reinterpret_cast<uintptr_t>(bias) & 15u) == 0;
        uint8_t* const out_blocks = smem + C::OFF_OUT + ew * C::OUT_WARP_BYTES;
        uint32_t out_buf = 0;   // staging block of the next 32 x 32 block (alternates when there are two)
        for (long long w = blockIdx.x; w < p.shape.work; w += gridDim.x) {
            const TileCoord tc = decode_tile(w, p.shape);
            if (!mbar_wait_bounded(&acc_full[acc], acc_phase, cta_abort, p.status, DEV_WAIT_MMA)) break;
            tc_fence_after();
            float* cmat = scatter_base(p.epi, p.c, tc.tm * C::BM) + static_cast<long long>(tc.bidx) * p.shape.M * p.shape.N;
            const int n0 = tc.tn * p.bn;
            // One 32 x 32 block: bias / activation, through the staging block, out with 8 lanes per
            // row.  (The TMEM load gives lane l the 32 columns of row l; stored that way one
            // instruction would touch 32 rows with 16 bytes each.  After the exchange an
            // instruction writes 4 rows x 128 contiguous bytes: full sectors for L2, full-size
            // packets when the row block belongs to another GPU.)
            const auto emit = [&](const uint32_t (&r)[32], int row0, int c0) {
                uint8_t* const out_stage = out_blocks + out_buf * C::OUT_BLOCK_BYTES;
                if (C::EPI_BUFS == 2) out_buf ^= 1u;
                // the TMA store that last used this block has read it (with two blocks: all but
                // the most recent store)
                if (p.c_tma && lane == 0) {
                    if (C::EPI_BUFS == 2) bulk_wait_group_read1(); else bulk_wait_group_read0();
                }
                __syncwarp();   // the previous reads of this staging block are done
                // Stage the block.  Without bias and activation this is a straight copy of the 32
                // registers; the general form is kept out of that path (with two epilogue warps per
                // scheduler every instruction of the read-out costs about ten cycles, and per-element
                // bias / activation tests were three quarters of its instructions).
                uint8_t* const my_row = out_stage + lane * 128;
                const uint32_t sw = lane & 7;
                if (plain) {
#pragma unroll
                    for (int v4 = 0; v4 < 8; v4++)
                        *reinterpret_cast<uint4*>(my_row + ((v4 ^ sw) << 4)) =
                            make_uint4(r[v4 * 4], r[v4 * 4 + 1], r[v4 * 4 + 2], r[v4 * 4 + 3]);
                } else {
                    const int col0 = n0 + c0;
                    const bool bias_whole = bias && bias_vec && col0 + 31 < p.shape.N;
#pragma unroll
                    for (int v4 = 0; v4 < 8; v4++) {
                        float4 t = make_float4(__uint_as_float(r[v4 * 4]), __uint_as_float(r[v4 * 4 + 1]),
                                               __uint_as_float(r[v4 * 4 + 2]), __uint_as_float(r[v4 * 4 + 3]));
                        if (bias_whole) {
                            const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + col0) + v4);
                            t.x += b4.x; t.y += b4.y; t.z += b4.z; t.w += b4.w;
                        } else if (bias) {
                            const int col = col0 + v4 * 4;
                            if (col < p.shape.N) t.x += __ldg(bias + col);
                            if (col + 1 < p.shape.N) t.y += __ldg(bias + col + 1);
                            if (col + 2 < p.shape.N) t.z += __ldg(bias + col + 2);
                            if (col + 3 < p.shape.N) t.w += __ldg(bias + col + 3);
                        }
                        if (act == 1) {
                            t.x = t.x > 0.f ? t.x : 0.f; t.y = t.y > 0.f ? t.y : 0.f;
                            t.z = t.z > 0.f ? t.z : 0.f; t.w = t.w > 0.f ? t.w : 0.f;
                        } else if (act == 2) {
                            t.x = tanhf(t.x); t.y = tanhf(t.y); t.z = tanhf(t.z); t.w = tanhf(t.w);
                        }
                        *reinterpret_cast<float4*>(my_row + ((v4 ^ sw) << 4)) = t;
                    }
                }
                if (p.c_tma) {
                    // one asynchronous bulk store of the 32 x 32 block; rows >= M and columns >= N
                    // are clipped by the tensor map
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_5d(&map_c, out_stage, n0 + c0, row0, tc.bidx, 0, 0);
                        bulk_commit_group();
                    }
                    return;
                }
                __syncwarp();
                const int col = n0 + c0 + (lane & 7) * 4;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int lr = i * 4 + (lane >> 3);
                    const int grow = row0 + lr;
                    if (grow >= p.shape.M) continue;
                    const float4 v = *reinterpret_cast<const float4*>(out_stage + lr * 128 + (((lane & 7) ^ (lr & 7)) << 4));
                    float* crow = cmat + static_cast<long long>(grow) * p.shape.N;
                    if (p.c_vec_ok && col + 3 < p.shape.N) {
                        *reinterpret_cast<float4*>(crow + col) = v;
                    } else {
                        const float ve[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            if (col + e < p.shape.N) crow[col + e] = ve[e];
                    }
                }
            };
#pragma unroll 1
            for (int j = 0; j < MT; j++) {
                const int row0 = tc.tm * C::BM + j * 128 + q * 32;   // first row of this warp's blocks
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * (MT * BN) + j * BN;
                // chunks of 32 columns, two register sets: the load of chunk i + 1 is issued before
                // chunk i is stored (all conditions are warp-uniform)
                uint32_t ra[32], rb[32];
                if (n0 + cbeg < p.shape.N) tmem_ld_32x32(t_row + cbeg, ra);
#pragma unroll 1
                for (int c0 = cbeg; c0 < cend && n0 + c0 < p.shape.N; c0 += 64) {
                    tmem_ld_wait(ra);
                    const bool more_b = c0 + 32 < cend && n0 + c0 + 32 < p.shape.N;
                    if (more_b) tmem_ld_32x32(t_row + c0 + 32, rb);
                    emit(ra, row0, c0);
                    if (!more_b) break;
                    tmem_ld_wait(rb);
                    if (c0 + 64 < cend && n0 + c0 + 64 < p.shape.N) tmem_ld_32x32(t_row + c0 + 64, ra);
                    emit(rb, row0, c0 + 32);
                }
            }
            // all of this warp's TMEM reads of the buffer have completed (wait::ld above)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
            if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
        }
        if (p.c_tma && lane == 0) bulk_wait_group0();   // this thread's bulk stores are complete
    }

    // ---- teardown: every role ends up here, also after a wait that gave up ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// hi = tf32(x) (round to nearest, ties away), lo = tf32(x - hi); x - hi is exact in FP32.
__device__ __forceinline__ void split_one(float x, float& h, float& l)
{
    uint32_t hb, lb;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x));
    h = __uint_as_float(hb);
    const float rem = x - h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(rem));
    l = __uint_as_float(lb);
}

__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                                        float* __restrict__ lo, long long n)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n4 = n >> 2;
    for (long long i = tid; i < n4; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        float4 h, l;
        split_one(v.x, h.x, l.x);
        split_one(v.y, h.y, l.y);
        split_one(v.z, h.z, l.z);
        split_one(v.w, h.w, l.w);
        reinterpret_cast<float4*>(hi)[i] = h;
        reinterpret_cast<float4*>(lo)[i] = l;
    }
    for (long long i = (n4 << 2) + tid; i < n; i += stride) split_one(x[i], hi[i], lo[i]);
}

// ---- host side --------------------------------------------------------------------------

namespace {

struct HostBatch {
    int rank;
    const int* dims;
    const int* as;
    const int* bs;
};

bool plan_batch(const HostBatch& hb, const int* strides, signed char* slot, int* mult, OperandView& view)
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
    for (int s = 0; s < nslots; s++) {
        if (slot_stride[s] < 0) return false;
        view.dim[view.rank] = static_cast<uint64_t>(slot_extent[s]);
        view.stride_elems[view.rank] = static_cast<uint64_t>(slot_stride[s]);
        view.rank++;
    }
    return true;
}

// 1 K-major, 0 MN-major, -1 neither.  The tensor-core path takes strictly positive,
// TMA-legal strides only.
int classify(const float* base, int rows, int K, int row_stride, int k_stride, OperandView& v)
{
    v.base = base;
    v.rank = 2;
    v.stride_elems[0] = 1;
    if (k_stride == 1 && (rows == 1 || row_stride > 0)) {
        v.dim[0] = K; v.dim[1] = rows;
        v.stride_elems[1] = rows == 1 ? static_cast<uint64_t>(((K + 3) / 4) * 4) : static_cast<uint64_t>(row_stride);
        return 1;
    }
    if (row_stride == 1 && (K == 1 || k_stride > 0)) {
        v.dim[0] = rows; v.dim[1] = K;
        v.stride_elems[1] = K == 1 ? static_cast<uint64_t>(((rows + 3) / 4) * 4) : static_cast<uint64_t>(k_stride);
        return 0;
    }
    return -1;
}

// Number of floats from the operand base to one past its last addressed element.
long long operand_span(const OperandView& v)
{
    long long span = 1;
    for (int i = 0; i < v.rank; i++) span += static_cast<long long>(v.dim[i] - 1) * static_cast<long long>(v.stride_elems[i]);
    return span;
}

template <int MT, bool AK, bool BK_, bool SPLIT>
cudaError_t set_attr()
{
    return cudaFuncSetAttribute(tf32_gemm_kernel<MT, AK, BK_, SPLIT>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MT, SPLIT>::SMEM_BYTES);
}

template <int MT, bool SPLIT>
cudaError_t set_attr_layouts()
{
    cudaError_t e;
    if ((e = set_attr<MT, true, true, SPLIT>()) != cudaSuccess) return e;
    if ((e = set_attr<MT, true, false, SPLIT>()) != cudaSuccess) return e;
    if ((e = set_attr<MT, false, true, SPLIT>()) != cudaSuccess) return e;
    return set_attr<MT, false, false, SPLIT>();
}

template <int MT, bool SPLIT>
int launch_cfg(bool ak, bool bk, int grid, cudaStream_t st, const CUtensorMap* maps, const Params& p)
{
    constexpr int smem = Cfg<MT, SPLIT>::SMEM_BYTES;
    if (ak && bk) tf32_gemm_kernel<MT, true, true, SPLIT><<<grid, THREADS, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
    else if (ak && !bk) tf32_gemm_kernel<MT, true, false, SPLIT><<<grid, THREADS, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
    else if (!ak && bk) tf32_gemm_kernel<MT, false, true, SPLIT><<<grid, THREADS, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
    else tf32_gemm_kernel<MT, false, false, SPLIT><<<grid, THREADS, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace

int init_device()
{
    if (set_attr_layouts<1, false>() != cudaSuccess) return 1;
    if (set_attr_layouts<2, false>() != cudaSuccess) return 1;
    if (set_attr_layouts<1, true>() != cudaSuccess) return 1;
    return 0;
}

int try_launch(int math_mode, cudaStream_t st, const float* a, const float* b, float* c, int M, int N,
               int K, int aMs, int aKs, int bKs, int bNs, int batch_count, int batch_rank,
               const int* batch_dims, const int* a_bs, const int* b_bs, const Epilogue& epi,
               int num_sms, unsigned int* status, void* workspace, size_t workspace_bytes,
               int* launches, int forced_mt)
{
    const bool split = math_mode == 4;
    OperandView va, vb;
    const int ak = classify(a, M, K, aMs, aKs, va);
    const int bk = classify(b, N, K, bNs, bKs, vb);
    if (ak < 0 || bk < 0) return 3;
    if (batch_rank > MAX_BATCH_RANK) return 3;

    Params p;
    memset(&p, 0, sizeof(p));
    p.batch.rank = batch_rank;
    for (int i = 0; i < batch_rank; i++) {
        p.batch.dims[i] = batch_dims[i];
        p.batch.a_stride[i] = a_bs[i];
        p.batch.b_stride[i] = b_bs[i];
        p.batch.a_slot[i] = p.batch.b_slot[i] = -1;
    }
    const HostBatch hb{batch_rank, batch_dims, a_bs, b_bs};
    if (!plan_batch(hb, a_bs, p.batch.a_slot, p.batch.a_mult, va)) return 3;
    if (!plan_batch(hb, b_bs, p.batch.b_slot, p.batch.b_mult, vb)) return 3;
    if (!tma_compatible(va) || !tma_compatible(vb)) return 3;

    // Tile shape from a cost model in SM clocks per CTA (shape and SM count only, so the choice --
    // and with it the summation order -- is a function of the call alone).  Measured: a k-tile of
    // a 128-row tile is bound by the operand bytes it pulls through L2 -> SM, about 980 clk for
    // 128 x 256 (48 KB), in proportion for narrower tiles; a 256-row tile (two MMAs per B tile)
    // takes about 1545 clk per k-tile for twice the work.  Reading a 128 x 256 accumulator out
    // takes about 3500 clk: hidden behind the next tile's MMAs in the 128-row form (two accumulator
    // sets), exposed in the 256-row form (one set); handing a tile over costs about 3000 clk.
    //   width:  256 columns unless a narrower tile is cheaper -- N = 192 is one 192-wide tile
    //           instead of a 256-wide one that is a quarter padding, and a grid of few tiles
    //           (1024^3: 32 tiles of 128 x 256) is cut into more, narrower ones to fill the SMs;
    //   height: 256 rows when that is cheaper than the best 128-row form (large products).
    const double k_tiles = (K + BK - 1) / BK;
    const auto waves = [&](int bm, int w) {
        const long long work = static_cast<long long>(batch_count) * ((M + bm - 1) / bm) * ((N + w - 1) / w);
        return static_cast<double>((work + num_sms - 1) / num_sms);
    };
    int bn = 256;
    double t1 = 1e300;
    for (int w : {256, 192, 128, 64}) {
        const double mma = k_tiles * 980.0 * (128 + w) / 384.0, readout = 3500.0 * w / 256.0;
        const double t = waves(128, w) * ((mma > readout ? mma : readout) + 3000.0);
        if (t < t1 * 0.98) { t1 = t; bn = w; }      // a narrower tile has to win by 2 %
    }
    int mt = 1;
    if (!split) {
        const double t2 = waves(256, 256) * (k_tiles * 1545.0 + 7000.0 + 3000.0);
        if (t2 < t1) { mt = 2; bn = 256; }
    }
    if (forced_mt == 1 || forced_mt == 2) { mt = split ? 1 : forced_mt; if (mt == 2) bn = 256; }
    const int bm = 128 * mt;

    OperandView views[4] = {va, vb, va, vb};
    int n_launch = 0;
    if (split) {
        // hi/lo copies of both operands live in the workspace for the duration of the call
        const long long na = operand_span(va), nb = operand_span(vb);
        const long long sa = (na + 3) & ~3ll, sb = (nb + 3) & ~3ll;
        const size_t need = sizeof(float) * static_cast<size_t>(2 * (sa + sb));
        if (need > workspace_bytes) return 3;
        float* ws = static_cast<float*>(workspace);
        float* a_hi = ws;
        float* a_lo = ws + sa;
        float* b_hi = ws + 2 * sa;
        float* b_lo = ws + 2 * sa + sb;
        const int blocks = num_sms * 8;
        split_tf32_kernel<<<blocks, 256, 0, st>>>(a, a_hi, a_lo, na);
        split_tf32_kernel<<<blocks, 256, 0, st>>>(b, b_hi, b_lo, nb);
        n_launch += 2;
        views[0].base = a_hi; views[2].base = a_lo;
        views[1].base = b_hi; views[3].base = b_lo;
    }

    // MN-major operands: all boxes of a k-tile in one instruction when the row axis splits evenly
    const auto can_group = [](const OperandView& v) { return v.dim[0] % 32 == 0 && v.rank <= 4; };
    const auto grouped_view = [](const OperandView& v) {
        OperandView g;
        g.base = v.base;
        g.rank = v.rank + 1;
        g.dim[0] = 32;            g.stride_elems[0] = 1;
        g.dim[1] = v.dim[1];      g.stride_elems[1] = v.stride_elems[1];
        g.dim[2] = v.dim[0] / 32; g.stride_elems[2] = 32;
        for (int i = 2; i < v.rank; i++) { g.dim[i + 1] = v.dim[i]; g.stride_elems[i + 1] = v.stride_elems[i]; }
        return g;
    };
    p.a_grouped = (!ak && can_group(va)) ? 1 : 0;
    p.b_grouped = (!bk && can_group(vb)) ? 1 : 0;
    CUtensorMap maps[5];
    for (int i = 0; i < (split ? 4 : 2); i++) {
        const bool is_a = (i % 2) == 0;
        const bool kmaj = is_a ? ak : bk;
        const int rows_box = is_a ? bm : bn;
        int r;
        if (kmaj) r = encode_tensor_map(&maps[i], views[i], BK, rows_box, Swizzle::B128);
        else if (is_a ? p.a_grouped : p.b_grouped)
            r = encode_tensor_map(&maps[i], grouped_view(views[i]), 32, BK, Swizzle::B128_A32, rows_box / 32);
        else r = encode_tensor_map(&maps[i], views[i], 32, BK, Swizzle::B128_A32);
        if (r != 0) return 3;
    }
    if (!split) { maps[2] = maps[0]; maps[3] = maps[1]; }
    // C through TMA stores when it is a plain (unscattered), 16-byte-aligned tensor
    p.c_tma = 0;
    maps[4] = maps[0];
    if (epi.scatter_rows == 0 && ((reinterpret_cast<uintptr_t>(c) & 15u) == 0) && N % 4 == 0) {
        OperandView vc;
        vc.base = c;
        vc.rank = 3;
        vc.dim[0] = static_cast<uint64_t>(N);           vc.stride_elems[0] = 1;
        vc.dim[1] = static_cast<uint64_t>(M);           vc.stride_elems[1] = static_cast<uint64_t>(N);
        vc.dim[2] = static_cast<uint64_t>(batch_count); vc.stride_elems[2] = static_cast<uint64_t>(M) * static_cast<uint64_t>(N);
        if (tma_compatible(vc) && encode_tensor_map(&maps[4], vc, 32, 32, Swizzle::B128) == 0) p.c_tma = 1;
    }

    p.shape.M = M; p.shape.N = N; p.shape.K = K;
    p.shape.tiles_m = (M + bm - 1) / bm;
    p.shape.tiles_n = (N + bn - 1) / bn;
    p.bn = bn;
    p.shape.batch = batch_count;
    p.shape.work = static_cast<long long>(batch_count) * p.shape.tiles_m * p.shape.tiles_n;
    p.epi = epi;
    p.c = c;
    p.status = status;
    p.c_vec_ok = ((reinterpret_cast<uintptr_t>(c) & 15u) == 0) && (N % 4 == 0);
    const int grid = static_cast<int>(p.shape.work < num_sms ? p.shape.work : num_sms);
    int rc;
    if (split) rc = launch_cfg<1, true>(ak, bk, grid, st, maps, p);
    else if (mt == 2) rc = launch_cfg<2, false>(ak, bk, grid, st, maps, p);
    else rc = launch_cfg<1, false>(ak, bk, grid, st, maps, p);
    if (rc != 0) return rc;
    n_launch += 1;
    if (launches) *launches = n_launch;
    return 0;
}

}  // namespace tf32
}  // namespace tt
