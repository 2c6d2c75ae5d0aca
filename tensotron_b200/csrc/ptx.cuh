// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (bulk tensor copies, always
// CTA-local destinations), and a bounded wait that gives up instead of hanging.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tt {

// Device-side status word values (written once, first error wins).
enum : unsigned int {
    DEV_OK = 0,
    DEV_WAIT_FULL = 1,    // consumer gave up waiting for a TMA-filled stage
    DEV_WAIT_EMPTY = 2,   // producer gave up waiting for a free stage
    DEV_WAIT_MMA = 3,     // epilogue gave up waiting for tcgen05 completion
    DEV_WAIT_TMEM = 4,    // MMA issuer gave up waiting for a drained accumulator
    DEV_WAIT_PEER = 5,    // a wait for another GPU's flag (gradient / parameter exchange) gave up
    DEV_WAIT_STREAMK = 6, // a stream-K CTA gave up waiting for a neighbour's partial tile
    DEV_BAD_LABEL = 7,    // cross-entropy met a label outside [0, classes)
};

// Upper bound on one wait, in nanoseconds of %globaltimer.  The longest legitimate
// wait is one output tile of the largest supported K (tens of milliseconds).
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for `parity` on `bar`.  Returns false (after recording `code` in *status and
// raising the CTA-wide abort flag) when the wait exceeds WAIT_LIMIT_NS or another
// role of this CTA already aborted; callers then leave their loops.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile uint32_t* cta_abort,
                                                  unsigned int* status, unsigned int code)
{
    if (mbar_try_wait(bar, parity)) return true;
    // The timer is only consulted once a wait has been spinning for a while: reading
    // %globaltimer is slow and most waits end within a few polls.
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3FFu) == 0) {
            if (*cta_abort) return false;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > WAIT_LIMIT_NS) {
                *cta_abort = 1u;
                if (status) atomicCAS(status, 0u, code);
                return false;
            }
        }
    }
    return true;
}

// On the way out after a wait gave up: waits for `parity` on `bar` for at most DRAIN_LIMIT_NS,
// whatever the abort flag says.  A thread uses it for the asynchronous copies or MMAs it issued
// itself, so that the CTA does not release its shared memory or TMEM under them.
constexpr unsigned long long DRAIN_LIMIT_NS = 200000000ull;
__device__ __forceinline__ bool mbar_wait_drain(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xFFu) == 0 && global_timer_ns() - t0 > DRAIN_LIMIT_NS) return false;
    }
    return true;
}

// 5-D tiled TMA load, global -> this CTA's shared memory, completion on `bar`.
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3), "r"(c4)
        : "memory");
}

// 5-D tiled TMA store (the tensor maps built here always have rank 5, and the instruction's
// dimensionality has to equal the map's rank), this CTA's shared memory -> global, clipped at the
// tensor's extents, tracked by the issuing thread's bulk async-group.  c0 a multiple of 4 floats.
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2,
                                             int c3, int c4)
{
    asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
                 ::"l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the issuing thread's bulk stores have finished reading shared memory ...
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... until all but the most recent one have ...
__device__ __forceinline__ void bulk_wait_group_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// ... and until they are complete.
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Register reallocation between the warpgroups of a CTA (all threads of a warpgroup execute
// the same one): the producer warpgroup hands registers back, the consumers take them.
template <int REGS>
__device__ __forceinline__ void setmaxnreg_dec()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void setmaxnreg_inc()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}

__device__ __forceinline__ float4 lds128(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr));
    return v;
}

}  // namespace tt
