// Gradient exchange between the GPUs of one node over peer memory (NVLink), for the
// data-parallel training step.  Every rank maps every other rank's buffers (CUDA IPC); the
// kernels here use plain loads and stores on those addresses.
//
// Layout per rank (n = floats in the flat parameter / gradient buffer, world <= 8 ranks):
//   stage   world x n floats   slot s holds the gradients rank s produced, as far as this rank
//                              needs them: the rows of the weight matrices this rank owns
//                              (stored there by rank s's weight-gradient GEMM, tile by tile)
//                              and the small replicated segments (pushed by push_segments)
//   params  n floats           the parameters; owners store updated rows into every rank's copy
//   flags   256 words          channel c (0..7): [16c + s]: gradients of channel c, step e, from
//                              rank s have landed (value e); [16c + 8 + s]: rank s's rows of
//                              channel c are updated for step e;
//                              [128]: this rank's step counter e (device-resident, so that the
//                              calls of a step carry no per-step host state and a captured
//                              graph of the step can be replayed)
// A channel is an independent part of the exchange (a layer): its optimizer step can run, and
// its updated rows can travel, while the backward pass of the layers below is still computing.
//
// One step on every rank, all on one stream:
//   backward GEMMs (scatter epilogue) -> push_segments -> signal(grads) ->
//   wait(grads) -> reduce_adam (sum the slots in rank order, Adam, store parameters to all
//   ranks) -> signal(params) -> wait(params)
// A signal is a kernel that runs after the kernels whose stores it announces (stream order),
// fences at system scope and stores the step number into every rank's flag word.  A wait
// spins with a time limit and records DEV_WAIT_PEER in the status word when it gives up, so
// a missing rank ends in an error code, not a hang.  The sums run in ascending rank order on
// the one rank that owns the element (or identically on every rank for the replicated
// segments): all ranks hold bit-identical parameters after every step.
#pragma once
#include <stdint.h>

#include "elementwise.cuh"
#include "gemm_common.h"
#include "ptx.cuh"

namespace tt {
namespace peer {

constexpr int MAX_SEGS = 16;
constexpr int CHANNELS = 8;
constexpr int CHANNEL_WORDS = 2 * MAX_PEERS;           // grads flags, params flags
constexpr int STEP_COUNTER_WORD = CHANNELS * CHANNEL_WORDS;
constexpr int FLAG_WORDS = 256;
constexpr unsigned long long PEER_WAIT_LIMIT_NS = 5000000000ull;   // default limit of one wait: 5 s

// Segments of the flat buffer: float offsets and lengths, all multiples of 4 (128-bit accesses).
struct SegList {
    int n;
    long long off[MAX_SEGS];
    long long len[MAX_SEGS];
};

struct PeerPtrs {
    float* p[MAX_PEERS];
};

struct FlagPtrs {
    unsigned int* p[MAX_PEERS];
};

// Segment lookup for a linear float4 index over the concatenated segments.
__device__ __forceinline__ long long seg_locate(const SegList& s, long long i4)
{
    for (int k = 0; k < s.n; k++) {
        const long long l4 = s.len[k] >> 2;
        if (i4 < l4) return (s.off[k] >> 2) + i4;
        i4 -= l4;
    }
    return -1;
}

// Copies the listed segments of this rank's own slot into this rank's slot on every other
// rank (dst.p[o] = base of that slot as mapped here, null for o == rank).
__global__ void __launch_bounds__(256)
push_segments_kernel(const float* __restrict__ src, PeerPtrs dst, int world, SegList segs, long long total4)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total4; i += stride) {
        const long long at = seg_locate(segs, i);
        const float4 v = reinterpret_cast<const float4*>(src)[at];
        for (int o = 0; o < world; o++)
            if (dst.p[o]) reinterpret_cast<float4*>(dst.p[o])[at] = v;
    }
}

// dst[i] = src[i] for n4 float4s (row blocks of a gradient computed locally, sent to their owner).
__global__ void __launch_bounds__(256)
copy_to_peer_kernel(const float* __restrict__ src, float* __restrict__ dst, long long n4)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride)
        reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
}

// Thread o stores this rank's step number into flag word dst.p[o] (already offset to this
// rank's word).  advance = 1: the step counter is incremented first (start of an exchange).
__global__ void signal_kernel(FlagPtrs dst, int world, unsigned int* step_counter, int advance)
{
    __shared__ unsigned int s_epoch;
    if (threadIdx.x == 0) {
        unsigned int e = *step_counter;
        if (advance) *step_counter = ++e;
        s_epoch = e;
    }
    __syncthreads();
    __threadfence_system();
    const int o = threadIdx.x;
    if (o < world && dst.p[o]) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst.p[o]), "r"(s_epoch) : "memory");
    }
}

// Warp c, lane s waits until flags[c * CHANNEL_WORDS + s] has reached this rank's step number
// (wrap-safe comparison), at most limit_ns.  One warp per channel waited for.
__global__ void wait_kernel(const unsigned int* flags, int world, const unsigned int* step_counter,
                            unsigned int* status, unsigned long long limit_ns)
{
    const int s = threadIdx.x & 31;
    if (s >= world) return;
    flags += (threadIdx.x >> 5) * CHANNEL_WORDS;
    const unsigned int epoch = *step_counter;
    const unsigned long long t0 = global_timer_ns();
    unsigned int spins = 0;
    for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + s) : "memory");
        if (static_cast<int>(v - epoch) >= 0) break;
        if ((++spins & 255u) == 0 && global_timer_ns() - t0 > limit_ns) {
            atomicCAS(status, 0u, static_cast<unsigned int>(DEV_WAIT_PEER));
            break;
        }
        __nanosleep(200);
    }
    __threadfence_system();
}

// For every element of the owned segments: g = sum over slots 0..world-1 (ascending) of
// stage[slot][i], Adam on (p, m, v), and the new p goes to every rank's parameter buffer
// (params.p[o], all o; this rank's own copy included).  Replicated segments: same sum and
// update, stored to this rank's copy only.  The arithmetic per element is ew::adam_one, so
// with world == 1 the result equals ew::adam_step_kernel bit for bit.
__global__ void __launch_bounds__(256)
reduce_adam_kernel(const float* __restrict__ stage, long long n, int world, int rank, PeerPtrs params,
                   float* __restrict__ m, float* __restrict__ v, const float* __restrict__ adv,
                   SegList owned, long long owned4, SegList repl, long long repl4, float b1, float b2,
                   float lr, float eps, float cwd, float dfac)
{
    const float ibc1 = adv[1], ibc2 = adv[2];
    const float omb1 = 1.f - b1, omb2 = 1.f - b2;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    float* own = params.p[rank];
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < owned4 + repl4; i += stride) {
        const bool is_owned = i < owned4;
        const long long at = is_owned ? seg_locate(owned, i) : seg_locate(repl, i - owned4);
        float4 g = reinterpret_cast<const float4*>(stage)[at];
        for (int s = 1; s < world; s++) {
            const float4 q = reinterpret_cast<const float4*>(stage + s * n)[at];
            g.x += q.x; g.y += q.y; g.z += q.z; g.w += q.w;
        }
        float4 pp = reinterpret_cast<const float4*>(own)[at];
        float4 mm = reinterpret_cast<float4*>(m)[at];
        float4 vv = reinterpret_cast<float4*>(v)[at];
        ew::adam_one(pp.x, g.x, mm.x, vv.x, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
        ew::adam_one(pp.y, g.y, mm.y, vv.y, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
        ew::adam_one(pp.z, g.z, mm.z, vv.z, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
        ew::adam_one(pp.w, g.w, mm.w, vv.w, b1, omb1, b2, omb2, lr, eps, ibc1, ibc2, cwd, dfac);
        reinterpret_cast<float4*>(m)[at] = mm;
        reinterpret_cast<float4*>(v)[at] = vv;
        if (is_owned) {
            for (int o = 0; o < world; o++) reinterpret_cast<float4*>(params.p[o])[at] = pp;
        } else {
            reinterpret_cast<float4*>(own)[at] = pp;
        }
    }
}

}  // namespace peer
}  // namespace tt
