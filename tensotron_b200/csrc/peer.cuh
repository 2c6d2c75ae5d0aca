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
// One step on every rank, all on one stream, per channel:
//   backward GEMMs (scatter epilogue) -> push (copy the replicated segments, signal "gradients
//   stored") -> reduce_adam (wait for every rank's signal, sum the slots in rank order, Adam,
//   store parameters to all ranks, signal "rows updated") ... -> wait(rows updated, all channels)
// A signal comes after the stores it announces: a later kernel in stream order for the GEMM
// epilogue's stores, a system-scope fence + CTA barrier (+ a last-block-done counter) for the
// stores of its own kernel; it stores the step number into every rank's flag word.  A wait
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
constexpr int DONE_COUNTER_WORD = STEP_COUNTER_WORD + 1;   // + channel: blocks of reduce_adam that have finished
constexpr int PUSH_SINGLE_BLOCK_MAX4 = 32768;              // replicated segments up to this many float4s: one kernel
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

// Polls flags[s] until it has reached `epoch` (wrap-safe), at most limit_ns.  Returns false
// (after recording DEV_WAIT_PEER in *status) when the limit ran out.
__device__ __forceinline__ bool wait_flag(const unsigned int* flags, int s, unsigned int epoch,
                                          unsigned int* status, unsigned long long limit_ns)
{
    const unsigned long long t0 = global_timer_ns();
    unsigned int spins = 0;
    for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + s) : "memory");
        if (static_cast<int>(v - epoch) >= 0) return true;
        if ((++spins & 255u) == 0 && global_timer_ns() - t0 > limit_ns) {
            atomicCAS(status, 0u, static_cast<unsigned int>(DEV_WAIT_PEER));
            return false;
        }
        __nanosleep(200);
    }
}

// push_segments_kernel + signal_kernel in one launch of one block, for small segment lists
// (biases, narrow layers): copy, fence, CTA barrier, flags.
__global__ void __launch_bounds__(1024)
push_signal_kernel(const float* __restrict__ src, PeerPtrs dst, int world, SegList segs, long long total4,
                   FlagPtrs flags, unsigned int* step_counter, int advance)
{
    __shared__ unsigned int s_epoch;
    if (threadIdx.x == 0) {
        unsigned int e = *step_counter;
        if (advance) *step_counter = ++e;
        s_epoch = e;
    }
    for (long long i = threadIdx.x; i < total4; i += blockDim.x) {
        const long long at = seg_locate(segs, i);
        const float4 v = reinterpret_cast<const float4*>(src)[at];
        for (int o = 0; o < world; o++)
            if (dst.p[o]) reinterpret_cast<float4*>(dst.p[o])[at] = v;
    }
    __threadfence_system();
    __syncthreads();
    const int o = threadIdx.x;
    if (o < world && flags.p[o]) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[o]), "r"(s_epoch) : "memory");
    }
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
    (void)wait_flag(flags, s, *step_counter, status, limit_ns);
    __threadfence_system();
}

// The optimizer step of one channel, one launch:
//  1. every block waits (bounded) until all ranks' gradients of the channel have been stored;
//  2. for every element of the owned segments: g = sum over slots 0..world-1 (ascending) of
//     stage[slot][i], Adam on (p, m, v), and the new p goes to every rank's parameter buffer
//     (params.p[o], all o; this rank's own copy included).  Replicated segments: same sum and
//     update, stored to this rank's copy only.  The arithmetic per element is ew::adam_one, so
//     with world == 1 the result equals ew::adam_step_kernel bit for bit;
//  3. the last block to finish tells every rank that this rank's rows are updated, and, when
//     `advance` is set (first optimizer call of a step), stores the step's bias corrections:
//     adv = [t, 1/(1-b1^t), 1/(1-b2^t)] with the expressions of ew::adam_advance_kernel.  With
//     `advance` every block computes the same corrections for itself from adv[0] + 1.
__global__ void __launch_bounds__(256)
reduce_adam_kernel(const float* __restrict__ stage, long long n, int world, int rank, PeerPtrs params,
                   float* __restrict__ m, float* __restrict__ v, float* adv, int advance,
                   SegList owned, long long owned4, SegList repl, long long repl4, float b1, float b2,
                   float lr, float eps, float cwd, float dfac, const unsigned int* wait_flags,
                   const unsigned int* step_counter, unsigned int* status, unsigned long long limit_ns,
                   FlagPtrs signal, unsigned int* done_counter)
{
    __shared__ unsigned int s_last, s_bad;
    if (threadIdx.x == 0) s_bad = 0u;
    __syncthreads();
    if (threadIdx.x < world && !wait_flag(wait_flags, threadIdx.x, *step_counter, status, limit_ns)) atomicOr(&s_bad, 1u);
    __syncthreads();
    // A rank that never signalled (or any error already recorded on this handle: another block of
    // this launch may be the one whose wait ran out) ends the step here: no sum over slots that
    // may be stale, no Adam, nothing stored to any rank, no "rows updated" signal.  The block is
    // still counted, so that the last one resets the counter for the next launch.
    if (threadIdx.x == 0 && *reinterpret_cast<volatile unsigned int*>(status) != 0u) s_bad = 1u;
    __syncthreads();
    const bool bad = s_bad != 0u;
    float t = adv[0], ibc1 = adv[1], ibc2 = adv[2];
    if (advance) {
        t += 1.f;
        ibc1 = 1.f / (1.f - powf(b1, t));
        ibc2 = 1.f / (1.f - powf(b2, t));
    }
    const float omb1 = 1.f - b1, omb2 = 1.f - b2;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    float* own = params.p[rank];
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; !bad && i < owned4 + repl4; i += stride) {
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
    // last block done: every thread's stores are fenced before its block is counted
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int done = atomicAdd(done_counter, 1u);
        s_last = (done == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    // (a block that gave up recorded its code before it was counted: the last block sees it)
    const bool failed = *reinterpret_cast<volatile unsigned int*>(status) != 0u;
    if (threadIdx.x == 0) {
        *done_counter = 0u;
        if (advance && !failed) { adv[0] = t; adv[1] = ibc1; adv[2] = ibc2; }
    }
    const int o = threadIdx.x;
    if (!failed && o < world && signal.p[o]) {
        const unsigned int e = *step_counter;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(signal.p[o]), "r"(e) : "memory");
    }
}

}  // namespace peer
}  // namespace tt
