/*
 * tensotron_gemm.h -- C ABI of libtensotron_gemm.so, the B200 (sm_100a) matmul
 * engine that sits behind Tensotron's CUDA backend.
 *
 * Conventions (they follow the reference's existing native call sites, the cuBLAS
 * P/Invoke at src/Tensotron/TensorRuntime.cs:1011-1081):
 *   - cdecl, plain pointers and integers only; every entry returns an int status
 *     (0 = success), the caller throws on non-zero like it does for cuBLAS.
 *   - device pointers are raw addresses owned by the caller; the library never
 *     frees or keeps them.  Element type is float32 everywhere; strides and
 *     offsets are in ELEMENTS and fit int32 (src/Tensotron/TensorRuntime.cs:219).
 *   - `stream` is a CUstream / cudaStream_t passed as void*; NULL is the default
 *     stream.  Every call only enqueues stream-ordered work: no synchronisation,
 *     no allocation, no host-visible side effect, so a call can be re-fired under
 *     stream capture (src/Tensotron/TensorRuntime.cs:596-698).
 *   - single caller thread per handle (README.md:168-170); no internal locking.  One handle
 *     serves ONE stream at a time: its workspace, its split-K / stream-K partial tiles and flags
 *     and its status word are shared by all calls on the handle, so calls that may overlap on the
 *     GPU (two streams) need two handles.
 *   - the handle lives in the CUDA context that is current on the calling thread at tt_create
 *     (the device's primary context only when none is current).  Every later entry runs in that
 *     context: when another context, or none, is current, the handle's context is pushed for the
 *     duration of the call and popped again.
 *   - results are bit-stable from run to run for a given call on a given handle.  Forms that cut
 *     K (small outputs, partial last waves) regroup the sum; whether they are used depends on the
 *     shape, the SM count and the handle's free workspace.
 */
#ifndef TENSOTRON_GEMM_H
#define TENSOTRON_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported entry points (the library is built with hidden default visibility). */
#if defined(_WIN32)
#define TT_API __declspec(dllexport)
#else
#define TT_API __attribute__((visibility("default")))
#endif

typedef struct tt_handle_s* tt_handle_t;

/* status codes */
#define TT_OK 0
#define TT_ERR_INVALID_ARG 1   /* null pointer, negative size, K mismatch, bad mode    */
#define TT_ERR_CUDA 2          /* a CUDA runtime / driver call failed                   */
#define TT_ERR_UNSUPPORTED 3   /* shape / stride combination outside the contract       */
#define TT_ERR_WORKSPACE 4     /* handle workspace too small for the requested variant  */
#define TT_ERR_DEVICE_WAIT 5   /* a bounded device-side wait ran out (see tt_check)     */
#define TT_ERR_STATIC_LIMIT 6  /* size beyond what a *_static entry's built-in scratch holds */
#define TT_ERR_BAD_LABEL 7     /* tt_check: a cross-entropy label was outside [0, classes)   */

/* math modes: 0 and 3 carry the meaning of SetCuBlasMathMode
 * (src/Tensotron/TensorRuntime.cs:332-338: 0 = FP32, 3 = TF32); 4 is new. */
#define TT_MATH_FP32 0    /* strict IEEE float32 FFMA, the default                      */
#define TT_MATH_TF32 3    /* AllowTf32: tcgen05 kind::tf32, fp32 accumulate             */
#define TT_MATH_3XTF32 4  /* three tf32 products per term, recovers ~fp32 accuracy      */
/* The tensor-core modes are permissions, as AllowTf32 is: products with a dimension of at most
 * 16, and in mode 4 single products up to M*N*K = 2^28, run on the strict-FP32 kernels where those
 * are faster (and at least as accurate). */

/* activations fused into the Linear epilogue (src/Tensotron/Ops.Unary.cs:89-105) */
#define TT_ACT_NONE 0
#define TT_ACT_RELU 1
#define TT_ACT_TANH 2

TT_API const char* tt_version(void);

/* Created once next to the cuBLAS handle (src/Tensotron/TensorRuntime.cs:509-510)
 * and destroyed in Dispose (:1402-1415).  `workspace_bytes` sizes the split-K /
 * backward scratch owned by the handle (0 picks a default: 256 MiB).  The handle binds to the
 * context that is current on the calling thread when it belongs to `device`, else to the
 * device's primary context (which is then made current). */
TT_API int tt_create(int device, size_t workspace_bytes, tt_handle_t* out_handle);
TT_API int tt_destroy(tt_handle_t h);

/* Static, human-readable text for the last non-zero status on this handle. */
TT_API const char* tt_last_error(tt_handle_t h);

/* Replaces AllowTf32 / SetCuBlasMathMode (src/Tensotron/TensorRuntime.cs:158-159,
 * :332-338).  Accepts 0, 3, 4 and 1 (cuBLAS's legacy tensor-op math, which the reference's setter
 * also takes: served by the TF32 kernel). */
TT_API int tt_set_math_mode(tt_handle_t h, int mode);
TT_API int tt_get_math_mode(tt_handle_t h, int* mode);

/* Replaces the body of IlgpuRuntime.LaunchMatMul
 * (src/Tensotron/TensorRuntime.cs:242-243 contract, :959-988 implementation):
 *   C[m,n] = sum_k A[m*aMs + k*aKs] * B[n*bNs + k*bKs],  C contiguous (M,N). */
TT_API int tt_matmul(tt_handle_t h, void* stream, const float* a, const float* b, float* c,
              int M, int N, int K, int aMs, int aKs, int bKs, int bNs);

/* Replaces IlgpuRuntime.LaunchMatMulBatched
 * (src/Tensotron/TensorRuntime.cs:252-254 contract, :1149-1211 implementation):
 * the same product per batch entry; the batch index is decoded last-axis-fastest
 * over batchDims and the operand offsets are sum(idx[ax] * stride[ax]) (stride 0 =
 * broadcast).  C is contiguous (batch..., M, N).  The three int arrays are host
 * memory, read during the call and not retained. */
TT_API int tt_matmul_batched(tt_handle_t h, void* stream, const float* a, const float* b, float* c,
                      int batchCount, int M, int N, int K, int aMs, int aKs, int bKs, int bNs,
                      int batchRank, const int* batchDims, const int* aBatchStrides,
                      const int* bBatchStrides);

/* Batched product whose output is summed over some batch axes: what the MatMulND backward
 * closures compute as RawBmm followed by ReduceGradToShape
 * (src/Tensotron/TensorOps.MatMulND.cs:80-103, src/Tensotron/TensorOps.cs:76-100) when an
 * operand was broadcast along batch axes.  reduceAxis[ax] != 0 marks an axis that is summed;
 * C is contiguous over the remaining axes (in order) x (M, N).  The sum runs inside the
 * kernel's k loop in ascending axis order (no temporary of the full batch shape, no
 * atomics).  The summed axes must merge into one strided axis (TT_ERR_UNSUPPORTED
 * otherwise; the caller then uses the unfused path).  Always strict FP32. */
TT_API int tt_matmul_batched_reduce(tt_handle_t h, void* stream, const float* a, const float* b, float* c,
                             int M, int N, int K, int aMs, int aKs, int bKs, int bNs, int batchRank,
                             const int* batchDims, const int* aBatchStrides,
                             const int* bBatchStrides, const int* reduceAxis);

/* ReduceGradToShape (src/Tensotron/TensorOps.cs:76-100): sums a contiguous row-major tensor of
 * `rank` axes (<= 8) over the axes with reduceAxis[ax] != 0; dst is contiguous over the remaining
 * axes in order.  One thread per output walks the summed axes in ascending row-major order (fixed
 * order, no atomics).  The unfused companion of tt_matmul_batched_reduce, for broadcast axes that do
 * not merge into one. */
TT_API int tt_reduce_sum_axes(tt_handle_t h, void* stream, const float* src, float* dst, int rank,
                              const int* dims, const int* reduceAxis);

/* Linear.Forward (+ the Activation module that follows it) as one launch
 * (src/Tensotron/Module.cs:100-105, src/Tensotron/TensorOps.LinearNT.cs:13-25):
 *   y = act(x (M,K) . w (N,K)^T + bias (N)),  bias may be NULL. */
TT_API int tt_linear_fwd(tt_handle_t h, void* stream, const float* x, const float* w, const float* bias,
                  float* y, int M, int N, int K, int act);

/* Backward of the same (src/Tensotron/TensorOps.LinearNT.cs:27-48,
 * src/Tensotron/TensorOps.cs:143-147, src/Tensotron/Ops.Unary.cs:89-105):
 *   g  = dy * act'(y)            (ReLU: y>0 ? dy : 0;  Tanh: dy*(1-y*y))
 *   dx = g . w        (M,K)  NN  -- skipped when dx is NULL
 *   dw = g^T . x      (N,K)  TN
 *   dbias[n] = sum_m g[m,n]  in a fixed order (no atomics) -- skipped when NULL
 * Outputs are written, not accumulated (accumulation stays with Tensor.AddGrad).
 * When act != TT_ACT_NONE the masked gradient g needs M*N floats of the handle
 * workspace.  Layers up to M*N*K = 2^21 run as ONE launch (g formed on the fly, no
 * workspace); larger ones as three (activation backward + column sums, dx, dw). */
TT_API int tt_linear_bwd(tt_handle_t h, void* stream, const float* x, const float* w, const float* y,
                  const float* dy, float* dx, float* dw, float* dbias, int M, int N, int K, int act);

/* CrossEntropy(mean-style) forward+backward in one launch
 * (src/Tensotron/TensorOps.Losses.cs:97-108, src/Tensotron/TensorOps.Reduce.cs:122-141):
 * labels are device int32 in [0, classes); dlogits = (softmax - onehot) * scale; *loss (device
 * float) = scale * sum_rows(-log softmax[label]); row sums are reduced in a fixed
 * order.  `loss` and `dlogits` may each be NULL.  A label outside the range is never used as an
 * index: that row's loss (and so *loss) becomes NaN, its gradient is the plain softmax, and
 * tt_check reports TT_ERR_BAD_LABEL (the reference throws on the host for such a target). */
TT_API int tt_softmax_cross_entropy(tt_handle_t h, void* stream, const float* logits, const int* labels,
                             float* dlogits, float* loss, int rows, int classes, float scale);

/* MseLoss (mean reduction) forward + backward in one pass
 * (src/Tensotron/TensorOps.Losses.cs:29-61): *loss = sum((input - target)^2) / count and
 * dinput = (2 / count) * (input - target); sums in a fixed two-level order.  `loss` and
 * `dinput` may each be NULL.  Needs 8 KiB of the handle workspace. */
TT_API int tt_mse_loss(tt_handle_t h, void* stream, const float* input, const float* target, float* dinput,
                       float* loss, long long count);

/* GradUtils.ClipGradNorm over one flat gradient span (src/Tensotron/Optimizers.cs:383-422):
 * norm = sqrt(sum g^2) (fixed-order sum), every g scaled by clamp(max_norm / (norm + eps), 0, 1)
 * unconditionally; *norm_out (device float, optional) receives the pre-clip norm, so nothing
 * synchronises.  Needs 8 KiB of the handle workspace. */
TT_API int tt_clip_grad_norm(tt_handle_t h, void* stream, float* grads, long long n, float max_norm, float eps,
                             float* norm_out);

/* Conv2d through the batched GEMM engine (src/Tensotron/TensorOps.Conv.cs:60-80: Im2Col, then
 * MatMul((1, O, K), (N, K, L)), then the broadcast bias add; K = C*kh*kw, L = Ho*Wo; symmetric
 * stride / padding / dilation as there).  x (N,C,H,W), w (O,C,kh,kw), bias (O) or NULL,
 * y (N,O,Ho,Wo), all contiguous.  The columns and the packed weights live in the handle workspace
 * (tt_conv2d_workspace bytes; TT_ERR_WORKSPACE when it is smaller); the bias rides in the GEMM as
 * one extra k term, so forward is im2col + weight packing + ONE batched GEMM launch.
 * Backward (what the reference's autograd chain computes: Kernels.Col2Im, src/Tensotron/Kernels.cs:803-814;
 * the broadcast-reduced dW of src/Tensotron/TensorOps.MatMulND.cs:80-103):
 *   dbias[o] = sum_{n,l} dy      dw = sum_n dy[n] . col[n]^T      dx = col2im(w^T . dy[n])
 * every sum in a fixed order, no atomics (col2im gathers).  dx and dbias may be NULL.  The math
 * mode of the handle applies to the GEMMs. */
typedef struct tt_conv2d_desc {
    int n, c, h, w;          /* input  (N, C, H, W)           */
    int o, kh, kw;           /* weight (O, C, kh, kw)         */
    int stride, padding, dilation;
} tt_conv2d_desc;
TT_API size_t tt_conv2d_workspace(const tt_conv2d_desc* d, int backward);
TT_API int tt_conv2d_fwd(tt_handle_t h, void* stream, const tt_conv2d_desc* d, const float* x, const float* w,
                         const float* bias, float* y);
TT_API int tt_conv2d_bwd(tt_handle_t h, void* stream, const tt_conv2d_desc* d, const float* x, const float* w,
                         const float* dy, float* dx, float* dw, float* dbias);

/* Same result as tt_softmax_cross_entropy, for callers that may not allocate device
 * memory.  No counterpart in the reference: there the per-row losses live in tensors from
 * its own allocator.  It takes no handle (tt_create allocates) and keeps the per-row losses
 * in an array built into the library image, which every GPU that loads the library holds
 * until exit (TT_STATIC_CE_MAX_ROWS floats).  rows above that limit are refused with
 * TT_ERR_STATIC_LIMIT.  The call runs on the current device; its first call on a device
 * looks the array's address up, so make that call before any stream capture.  All calls
 * share the array: calls that overlap on the GPU race on it.  A label outside [0, classes)
 * makes *loss NaN (there is no handle to report it through). */
#define TT_STATIC_CE_MAX_ROWS 65536
TT_API int tt_softmax_cross_entropy_static(void* stream, const float* logits, const int* labels,
                                    float* dlogits, float* loss, int rows, int classes, float scale);

/* Fused Adam over one flat parameter span (src/Tensotron/Kernels.cs:126-157,
 * src/Tensotron/Optimizers.cs:144-193).  adv = device [t, 1/(1-b1^t), 1/(1-b2^t)];
 * when `advance` is non-zero the step counter is advanced on the device first, so a
 * captured step keeps its bias correction moving across replays. */
TT_API int tt_adam_step(tt_handle_t h, void* stream, float* p, const float* g, float* m, float* v,
                 float* adv, long long n, float beta1, float beta2, float lr, float eps,
                 float coupled_wd, float decoupled_factor, int advance);

/* The whole training step of a small MLP -- forward, loss, backward, gradient-norm clip, Adam --
 * as ONE launch (a thread-block cluster; everything stays in shared memory).  It replaces the
 * op-by-op step the reference captures for its control / PPO-sized networks
 * (examples/Tensotron.Examples/BenchExample.cs:140-193: Sequential(Linear, Tanh, Linear, Tanh,
 * Linear) + MseLoss + ZeroGrad + Backward + ClipGradNorm + Adam.Step; nets of
 * showcase/Tensotron.Showcase/Rl/ActorCritic.cs:21-32), which is launch-bound there.
 *   net      n_layers Linear layers (1..TT_MLP_MAX_LAYERS) of widths dims[0] -> ... -> dims[n_layers],
 *            every width 1..64; `act` after every layer but the last; loss TT_LOSS_MSE (mean over
 *            batch x outputs, src/Tensotron/TensorOps.Losses.cs:29-61; target = float (batch, out))
 *            or TT_LOSS_CE (softmax cross-entropy, mean over the batch; target = int32 labels)
 *   params, m, v   flat buffers, layer by layer: W_l (out, in) row-major, then b_l, each layer padded
 *            to a multiple of 4 floats (16-byte aligned bases)
 *   adv      [t, 1/(1-b1^t), 1/(1-b2^t)] as in tt_adam_step; always advanced on the device
 *   grads_out  optional: receives the (clipped) gradients in the flat layout
 *   loss_out   optional: device float, the loss before the update
 *   max_grad_norm > 0: ClipGradNorm (src/Tensotron/Optimizers.cs:394-416): every gradient is
 *            scaled by clamp(max_grad_norm / (norm + clip_eps), 0, 1); <= 0: no clipping
 * batch up to 1024 rows.  All sums run in a fixed order that depends on the batch size only, so
 * results are bit-stable from run to run.  TT_ERR_UNSUPPORTED when the network or the batch does
 * not fit (the caller then runs the step layer by layer with the entries above). */
#define TT_MLP_MAX_LAYERS 4
#define TT_LOSS_MSE 0
#define TT_LOSS_CE 1
typedef struct tt_mlp_desc {
    int n_layers;
    int dims[TT_MLP_MAX_LAYERS + 1];
    int act;   /* TT_ACT_* */
    int loss;  /* TT_LOSS_* */
} tt_mlp_desc;
TT_API int tt_mlp_train_step(tt_handle_t h, void* stream, const tt_mlp_desc* net, float* params, float* m,
                             float* v, float* adv, float* grads_out, const float* x, const void* target,
                             float* loss_out, int batch, float lr, float beta1, float beta2, float eps,
                             float max_grad_norm, float clip_eps);

/* target[i] += source[i]  (Kernels.AddInto, src/Tensotron/Kernels.cs:111-114). */
TT_API int tt_add_into(tt_handle_t h, void* stream, float* target, const float* source, long long n);

/* BroadcastBatch of TensorOps.MatMulND (src/Tensotron/TensorOps.MatMulND.cs:11-31):
 * right-aligns the two batch shapes, returns the broadcast dims and per-operand
 * element strides (0 on broadcast axes).  Pure host logic.  Returns
 * TT_ERR_INVALID_ARG when the shapes do not broadcast.  *rank = max(ra, rb). */
TT_API int tt_broadcast_batch(int ra, const int* a_dims, const int* a_strides, int rb, const int* b_dims,
                       const int* b_strides, int* rank, int* dims, int* a_bs, int* b_bs);

/* The multi-GPU forms of LaunchMatMul / LaunchMatMulBatched shard the rows of A and C (or the
 * outermost batch axis) over one process per GPU with the other operand replicated: every rank
 * calls tt_matmul / tt_matmul_batched on its own shard, there is no collective on the data path.
 * This is the split every rank uses: `total` units cut into `world` contiguous blocks of
 * ceil(total / world) (the row split of the reference's ParallelRows,
 * src/Tensotron/CpuKernels.cs:461-472); *start / *count describe block `rank` (count may be 0).
 * Pure host logic. */
TT_API int tt_shard_range(long long total, int world, int rank, long long* start, long long* count);

/* Counters in the spirit of TensorRuntime.Launches (src/Tensotron/TensorRuntime.cs:143-151). */
typedef struct tt_stats {
    long long launches;        /* kernels enqueued by this handle                        */
    long long calls;           /* C-ABI compute calls                                     */
    long long simt_tma;        /* calls served by the TMA-fed FP32 FFMA kernel            */
    long long tcgen05;         /* calls served by the tcgen05 TF32 / 3xTF32 kernel        */
    long long generic;         /* calls served by the any-stride kernel                   */
    long long splitk;          /* calls that used the split-K workspace                   */
    long long skinny;          /* calls served by the tiny-dimension streaming kernels    */
    long long workspace_bytes; /* size of the handle workspace                            */
    long long tensor_map_hits;   /* TMA descriptors served from the calling thread's cache  */
    long long tensor_map_misses; /* TMA descriptors encoded (cuTensorMapEncodeTiled)        */
} tt_stats;
TT_API int tt_get_stats(tt_handle_t h, tt_stats* out);
TT_API int tt_reset_stats(tt_handle_t h);

/* Reads the device-side status word (bounded waits that gave up).  This call
 * synchronises the stream; it is for tests and debugging, not the hot path. */
TT_API int tt_check(tt_handle_t h, void* stream);

/* Forces a kernel variant for A/B measurements: 0 auto, 1 any-stride kernel,
 * 2 TMA-fed FFMA kernel with 256x128 tiles, 3 the same with 128x128 tiles,
 * 4 / 5 tcgen05 kernel (TF32 modes only) with 128- / 256-row tiles,
 * 6 FFMA kernel with 256x128 tiles and stream-K work distribution,
 * 7 FFMA kernel with 128x192 tiles (B contiguous along N only),
 * 8 any-stride kernel with its K ranges added through the workspace (two launches) instead of
 *   through a thread-block cluster,
 * 9 FFMA kernel with 128x128 tiles and stream-K work distribution,
 * 10 automatic, but tall products with N <= 16 keep the K-cut streaming kernel instead of the
 *   TMA-fed one. */
TT_API int tt_set_variant(tt_handle_t h, int variant);

/* ---- Data-parallel gradient exchange over peer memory ---------------------------------
 *
 * No counterpart in the reference, which runs on one GPU: this is the multi-GPU form of its
 * Linear backward + Adam step (src/Tensotron/TensorOps.LinearNT.cs:31-52,
 * src/Tensotron/Optimizers.cs:144-193).  One process per GPU; every rank maps every other
 * rank's buffers through CUDA IPC and the kernels load / store peer memory directly (NVLink).
 *
 * Buffers (each allocated with tt_peer_alloc on its own rank, zero-filled, exported with
 * tt_peer_export, opened on the other ranks with tt_peer_open), n = floats of the flat
 * parameter buffer:
 *   stage   world x n floats  slot s = gradients produced by rank s; this rank's own slot
 *                             (stage + rank * n) is its local gradient buffer
 *   params  n floats          flat parameters
 *   flags   TT_PEER_FLAG_WORDS x uint32  arrival flags and the step counter, zero at the start
 * Row ownership: rows [o * own_rows, (o + 1) * own_rows) of a weight matrix belong to rank o
 * (own_rows a multiple of 256).  The owner sums the world slots in ascending rank order, runs
 * Adam on its rows and stores the new rows into every rank's params; small segments
 * (biases, narrow layers) are replicated: pushed to everybody, summed and updated identically
 * everywhere.  All ranks hold bit-identical parameters after every step.
 *
 * Every wait on another GPU is bounded (5 s); a wait that gives up records a code that
 * tt_check returns as TT_ERR_DEVICE_WAIT.  The step number lives in device memory (a word of
 * `flags`), none of these calls allocates or synchronises, and a step's calls take the same
 * arguments every step.  All ranks must issue the same sequence of tt_peer_* calls. */
#define TT_MAX_PEERS 8
#define TT_MAX_SEGMENTS 16
#define TT_IPC_HANDLE_BYTES 64
typedef struct tt_peer_group_s* tt_peer_group_t;

TT_API int tt_peer_alloc(tt_handle_t h, size_t bytes, void** out_ptr);
TT_API int tt_peer_free(tt_handle_t h, void* ptr);
TT_API int tt_peer_export(tt_handle_t h, void* ptr, unsigned char* handle_out /* TT_IPC_HANDLE_BYTES */);
TT_API int tt_peer_open(tt_handle_t h, const unsigned char* handle, void** out_ptr);
TT_API int tt_peer_close(tt_handle_t h, void* ptr);

/* stage / params / flags: world pointers each, entry r = rank r's buffer as mapped in this
 * process (entry `rank` is the local allocation).  world <= TT_MAX_PEERS. */
TT_API int tt_peer_group_create(tt_handle_t h, int world, int rank, long long n, void* const* stage,
                                void* const* params, void* const* flags, tt_peer_group_t* out);
TT_API int tt_peer_group_destroy(tt_peer_group_t g);
/* Upper bound of one wait for another rank's flag (default 5000 ms). */
TT_API int tt_peer_set_wait_limit(tt_peer_group_t g, int milliseconds);

/* tt_linear_bwd whose weight gradient (N x K, at float offset w_off of the flat buffer) is
 * stored row block by row block into the owners' slots for this rank, straight from the GEMM
 * epilogue (stream-K FFMA kernel in strict FP32, tcgen05 kernel in the TF32 modes); when the
 * shape is outside those kernels it is computed into the local slot and copied to the owners.
 * The bias gradient (b_off >= 0) goes to the local slot.  own_rows = 0: the whole weight
 * gradient goes to the local slot (a replicated layer).  *fused (optional) reports whether
 * the epilogue did the scatter. */
TT_API int tt_peer_linear_bwd(tt_handle_t h, void* stream, tt_peer_group_t g, const float* x, const float* w,
                              const float* y, const float* dy, float* dx, long long w_off, long long b_off,
                              int M, int N, int K, int act, int own_rows, int* fused);

/* Channels.  The exchange of a step can be cut into up to TT_PEER_CHANNELS independent parts
 * (one per layer): each channel has its own arrival flags, so the optimizer step of one layer
 * (and the NVLink traffic of its updated rows) can run while the backward pass of the layers
 * below it is still computing.  A step's first tt_peer_push passes new_step = 1 (it advances the
 * step counter); the other pushes of the step pass 0. */
#define TT_PEER_CHANNELS 8
#define TT_PEER_FLAG_WORDS 256   /* uint32 words of a `flags` buffer */

/* Ends the gradient production of one channel: copies the replicated segments (float offsets /
 * lengths, multiples of 4, at most TT_MAX_SEGMENTS) of the local slot to every other rank, then
 * tells every rank that this rank's gradients of this channel and step have been stored. */
TT_API int tt_peer_push(tt_handle_t h, void* stream, tt_peer_group_t g, int channel, int new_step, int n_segments,
                        const long long* offsets, const long long* lengths);

/* Waits for every rank's gradients of the channel, sums the slots, runs Adam (arguments as
 * tt_adam_step) on the owned segments (result stored to every rank's params) and on the
 * replicated segments (result stored locally) and tells the other ranks.  m, v: n floats each,
 * local.  advance = 1 on the first optimizer call of a step only. */
TT_API int tt_peer_adam_step(tt_handle_t h, void* stream, tt_peer_group_t g, int channel, int n_owned,
                             const long long* owned_off, const long long* owned_len, int n_repl,
                             const long long* repl_off, const long long* repl_len, float* m, float* v, float* adv,
                             float beta1, float beta2, float lr, float eps, float coupled_wd,
                             float decoupled_factor, int advance);

/* Ends a step: waits until every rank's updated rows of channels 0 .. n_channels-1 of this step
 * have arrived in this rank's params (must precede the next forward pass, and the next step's
 * stores into the slots). */
TT_API int tt_peer_sync(tt_handle_t h, void* stream, tt_peer_group_t g, int n_channels);

#ifdef __cplusplus
}
#endif
#endif /* TENSOTRON_GEMM_H */
