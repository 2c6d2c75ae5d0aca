// tt_softmax_cross_entropy_static: the cross-entropy entry point for callers that must
// not allocate device memory.
//
// The regular entry (tt_softmax_cross_entropy) parks its per-row losses in the workspace
// a handle obtained from tt_create owns, and tt_create calls cudaMalloc.  Some hosts cannot
// go that way: a runtime whose own pool allocator has claimed the device heap and does not
// tolerate foreign allocations, or a component that is only handed a stream and buffers and
// has no say over device memory at all.  For them the same two kernels run here against a
// scratch array that is part of the library image: it exists on every GPU that loads the
// library, from load until the process exits, and costs TT_STATIC_CE_MAX_ROWS floats
// (256 KiB) there.
//
// Host code cannot pass the array's name to a kernel (on the host the name is only a
// stand-in); the device address is looked up once per device (per CUDA context on it)
// with cudaGetSymbolAddress while that device is current.  The first call on a device performs
// that look-up, so make it before starting any stream capture.  Nothing here calls cudaMalloc, cudaFree or an
// allocating library routine.
//
// The array is shared by all calls and keeps whatever the last call left in it.  Every row
// slot that a call reads is written by that same call first, so nothing has to be cleared;
// but two calls whose kernels overlap on the GPU (different streams) race on it.
#include "../../include/tensotron_gemm.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include "elementwise.cuh"

namespace {

static __device__ __align__(256) float g_static_row_loss[TT_STATIC_CE_MAX_ROWS];

// The array exists once per CUDA context that has loaded the library (a `__device__` variable
// belongs to the module, and a module is loaded per context), so its address is cached per
// context, not per device ordinal: a host that runs its own driver-API context beside the
// primary one gets the address that is valid in the context it calls from.
constexpr int MAX_CONTEXTS = 64;
struct ScratchSlot {
    CUcontext ctx;
    float* addr;
};
ScratchSlot g_slots[MAX_CONTEXTS] = {};
int g_n_slots = 0;

CUcontext current_context()
{
    static PFN_cuCtxGetCurrent_v4000 get_current = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<PFN_cuCtxGetCurrent_v4000>(fn);
    }();
    CUcontext ctx = nullptr;
    if (!get_current || get_current(&ctx) != CUDA_SUCCESS) return nullptr;
    return ctx;
}

// Device address of the scratch array in the current context (set-up on first use there).
int scratch_address(float** out)
{
    CUcontext ctx = current_context();
    if (!ctx) {
        // no context yet on this thread: the runtime creates / binds the primary one
        if (cudaFree(nullptr) != cudaSuccess || !(ctx = current_context())) return TT_ERR_CUDA;
    }
    for (int i = 0; i < g_n_slots; i++)
        if (g_slots[i].ctx == ctx) { *out = g_slots[i].addr; return TT_OK; }
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_row_loss);
    if (e != cudaSuccess || !ptr) return TT_ERR_CUDA;
    if (g_n_slots < MAX_CONTEXTS) g_slots[g_n_slots++] = ScratchSlot{ctx, ptr};
    *out = ptr;
    return TT_OK;
}

}  // namespace

// The kernels are the handle-based entry's own (elementwise.cuh), launched on the built-in array,
// so both entries return identical bits.  A label outside [0, classes) makes the loss NaN (there
// is no handle whose status word could record it).
extern "C" TT_API int tt_softmax_cross_entropy_static(void* stream, const float* logits,
                                                      const int* labels, float* dlogits, float* loss,
                                                      int rows, int classes, float scale)
{
    if (rows < 0 || classes <= 0 || !logits || !labels) return TT_ERR_INVALID_ARG;
    if (rows > TT_STATIC_CE_MAX_ROWS) return TT_ERR_STATIC_LIMIT;
    if (rows == 0) return TT_OK;
    float* row_loss = nullptr;
    if (loss) {
        const int rc = scratch_address(&row_loss);
        if (rc != TT_OK) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps_per_block = 8;
    tt::ew::softmax_ce_rows_kernel<<<(rows + warps_per_block - 1) / warps_per_block, 256, 0, st>>>(
        logits, labels, dlogits, row_loss, rows, classes, scale, nullptr);
    if (loss) tt::ew::sum_fixed_kernel<<<1, 1024, 0, st>>>(row_loss, loss, rows, scale);
    return cudaGetLastError() == cudaSuccess ? TT_OK : TT_ERR_CUDA;
}
