// Host-side construction of TMA descriptors (CUtensorMap) for float32 operands.
// The driver entry point is resolved at run time so the library does not link
// libcuda directly.  Descriptors are built (or fetched from a per-thread cache keyed by base,
// dims, strides, box and swizzle) per call and passed to kernels as __grid_constant__
// parameters, so they are baked into captured graph nodes.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tt {

// B128: 16-byte chunks swizzled within 128-byte rows.  B128_A32: 32-byte chunks swizzled
// within 128-byte rows (the only layout tcgen05 accepts for MN-major 32-bit operands).
enum class Swizzle { None, B128, B128_A32 };

// Describes one operand as a tensor of up to 5 dims, innermost first.
struct OperandView {
    const float* base;
    int rank;                 // number of real dims (2..5); the rest are padded with size 1
    uint64_t dim[5];          // extent in elements, innermost first
    uint64_t stride_elems[5]; // element stride of dim i (stride_elems[0] must be 1)
};

// Returns false when the view cannot be expressed as a TMA descriptor (alignment).
bool tma_compatible(const OperandView& v);

// box = extents of the copied tile for dims 0, 1 and 2 (dims 3.. use 1).
// Returns cudaSuccess-like 0 on success, non-zero CUresult otherwise.
int encode_tensor_map(CUtensorMap* out, const OperandView& v, uint32_t box0, uint32_t box1,
                      Swizzle swz, uint32_t box2 = 1);

// Hits / misses of the calling thread's descriptor cache (diagnostics, tests).
void tensor_map_cache_stats(unsigned long long* hits, unsigned long long* misses);

}  // namespace tt
