#include "tensor_map.h"

#include <cudaTypedefs.h>

namespace tt {

namespace {
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
bool g_encode_tried = false;

PFN_cuTensorMapEncodeTiled_v12000 get_encode()
{
    if (!g_encode_tried) {
        g_encode_tried = true;
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    return g_encode;
}
}  // namespace

bool tma_compatible(const OperandView& v)
{
    if (v.rank < 2 || v.rank > 5) return false;
    if ((reinterpret_cast<uintptr_t>(v.base) & 15u) != 0) return false;
    if (v.stride_elems[0] != 1) return false;
    for (int i = 0; i < v.rank; i++) {
        if (v.dim[i] == 0 || v.dim[i] > 0xFFFFFFFFull) return false;
        if (i > 0) {
            const uint64_t bytes = v.stride_elems[i] * 4ull;
            if (bytes == 0 || (bytes & 15ull) != 0 || bytes >= (1ull << 40)) return false;
        }
    }
    return true;
}

int encode_tensor_map(CUtensorMap* out, const OperandView& v, uint32_t box0, uint32_t box1,
                      Swizzle swz, uint32_t box2)
{
    PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode();
    if (!enc) return 999;
    cuuint64_t dims[5];
    cuuint64_t strides[4];
    cuuint32_t box[5];
    cuuint32_t estr[5];
    uint64_t last_bytes = 16;
    for (int i = 0; i < 5; i++) {
        dims[i] = i < v.rank ? v.dim[i] : 1;
        box[i] = i == 0 ? box0 : i == 1 ? box1 : i == 2 ? box2 : 1;
        estr[i] = 1;
        if (i > 0) {
            // Padded size-1 dims still need a legal stride: reuse the span of the last real dim.
            const uint64_t bytes = i < v.rank ? v.stride_elems[i] * 4ull : last_bytes;
            strides[i - 1] = bytes;
            last_bytes = bytes;
        }
    }
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(v.base),
                           dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swz == Swizzle::B128       ? CU_TENSOR_MAP_SWIZZLE_128B
                           : swz == Swizzle::B128_A32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                      : CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return static_cast<int>(r);
}

}  // namespace tt
