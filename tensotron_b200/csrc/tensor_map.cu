#include "tensor_map.h"

#include <cudaTypedefs.h>
#include <string.h>

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

namespace {
// Descriptor cache.  A training loop calls the same products on the same buffers step after
// step, and one cuTensorMapEncodeTiled costs about a microsecond of host time (2 to 5 per
// call), the same order as a kernel launch.  A descriptor is a pure function of (base, dims,
// strides, box, swizzle) -- it does not depend on the context or on what the memory holds -- so
// the encoded 128 bytes are kept in a small direct-mapped table per host thread, keyed by
// exactly those inputs.
struct MapKey {
    const void* base;
    uint64_t dim[5];
    uint64_t stride[5];
    uint32_t box[3];
    int32_t rank;
    int32_t swz;
    bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
    bool used = false;
    MapKey key;
    CUtensorMap map;
};
constexpr int CACHE_SLOTS = 256;
thread_local MapSlot t_cache[CACHE_SLOTS];
thread_local unsigned long long t_hits = 0, t_misses = 0;

uint64_t hash_key(const MapKey& k)
{
    uint64_t h = 1469598103934665603ull;   // FNV-1a over the key's words
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    for (size_t i = 0; i < sizeof(MapKey) / sizeof(uint64_t); i++) { h ^= w[i]; h *= 1099511628211ull; }
    return h ^ (h >> 29);
}
static_assert(sizeof(MapKey) % sizeof(uint64_t) == 0, "key is hashed word by word");
}  // namespace

void tensor_map_cache_stats(unsigned long long* hits, unsigned long long* misses)
{
    if (hits) *hits = t_hits;
    if (misses) *misses = t_misses;
}

int encode_tensor_map(CUtensorMap* out, const OperandView& v, uint32_t box0, uint32_t box1,
                      Swizzle swz, uint32_t box2)
{
    MapKey key;
    memset(&key, 0, sizeof(key));   // padding bytes too: the key is compared and hashed as raw bytes
    key.base = v.base;
    key.rank = v.rank;
    key.swz = static_cast<int32_t>(swz);
    for (int i = 0; i < v.rank && i < 5; i++) { key.dim[i] = v.dim[i]; key.stride[i] = v.stride_elems[i]; }
    key.box[0] = box0; key.box[1] = box1; key.box[2] = box2;
    MapSlot& slot = t_cache[hash_key(key) % CACHE_SLOTS];
    if (slot.used && slot.key == key) {
        *out = slot.map;
        t_hits++;
        return 0;
    }
    t_misses++;
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
    if (r == CUDA_SUCCESS) {
        slot.used = true;
        slot.key = key;
        slot.map = *out;
    }
    return static_cast<int>(r);
}

}  // namespace tt
