// Shared host/device parameter blocks for the GEMM kernels.
#pragma once
#include <stdint.h>

namespace tt {

constexpr int MAX_BATCH_RANK = 8;

constexpr int MAX_PEERS = 8;

// Epilogue fused into the store path: C = act(acc + bias[n]).
struct Epilogue {
    const float* bias;  // per output column, may be null
    int act;            // TT_ACT_*
    // Row-block scatter (gradient exchange between GPUs): with scatter_rows > 0, output row r
    // is stored at scatter[r / scatter_rows] + r * N + n instead of c + r * N + n; the bases may
    // be peer-GPU addresses.  scatter_rows is a multiple of every kernel's tile height, so a
    // tile never straddles two bases.  Honoured by the stream-K form of the FMA kernel and by
    // the tensor-core kernel; the host routes scatter calls to those only.
    int scatter_rows;
    float* scatter[MAX_PEERS];
};

__device__ __forceinline__ float* scatter_base(const Epilogue& e, float* c, int row)
{
    return e.scatter_rows > 0 ? e.scatter[row / e.scatter_rows] : c;
}

// Batch structure after the host collapsed mergeable axes.  The linear batch index
// is decoded last-axis-fastest over dims[0..rank).
struct BatchDesc {
    int rank;
    int dims[MAX_BATCH_RANK];
    // any-stride kernels: element offsets per axis
    int a_stride[MAX_BATCH_RANK];
    int b_stride[MAX_BATCH_RANK];
    // TMA kernels: axis -> (coordinate slot 0..2 or -1 for broadcast, multiplier)
    signed char a_slot[MAX_BATCH_RANK];
    signed char b_slot[MAX_BATCH_RANK];
    int a_mult[MAX_BATCH_RANK];
    int b_mult[MAX_BATCH_RANK];
    // One extra batch axis that is summed into the output (fused reduction of a broadcast
    // operand's gradient): red_count entries, visited in ascending order inside the k loop.
    int red_count;                 // 1 = no reduced axis
    int red_a_stride, red_b_stride;  // any-stride kernels: element strides of that axis
    signed char red_a_slot, red_b_slot;  // TMA kernels: coordinate slot or -1
};

struct GemmShape {
    int M, N, K;
    int tiles_m, tiles_n;
    int batch;          // number of matrices
    long long work;     // batch * tiles_m * tiles_n
};

// Grouped raster: consecutive work items walk GROUP tile-rows down before moving one
// tile-column right, so the CTAs in flight at one time share A and B panels in L2.
__host__ __device__ inline void raster_tile(int t, int tiles_m, int tiles_n, int group, int& tm,
                                            int& tn)
{
    const int per_group = group * tiles_n;
    const int g = t / per_group;
    const int first_m = g * group;
    const int gsize = (tiles_m - first_m) < group ? (tiles_m - first_m) : group;
    const int r = t - g * per_group;
    tm = first_m + r % gsize;
    tn = r / gsize;
}

}  // namespace tt
