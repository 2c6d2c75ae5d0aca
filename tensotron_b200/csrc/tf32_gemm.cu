#include "tf32_launch.h"

namespace tt {
namespace tf32 {

int init_device() { return 0; }

int try_launch(int, cudaStream_t, const float*, const float*, float*, int, int, int, int, int, int,
               int, int, int, const int*, const int*, const int*, const Epilogue&, int,
               unsigned int*)
{
    return 3;
}

}  // namespace tf32
}  // namespace tt
