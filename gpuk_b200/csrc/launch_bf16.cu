// Kernel instantiations for element type __nv_bfloat16.
#include "launch_impl.cuh"

namespace gpuk {
GPUK_INSTANTIATE_LAUNCHERS(__nv_bfloat16)
}  // namespace gpuk
