// Kernel instantiations for element type float.
#include "launch_impl.cuh"

namespace gpuk {
GPUK_INSTANTIATE_LAUNCHERS(float)
}  // namespace gpuk
