// Kernel instantiations for element type __half.
#include "launch_impl.cuh"

namespace gpuk {
GPUK_INSTANTIATE_LAUNCHERS(__half)
}  // namespace gpuk
