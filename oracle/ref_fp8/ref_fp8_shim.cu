// Host-side shim around the reference's software FP8 conversion (test infrastructure).
//
// It contains no conversion code of its own: it includes the reference's header where it
// lies (pass -I<reference>/src/common) and exposes the two FP8 types the reference's fused
// kernel uses (src/common/float8.h:215-279) through a C ABI so the Python oracle can be
// compared against them bit for bit.  The built library goes to oracle/_ref/ only.
#include <cstdint>
#include "device_common.h"   // pulls in float8.h exactly as the reference's kernels see it

extern "C" {

void ref_float_to_e4m3fn(const float *in, uint8_t *out, long n) {
    for (long i = 0; i < n; ++i) out[i] = fp8e4m3fn(in[i]).data;
}

void ref_float_to_e4m3fnuz(const float *in, uint8_t *out, long n) {
    for (long i = 0; i < n; ++i) out[i] = fp8e4m3fnuz(in[i]).data;
}

void ref_e4m3fn_to_float(const uint8_t *in, float *out, long n) {
    for (long i = 0; i < n; ++i) out[i] = static_cast<float>(fp8e4m3fn(in[i], fp8e4m3fn::from_bits()));
}

void ref_e4m3fnuz_to_float(const uint8_t *in, float *out, long n) {
    for (long i = 0; i < n; ++i) out[i] = static_cast<float>(fp8e4m3fnuz(in[i], fp8e4m3fnuz::from_bits()));
}

int ref_e4m3fn_max(void) { return fp8e4m3fn::max_value; }
int ref_e4m3fnuz_max(void) { return fp8e4m3fnuz::max_value; }

}  // extern "C"
