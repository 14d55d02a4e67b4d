// C wrapper around the reference's own host GEMV core, native::matmul_f32_m1
// (src/runtime/native_matmul.cpp:110-133), which oracle/Makefile compiles from the
// reference tree by path.  TEST INFRASTRUCTURE ONLY (validates orc_matmul_f32_m1 and
// serves as the single-threaded CPU baseline of the decode GEMV).
#include <motifcl/runtime/native_matmul.hpp>

extern "C" {
void ref_matmul_f32_m1(const float* a, const float* b, float* out, long long k, long long n) {
    motifcl::native::matmul_f32_m1(a, b, out, k, n);
}
const char* ref_matmul_f32_m1_kernel_name() { return motifcl::native::matmul_f32_m1_kernel_name(); }
}
