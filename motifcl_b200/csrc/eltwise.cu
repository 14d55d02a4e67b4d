// Elementwise fp32 helpers around the counter path: the handful of ops MotifCL's counter tests
// and autograd engine call between counter layers (gradient accumulation, residual adds, loss
// differences): MotifCL src/ops/basic_ops.cpp:67-92,208-211,409,462 and kernels/basic.cl.
// One HBM-bound grid-stride kernel; exact fp32 (single rounding per element, like the reference).
#include "kernels.h"

namespace mcl {
namespace {

template <int OP>
__global__ void __launch_bounds__(256) eltwise_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                      float* __restrict__ out, size_t n, float alpha) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float r;
        if (OP == 0) r = __fadd_rn(a[i], b[i]);
        else if (OP == 1) r = __fsub_rn(a[i], b[i]);
        else if (OP == 2) r = __fmul_rn(a[i], b[i]);
        else if (OP == 3) r = __fmul_rn(a[i], alpha);
        else if (OP == 4) r = __fadd_rn(a[i], alpha);
        else if (OP == 6) r = a[i] - alpha * b[i];      // sgd step (kernels/vulkan/sgd_update_f32.comp)
        else r = 0.0f;
        out[i] = r;
    }
}

}  // namespace

cudaError_t launch_eltwise_f32(int op, const float* a, const float* b, float* out, size_t n, float alpha,
                               int sm_count, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)sm_count * 16) blocks = (size_t)sm_count * 16;
    switch (op) {
        case 0: eltwise_kernel<0><<<(int)blocks, 256, 0, stream>>>(a, b, out, n, alpha); break;
        case 1: eltwise_kernel<1><<<(int)blocks, 256, 0, stream>>>(a, b, out, n, alpha); break;
        case 2: eltwise_kernel<2><<<(int)blocks, 256, 0, stream>>>(a, b, out, n, alpha); break;
        case 3: eltwise_kernel<3><<<(int)blocks, 256, 0, stream>>>(a, b, out, n, alpha); break;
        case 4: eltwise_kernel<4><<<(int)blocks, 256, 0, stream>>>(a, b, out, n, alpha); break;
        case 5: eltwise_kernel<5><<<(int)blocks, 256, 0, stream>>>(a, b, out, n, alpha); break;
        case 6: eltwise_kernel<6><<<(int)blocks, 256, 0, stream>>>(a, b, out, n, alpha); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace mcl
