// Ternary decode GEMV for M <= 16 activation rows: y[m,o] = scale[o] * sum_k x[m,k] * t[o,k],
// with t read from the 2-bit packed weights (16 weights per uint32, field = t + 1, LSB first).
//
// There is no such kernel in the reference: at M = 1 its counter layers run the same NT GEMM
// as training (MotifCL src/nn/compact_counter.cpp:287-293).  The result is defined by that
// path, matmul_transpose_b(x, decode_weight()).
//
// HBM-bound on the packed weights: out*in/4 bytes per call.  One warp per output row streams
// the row's words with 128-bit loads; the activations (M*in fp32, at most 0.9 MB) are reused
// by every warp and stay in L1/L2.  Each thread keeps M accumulators; lanes are combined with
// warp shuffles at the end of the row.
#include "kernels.h"

namespace mcl {
namespace {

template <int MB>
__global__ void __launch_bounds__(256) ternary_gemv_kernel(const float* __restrict__ x,
                                                           const uint32_t* __restrict__ packed2,
                                                           const float* __restrict__ scale,
                                                           float* __restrict__ y, int M, int I, int O) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int wpr = I >> 4;                       // words per row
    for (int o = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); o < O; o += gridDim.x * warps_per_cta) {
        const uint32_t* wrow = packed2 + (size_t)o * wpr;
        float acc[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] = 0.0f;
        for (int w = lane; w < wpr; w += 32) {
            const uint32_t word = __ldg(wrow + w);
            float t[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) t[j] = (float)((int)((word >> (2 * j)) & 3u) - 1);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                if (m < M) {
                    const float4* xp = reinterpret_cast<const float4*>(x + (size_t)m * I + (size_t)w * 16);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 xv = __ldg(xp + q);
                        acc[m] = fmaf(xv.x, t[4 * q + 0], acc[m]);
                        acc[m] = fmaf(xv.y, t[4 * q + 1], acc[m]);
                        acc[m] = fmaf(xv.z, t[4 * q + 2], acc[m]);
                        acc[m] = fmaf(xv.w, t[4 * q + 3], acc[m]);
                    }
                }
            }
        }
        const float s = __ldg(scale + o);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            float a = acc[m];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
            if (lane == 0 && m < M) y[(size_t)m * O + o] = a * s;
        }
    }
}

}  // namespace

cudaError_t launch_ternary_gemv(const float* x, const uint32_t* packed2, const float* scale, float* y,
                                int M, int in_features, int out_features, int sm_count,
                                cudaStream_t stream) {
    const int warps = 8;
    int grid = (out_features + warps - 1) / warps;
    const int cap = sm_count * 8;
    if (grid > cap) grid = cap;
    if (M <= 1)
        ternary_gemv_kernel<1><<<grid, warps * 32, 0, stream>>>(x, packed2, scale, y, M, in_features, out_features);
    else if (M <= 4)
        ternary_gemv_kernel<4><<<grid, warps * 32, 0, stream>>>(x, packed2, scale, y, M, in_features, out_features);
    else if (M <= 8)
        ternary_gemv_kernel<8><<<grid, warps * 32, 0, stream>>>(x, packed2, scale, y, M, in_features, out_features);
    else
        ternary_gemv_kernel<16><<<grid, warps * 32, 0, stream>>>(x, packed2, scale, y, M, in_features, out_features);
    return cudaGetLastError();
}

}  // namespace mcl
