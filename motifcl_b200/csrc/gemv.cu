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


// ---- M <= 4: one launch, CUDA cores, HBM-streaming -------------------------------------------------------------
// For one to four activation rows the tensor-core route (quantize, MMA, finalize: three dependent launches and an
// MMA whose A operand is fed at 64 B/clk) costs more than the weights take to stream.  Here a CTA owns R output rows
// at a time and its threads (128 for M = 1) split K: a thread takes one 2-bit word (16 weights) of each of the R rows per step, so
// the 16 activations it needs are loaded once (L1 / L2 resident: x is at most 57 KB per row) and used for all R rows,
// and every thread has R (and, one group ahead, 2 R) independent weight loads in flight.
// A 2-bit field f = t + 1 becomes the float v = 2 + f / 2 by integer arithmetic on the word (mask, shift, OR into the bit
// pattern of 2.0f: 0x40000000 | (f << 21) is 2.0, 2.5, 3.0 and, for the field 3 of the unreachable code 63, 3.5); one
// FMA per weight follows.  sum_k x t = 2 sum_k x v - 5 sum_k x; the threads add up the x they load.  (A 256-entry
// table of float4 digits in shared memory, one 128-bit load per byte of fields, was measured 1.7 x slower: the
// data-dependent 16-byte loads collide in the banks.)
// Threads are combined in a fixed order (shuffles, then the eight warps in order), so results are deterministic.
template <int MB, int R, int MINB, int NT>
__global__ void __launch_bounds__(NT, MINB) gemv_stream_kernel(const float* __restrict__ x, const uint32_t* __restrict__ packed2,
                                                                const float* __restrict__ scale, float* __restrict__ y, int M, int I,
                                                                int O) {
    constexpr int NV = R * MB + MB;             // values a thread contributes: R x MB dot products and MB sums of x
    constexpr int NW = NT / 32;
    __shared__ float red[NW][NV];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpr = I >> 4;
    const int groups = (O + R - 1) / R;
    // words of the first step of a group: loaded one group ahead, so that a thread has two groups' loads in flight
    uint32_t pre[R];
    {
        const int o0 = blockIdx.x * R;
#pragma unroll
        for (int r = 0; r < R; ++r)
            pre[r] = (blockIdx.x < groups && (int)threadIdx.x < wpr) ? __ldg(packed2 + (size_t)min(o0 + r, O - 1) * wpr + threadIdx.x) : 0u;
    }
    for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
        const int o0 = grp * R;
        float acc[R][MB], xs[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            xs[m] = 0.0f;
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r][m] = 0.0f;
        }
        for (int w = threadIdx.x; w < wpr; w += NT) {
            uint32_t word[R];
            if (w == (int)threadIdx.x) {
                const int on = (grp + (int)gridDim.x) * R;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    word[r] = pre[r];
                    if (grp + (int)gridDim.x < groups) pre[r] = __ldg(packed2 + (size_t)min(on + r, O - 1) * wpr + w);
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) word[r] = __ldg(packed2 + (size_t)min(o0 + r, O - 1) * wpr + w);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {            // four activations (one float4 per row of x) at a time
                float4 xv[MB];
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    xv[m] = m < M ? __ldg(reinterpret_cast<const float4*>(x + (size_t)m * I + (size_t)w * 16) + q)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                    xs[m] += (xv[m].x + xv[m].y) + (xv[m].z + xv[m].w);
                }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t b = word[r] >> (8 * q);       // the four fields of this step in the low byte
                    const float v0 = __uint_as_float(((b & 0x03u) << 21) | 0x40000000u);
                    const float v1 = __uint_as_float(((b & 0x0Cu) << 19) | 0x40000000u);
                    const float v2 = __uint_as_float(((b & 0x30u) << 17) | 0x40000000u);
                    const float v3 = __uint_as_float(((b & 0xC0u) << 15) | 0x40000000u);
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        acc[r][m] = fmaf(xv[m].x, v0, acc[r][m]);
                        acc[r][m] = fmaf(xv[m].y, v1, acc[r][m]);
                        acc[r][m] = fmaf(xv[m].z, v2, acc[r][m]);
                        acc[r][m] = fmaf(xv[m].w, v3, acc[r][m]);
                    }
                }
            }
        }
        // lanes, then warps
        float vals[NV];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MB; ++m) vals[r * MB + m] = acc[r][m];
#pragma unroll
        for (int m = 0; m < MB; ++m) vals[R * MB + m] = xs[m];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float a = vals[i];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
            if (lane == 0) red[warp][i] = a;
        }
        __syncthreads();
        if (threadIdx.x < R * MB) {
            const int r = threadIdx.x / MB, m = threadIdx.x - r * MB, o = o0 + r;
            float a = 0.0f, sx = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; ++w) { a += red[w][threadIdx.x]; sx += red[w][R * MB + m]; }
            if (m < M && o < O) y[(size_t)m * O + o] = __ldg(scale + o) * (2.0f * a - 5.0f * sx);
        }
        __syncthreads();
    }
}

}  // namespace

cudaError_t launch_ternary_gemv_stream(const float* x, const uint32_t* packed2, const float* scale, float* y, int M,
                                       int in_features, int out_features, int sm_count, cudaStream_t stream) {
    const int cap = sm_count * 16;
    auto grid_for = [&](int rows_per_cta) {
        const int g = (out_features + rows_per_cta - 1) / rows_per_cta;
        return g < cap ? g : cap;
    };
    if (M <= 1)     // 128 threads per CTA measured best (1.84 ms per sweep; 256: 2.00, 64: 2.26)
        gemv_stream_kernel<1, 8, 6, 128><<<grid_for(8), 128, 0, stream>>>(x, packed2, scale, y, M, in_features, out_features);
    else
        gemv_stream_kernel<2, 4, 4, 256><<<grid_for(4), 256, 0, stream>>>(x, packed2, scale, y, M, in_features, out_features);
    return cudaGetLastError();
}

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
