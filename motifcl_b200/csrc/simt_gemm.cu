// fp32 CUDA-core contractions for the counter-linear path: the any-shape path.
//
// These kernels accept every shape the reference accepts (in_features % 4 == 0, no other
// alignment) and accumulate in fp32 with k ascending and separately rounded multiply and
// add, so each output equals the reference's per-element sum bit for bit when the reference
// is evaluated without FMA contraction -- like its register-blocked kernels do per output
// element (MotifCL kernels/matmul.cl:413-563,
// kernels/vulkan/counter_forward_f32_rb4.comp:38-131, counter_backward_input_f32_rb4.comp).
// The tensor-core kernels in tc_gemm.cu take over for shapes they support.
//
// One template: C[M,N] = sum_k A(m,k) * B(k,n), 64x64 output tile per 256-thread CTA,
// 4x4 outputs per thread, 16-deep k slices staged in shared memory.  The operand functors
// hide where an element comes from (fp32 tensor in either orientation, a column-scaled
// gradient, or the ternary digit decoded from the packed 6-bit state).
#include "counter_codec.cuh"
#include "kernels.h"

namespace mcl {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

// fp32 matrix element (r, c) of a logical [rows, cols] operand; `kfast` says which logical
// index is contiguous in memory, used only to pick a coalesced staging order.
struct OpF32 {
    const float* p;
    int rows, cols, ld;
    bool transposed;   // stored as [cols, rows]
    __device__ __forceinline__ float operator()(int r, int c) const {
        if (r >= rows || c >= cols) return 0.0f;
        return transposed ? __ldg(p + (size_t)c * ld + r) : __ldg(p + (size_t)r * ld + c);
    }
};

// grad_out[r, o] * scale[o]: the A operand of backward-to-input
// (kernels/compact_counter.cl:266 multiplies the gradient by the row scale first).
struct OpGradScaled {
    const float* g;
    const float* scale;
    int rows, cols;
    __device__ __forceinline__ float operator()(int r, int c) const {
        if (r >= rows || c >= cols) return 0.0f;
        return __fmul_rn(__ldg(g + (size_t)r * cols + c), __ldg(scale + c));
    }
};

// Ternary digit t[o, i] decoded from packed state, optionally times scale[o]
// (kernels/compact_counter.cl:7-12,25-31,53).  Logical element (k, n):
//   forward        B(k=i, n=o) = scale[o] * t[o, i]
//   backward-input B(k=o, n=i) = t[o, i]
struct OpTernary {
    const uint8_t* state;
    const float* scale;   // null: unscaled
    int in_features, out_features, lv;
    bool k_is_in;
    __device__ __forceinline__ float operator()(int k, int n) const {
        const int i = k_is_in ? k : n, o = k_is_in ? n : k;
        if (i >= in_features || o >= out_features) return 0.0f;
        const uint8_t* s = state + ((size_t)o * (in_features >> 2) + (i >> 2)) * 3;
        const uint32_t w = (uint32_t)__ldg(s) | ((uint32_t)__ldg(s + 1) << 8) | ((uint32_t)__ldg(s + 2) << 16);
        const int code = (int)((w >> (6 * (i & 3))) & 63u);
        const float t = (float)(code / lv - 1);
        return scale ? __fmul_rn(__ldg(scale + o), t) : t;
    }
};

// The same operand read from 2-bit packed weights (field = t + 1).
struct OpTernaryP2 {
    const uint32_t* packed2;
    const float* scale;   // null: unscaled
    int in_features, out_features;
    bool k_is_in;
    __device__ __forceinline__ float operator()(int k, int n) const {
        const int i = k_is_in ? k : n, o = k_is_in ? n : k;
        if (i >= in_features || o >= out_features) return 0.0f;
        const uint32_t w = __ldg(packed2 + (size_t)o * (in_features >> 4) + (i >> 4));
        const float t = (float)((int)((w >> (2 * (i & 15))) & 3u) - 1);
        return scale ? __fmul_rn(__ldg(scale + o), t) : t;
    }
};

template <class OpA, class OpB, bool A_KFAST, bool B_KFAST>
__global__ void __launch_bounds__(256) simt_gemm_kernel(OpA A, OpB B, float* __restrict__ C, int M,
                                                        int N, int K, int ldc) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int e = tid; e < TM * TK; e += 256) {
            const int mm = A_KFAST ? e / TK : e % TM;
            const int kk = A_KFAST ? e % TK : e / TM;
            As[kk][mm] = (k0 + kk < K) ? A(m0 + mm, k0 + kk) : 0.0f;
        }
#pragma unroll
        for (int e = tid; e < TN * TK; e += 256) {
            const int nn = B_KFAST ? e / TK : e % TN;
            const int kk = B_KFAST ? e % TK : e / TN;
            Bs[kk][nn] = (k0 + kk < K) ? B(k0 + kk, n0 + nn) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

template <class OpA, class OpB, bool AK, bool BK>
cudaError_t run(OpA a, OpB b, float* c, int M, int N, int K, int ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return cudaSuccess;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    simt_gemm_kernel<OpA, OpB, AK, BK><<<grid, 256, 0, stream>>>(a, b, c, M, N, K, ldc);
    return cudaGetLastError();
}

}  // namespace

// C[M,N] = op(A) op(B); transA: A stored [K,M]; transB: B stored [N,K]
// (MotifCL src/ops/matmul.cpp:1131-1233: matmul, matmul_transpose_a, matmul_transpose_b).
cudaError_t launch_simt_matmul_f32(const float* a, const float* b, float* c, int M, int K, int N,
                                   int transA, int transB, cudaStream_t stream) {
    OpF32 A{a, M, K, transA ? M : K, transA != 0};
    // logical B is [K, N]; stored [N, K] when transB
    OpF32 B{b, K, N, transB ? K : N, transB != 0};
    if (!transA && !transB) return run<OpF32, OpF32, true, false>(A, B, c, M, N, K, N, stream);
    if (!transA && transB) return run<OpF32, OpF32, true, true>(A, B, c, M, N, K, N, stream);
    if (transA && !transB) return run<OpF32, OpF32, false, false>(A, B, c, M, N, K, N, stream);
    return run<OpF32, OpF32, false, true>(A, B, c, M, N, K, N, stream);
}

cudaError_t launch_simt_counter_forward(const float* x, const uint8_t* state, const float* scale,
                                        float* y, int batch, int in_features, int out_features, int C,
                                        cudaStream_t stream) {
    OpF32 A{x, batch, in_features, in_features, false};
    OpTernary B{state, scale, in_features, out_features, 2 * C - 1, true};
    return run<OpF32, OpTernary, true, true>(A, B, y, batch, out_features, in_features, out_features, stream);
}

cudaError_t launch_simt_counter_backward_input(const uint8_t* state, const float* scale,
                                               const float* grad_out, float* grad_x, int batch,
                                               int in_features, int out_features, int C,
                                               cudaStream_t stream) {
    OpGradScaled A{grad_out, scale, batch, out_features};
    OpTernary B{state, nullptr, in_features, out_features, 2 * C - 1, false};
    return run<OpGradScaled, OpTernary, true, false>(A, B, grad_x, batch, in_features, out_features,
                                                     in_features, stream);
}

cudaError_t launch_simt_ternary_forward(const float* x, const uint32_t* packed2, const float* scale, float* y,
                                        int batch, int in_features, int out_features, cudaStream_t stream) {
    OpF32 A{x, batch, in_features, in_features, false};
    OpTernaryP2 B{packed2, scale, in_features, out_features, true};
    return run<OpF32, OpTernaryP2, true, true>(A, B, y, batch, out_features, in_features, out_features, stream);
}

cudaError_t launch_simt_ternary_backward_input(const uint32_t* packed2, const float* scale, const float* grad_out,
                                               float* grad_x, int batch, int in_features, int out_features,
                                               cudaStream_t stream) {
    OpGradScaled A{grad_out, scale, batch, out_features};
    OpTernaryP2 B{packed2, nullptr, in_features, out_features, false};
    return run<OpGradScaled, OpTernaryP2, true, false>(A, B, grad_x, batch, in_features, out_features, in_features,
                                                       stream);
}

cudaError_t launch_simt_grad_w(const float* grad_out, const float* x, float* grad_w, int batch,
                               int in_features, int out_features, int row0, int rows,
                               cudaStream_t stream) {
    // A(m = o - row0, k = r) = grad_out[r, row0 + m]: stored [batch, out] -> transposed operand
    OpF32 A{grad_out + row0, rows, batch, out_features, true};
    OpF32 B{x, batch, in_features, in_features, false};
    return run<OpF32, OpF32, false, false>(A, B, grad_w, rows, in_features, batch, in_features, stream);
}

}  // namespace mcl
