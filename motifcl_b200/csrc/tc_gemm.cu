// Tensor-core contractions of the counter-linear path for sm_100a: tcgen05.mma with fp32
// accumulators in tensor memory (TMEM), operands staged in shared memory by TMA.
//
// One kernel serves the three products of a training step (MotifCL
// src/nn/compact_counter.cpp:233-300 and kernels/matmul.cl:413-563 compute them with fp32
// scalar FMAs):
//     Y  [tokens,out] = X  . T^T          A = planes of X  [tokens,in],   B = T   [out,in]
//     dX [tokens,in ] = (dY.s) . T        A = planes of dY.s [tokens,out], B = T^T [in,out]
//     dW [out,in]     = dY^T . X          A = planes of dY^T [out,tokens], B = planes of X^T [in,tokens]
// Every operand is K-major bf16 ("NT" form), produced by the pre-pass kernels below:
//   * an fp32 tensor is split into bf16 terms a = a1 + a2 (+ a3), a1 = bf16(a),
//     a2 = bf16(a - a1), a3 = bf16(a - a1 - a2); products of terms are accumulated in fp32
//     in TMEM, so fp32 activations keep (nearly) fp32 accuracy on bf16 tensor cores;
//   * ternary weights {-1,0,1,(2)} are exact in bf16 and are expanded from the packed 6-bit
//     state, in both orientations.
// The kernel computes  C[M,N] = sum over a list of (plane of A, plane of B) pairs of
// A_p[M,K] . B_q[N,K]^T, optionally scaled per column, or writes split-K partial sums that a
// fixed-order reduction kernel adds up (deterministic).
//
// Structure of the persistent CTA (192 threads; work items = 128 x BN output tile x split-K slice, dealt
// round-robin; BN a multiple of 32 up to 256):
//   warp 0 lane 0   TMA producer: cp.async.bulk.tensor (3-D tile {64 k, rows, plane}, 128-byte
//                   swizzle) into a ring of `stages` shared-memory slots, mbarrier complete_tx
//   warp 1 lane 0   MMA issuer: four tcgen05.mma (K = 16 each) per slot, tcgen05.commit to
//                   release the slot, final commit to signal the accumulator; warp 1 owns TMEM
//   warps 2..5      epilogue: tcgen05.ld 32 lanes x 32 columns, scale, 128-bit stores
// Two accumulators in TMEM let the epilogue of one item overlap the main loop of the next.
// Every mbarrier wait is bounded: on time-out the kernel records an error word, skips the
// rest of its work, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include "counter_codec.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace mcl {
namespace {

constexpr int BM = 128;          // UMMA M
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int kMaxStages = 8;
constexpr int kATileBytes = BM * BK * 2;   // 16 KiB

struct TcParams {
    float* C;                 // output [M, ldc] (or split-K partials [splits][M][ldc])
    const float* col_scale;   // optional, applied when splits == 1
    int M, N, K, ldc;
    int BN, stages;
    int nterms;
    int pa[6], pb[6];
    int ktiles_per_split, splits;
    int* err;
};

// Instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = bf16 (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Persistent CTA of 192 threads; work items (output tile x split-K slice) are dealt round-robin.
//   warp 0        TMA producer (one elected lane)
//   warp 1        MMA issuer (one elected lane); also allocates / frees TMEM
//   warps 2..5    epilogue: TMEM lanes 32*(warp%4) .. +31
// Two accumulators live in TMEM (columns [0,BN) and [ACC,ACC+BN)), so the epilogue of one item
// overlaps the main loop of the next.
constexpr int kTcThreads = 192;

__global__ void __launch_bounds__(kTcThreads) tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                                                             const __grid_constant__ CUtensorMap tmB,
                                                             const TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kMaxStages + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BN = p.BN, S = p.stages;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t stage_bytes = kATileBytes + (uint32_t)BN * BK * 2;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
    auto acc_full = [&](int a) { return bar0 + 8u * (2 * kMaxStages + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (2 * kMaxStages + 2 + a); };
    uint32_t acc_cols = 32;                       // columns of one accumulator (power of two >= BN)
    while ((int)acc_cols < BN) acc_cols <<= 1;
    const uint32_t tmem_cols = 2 * acc_cols;      // <= 512

    const int tiles_n = (p.N + BN - 1) / BN, tiles_m = (p.M + BM - 1) / BM;
    const int ktiles = (p.K + BK - 1) / BK;
    const int n_items = tiles_m * tiles_n * p.splits;
    // item -> (m tile fastest, then n tile, then split): CTAs running together share a B tile

    if (threadIdx.x == 0) {
        abort_flag = (*reinterpret_cast<volatile int*>(p.err) != 0);   // an earlier CTA gave up: do not wait at all
        for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer --------------------------------------------------------------
            uint32_t it = 0;       // slot counter across all items of this CTA
            for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x) {
                const int mt = item % tiles_m, rest = item / tiles_m;
                const int nt = rest % tiles_n, split = rest / tiles_n;
                const int kt0 = split * p.ktiles_per_split;
                const int my_kt = min(p.ktiles_per_split, ktiles - kt0);
                for (int term = 0; term < p.nterms; ++term) {
                    const int pa = p.pa[term], pb = p.pb[term];
                    for (int kk = 0; kk < my_kt; ++kk, ++it) {
                        const int s = (int)(it % (uint32_t)S);
                        const uint32_t ph = (it / (uint32_t)S) & 1u;
                        if (!mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 1); break; }
                        const uint32_t a_dst = tiles + (uint32_t)s * stage_bytes;
                        mbar_expect_tx(full_bar(s), stage_bytes);
                        tma_load_3d(a_dst, &tmA, full_bar(s), (kt0 + kk) * BK, mt * BM, pa);
                        tma_load_3d(a_dst + kATileBytes, &tmB, full_bar(s), (kt0 + kk) * BK, nt * BN, pb);
                    }
                    if (abort_flag) break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----------------------------------------------------------------
            const uint32_t idesc = idesc_bf16(BM, BN);
            uint32_t it = 0, n_local = 0;
            for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x, ++n_local) {
                const int split = item / (tiles_m * tiles_n);
                const int kt0 = split * p.ktiles_per_split;
                const int my_kt = min(p.ktiles_per_split, ktiles - kt0);
                const int total = p.nterms * my_kt;
                const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
                if (!mbar_wait(acc_empty(acc), aph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 4); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_cols;
                for (int j = 0; j < total; ++j, ++it) {
                    const int s = (int)(it % (uint32_t)S);
                    const uint32_t ph = (it / (uint32_t)S) & 1u;
                    if (!mbar_wait(full_bar(s), ph, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 2); break; }
                    tc_fence_after();
                    const uint32_t a_addr = tiles + (uint32_t)s * stage_bytes;
                    const uint64_t da = smem_desc_k_sw128(a_addr), db = smem_desc_k_sw128(a_addr + kATileBytes);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)   // 16 bf16 = 32 bytes = +2 in the address field
                        umma_bf16(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (j | kk) != 0 ? 1u : 0u);
                    umma_commit(empty_bar(s));
                }
                if (abort_flag) break;
                umma_commit(acc_full(acc));
            }
        }
    } else {
        // ---- epilogue warps: TMEM -> registers -> global ---------------------------------------
        const int q = warp & 3;                        // TMEM lane quarter this warp may read
        const bool scale = (p.col_scale != nullptr) && p.splits == 1;
        uint32_t n_local = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n_local) {
            const int mt = item % tiles_m, rest = item / tiles_m;
            const int nt = rest % tiles_n, split = rest / tiles_n;
            const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
            bool ok = !abort_flag;
            if (ok && !mbar_wait(acc_full(acc), aph, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 3); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int n0 = nt * BN;
            const int row = mt * BM + q * 32 + lane;
            float* crow = p.C + ((size_t)split * p.M + row) * p.ldc;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= p.N) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + acc * acc_cols + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                tmem_ld_wait();
                if (row < p.M) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int col = n0 + c0 + j;
                        if (col >= p.N) break;
                        float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                               __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        if (scale) {
                            const float4 sc = __ldg(reinterpret_cast<const float4*>(p.col_scale + col));
                            o.x *= sc.x; o.y *= sc.y; o.z *= sc.z; o.w *= sc.w;
                        }
                        *reinterpret_cast<float4*>(crow + col) = o;    // N % 4 == 0, ldc % 4 == 0
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty(acc));               // 128 arrivals free the accumulator
        }
    }
    __syncwarp();
    if (abort_flag) {
        // gave up: let copies that are still in flight land before the shared memory is released
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 2000000ull) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// C[m,n] = scale[n] * sum_z partial[z][m][n], z ascending (deterministic split-K reduction).
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ C,
                                     const float* __restrict__ col_scale, int M, int N, int ldc, int splits) {
    const size_t n4 = (size_t)M * (N / 4);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / (N / 4)), c = (int)(i % (N / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < splits; ++z) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(partial + ((size_t)z * M + m) * N + c));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (col_scale) {
            const float4 s = __ldg(reinterpret_cast<const float4*>(col_scale + c));
            acc.x *= s.x; acc.y *= s.y; acc.z *= s.z; acc.w *= s.w;
        }
        *reinterpret_cast<float4*>(C + (size_t)m * ldc + c) = acc;
    }
}

// ---- pre-pass: fp32 -> bf16 term planes (optionally column-scaled, optionally transposed) ----
// src [R, Cc] fp32.  Writes, for t < nterms:
//   planes   [t][R ][ld_n]  = term t of (src * col_scale), t < nterms    (when planes   != null)
//   planes_t [t][Cc][ld_t]  = term t of  src (unscaled), transposed, t < nterms_t (when planes_t != null)
// 64 x 64 tiles through shared memory so that both outputs are written with coalesced rows.
__device__ __forceinline__ void split3(float v, __nv_bfloat16 (&h)[3]) {
    h[0] = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h[0]);
    h[1] = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(h[1]);
    h[2] = __float2bfloat16_rn(r2);
}

__global__ void __launch_bounds__(256) split_planes_kernel(const float* __restrict__ src, int R, int Cc,
                                                           const float* __restrict__ col_scale,
                                                           __nv_bfloat16* __restrict__ planes, int ld_n,
                                                           __nv_bfloat16* __restrict__ planes_t, int ld_t,
                                                           int nterms, int nterms_t) {
    __shared__ float tile[64][65];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;    // 64 x 4
    for (int rr = ty; rr < 64; rr += 4) {
        const int r = r0 + rr, c = c0 + tx;
        float v = 0.0f;
        if (r < R && c < Cc) v = __ldg(src + (size_t)r * Cc + c);
        tile[rr][tx] = v;
        if (planes != nullptr && r < R && c < Cc) {
            const float sv = col_scale ? __fmul_rn(v, __ldg(col_scale + c)) : v;
            __nv_bfloat16 h[3];
            split3(sv, h);
            for (int t = 0; t < nterms; ++t) planes[((size_t)t * R + r) * ld_n + c] = h[t];
        }
    }
    if (planes_t == nullptr) return;
    __syncthreads();
    for (int cc = ty; cc < 64; cc += 4) {
        const int c = c0 + cc, r = r0 + tx;
        if (c < Cc && r < R) {
            __nv_bfloat16 h[3];
            split3(tile[tx][cc], h);
            for (int t = 0; t < nterms_t; ++t) planes_t[((size_t)t * Cc + c) * ld_t + r] = h[t];
        }
    }
}

// Vectorised form of the same pre-pass for Cc % 4 == 0, R % 4 == 0 and 16-byte aligned src:
// 128-bit loads, 64-bit stores of four bf16 in both orientations.
__device__ __forceinline__ uint2 pack4(const __nv_bfloat16 a, const __nv_bfloat16 b, const __nv_bfloat16 c,
                                       const __nv_bfloat16 d) {
    uint2 o;
    o.x = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
    o.y = (uint32_t)__bfloat16_as_ushort(c) | ((uint32_t)__bfloat16_as_ushort(d) << 16);
    return o;
}

__global__ void __launch_bounds__(256) split_planes_vec_kernel(const float* __restrict__ src, int R, int Cc,
                                                               const float* __restrict__ col_scale,
                                                               __nv_bfloat16* __restrict__ planes, int ld_n,
                                                               __nv_bfloat16* __restrict__ planes_t, int ld_t,
                                                               int nterms, int nterms_t) {
    __shared__ float tile[64][65];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;    // 16 column quads x 16 rows
    const int c = c0 + tx * 4;
    float4 sc4 = make_float4(1.f, 1.f, 1.f, 1.f);
    if (col_scale != nullptr && c < Cc) sc4 = __ldg(reinterpret_cast<const float4*>(col_scale + c));
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int rr = pass * 16 + ty, r = r0 + rr;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < R && c < Cc) v = __ldg(reinterpret_cast<const float4*>(src + (size_t)r * Cc + c));
        tile[rr][tx * 4 + 0] = v.x; tile[rr][tx * 4 + 1] = v.y; tile[rr][tx * 4 + 2] = v.z; tile[rr][tx * 4 + 3] = v.w;
        if (planes != nullptr && r < R && c < Cc) {
            if (col_scale != nullptr) {
                v.x = __fmul_rn(v.x, sc4.x); v.y = __fmul_rn(v.y, sc4.y);
                v.z = __fmul_rn(v.z, sc4.z); v.w = __fmul_rn(v.w, sc4.w);
            }
            __nv_bfloat16 h0[3], h1[3], h2[3], h3[3];
            split3(v.x, h0); split3(v.y, h1); split3(v.z, h2); split3(v.w, h3);
#pragma unroll
            for (int t = 0; t < 3; ++t)
                if (t < nterms)
                    *reinterpret_cast<uint2*>(planes + ((size_t)t * R + r) * ld_n + c) = pack4(h0[t], h1[t], h2[t], h3[t]);
        }
    }
    if (planes_t == nullptr) return;
    __syncthreads();
    // transposed: thread owns 4 consecutive source rows (= 4 consecutive output columns) of one source column
    const int rq = threadIdx.x & 15, cl = threadIdx.x >> 4;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int cc = pass * 16 + cl, cg = c0 + cc, r = r0 + rq * 4;
        if (cg < Cc && r < R) {
            __nv_bfloat16 h0[3], h1[3], h2[3], h3[3];
            split3(tile[rq * 4 + 0][cc], h0); split3(tile[rq * 4 + 1][cc], h1);
            split3(tile[rq * 4 + 2][cc], h2); split3(tile[rq * 4 + 3][cc], h3);
#pragma unroll
            for (int t = 0; t < 3; ++t)
                if (t < nterms_t)
                    *reinterpret_cast<uint2*>(planes_t + ((size_t)t * Cc + cg) * ld_t + r) = pack4(h0[t], h1[t], h2[t], h3[t]);
        }
    }
}

// ---- pre-pass: packed 6-bit state -> bf16 ternary digits, both orientations ------------------
//   T  [O][ld_i] (when T  != null),  Tt [I][ld_o] (when Tt != null)
__global__ void __launch_bounds__(256) expand_ternary_kernel(const uint8_t* __restrict__ state, int C,
                                                             int O, int I, __nv_bfloat16* __restrict__ T,
                                                             int ld_i, __nv_bfloat16* __restrict__ Tt, int ld_o) {
    __shared__ DecodeLut lut;
    __shared__ __nv_bfloat16 tile[64][66];
    build_decode_lut(&lut, C, threadIdx.x, blockDim.x);
    __syncthreads();
    const int o0 = blockIdx.y * 64, i0 = blockIdx.x * 64;
    const int gpr = I >> 2;
    // 64 rows x 16 groups per tile; thread handles one group (4 weights) at a time
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
        const int oo = e >> 4, g = (i0 >> 2) + (e & 15);
        const int o = o0 + oo;
        if (o < O && g < gpr) {
            const uint8_t* s = state + ((size_t)o * gpr + g) * 3;
            const uint32_t w = (uint32_t)__ldg(s) | ((uint32_t)__ldg(s + 1) << 8) | ((uint32_t)__ldg(s + 2) << 16);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __nv_bfloat16 t = __float2bfloat16_rn(lut.e[(w >> (6 * k)) & 63u].x);
                tile[oo][(e & 15) * 4 + k] = t;
                if (T != nullptr) T[(size_t)o * ld_i + g * 4 + k] = t;
            }
        }
    }
    if (Tt == nullptr) return;
    __syncthreads();
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    for (int ii = ty; ii < 64; ii += 4) {
        const int i = i0 + ii, o = o0 + tx;
        if (i < I && o < O) Tt[(size_t)i * ld_o + o] = tile[tx][ii];
    }
}

// Same expansion from the 2-bit packed weights (field = t + 1, 16 per word): what ranks that do
// not own a layer's counter state use after the all-gather of packed weights.
__global__ void __launch_bounds__(256) expand_ternary_p2_kernel(const uint32_t* __restrict__ packed2, int O, int I,
                                                                __nv_bfloat16* __restrict__ T, int ld_i,
                                                                __nv_bfloat16* __restrict__ Tt, int ld_o) {
    __shared__ __nv_bfloat16 tile[64][66];
    const int o0 = blockIdx.y * 64, i0 = blockIdx.x * 64;
    const int wpr = I >> 4;
    // 64 rows x 4 words per tile; thread handles one word (16 weights)
    {
        const int oo = threadIdx.x >> 2, wq = threadIdx.x & 3;
        const int o = o0 + oo, wi = (i0 >> 4) + wq;
        if (o < O && wi < wpr) {
            const uint32_t word = __ldg(packed2 + (size_t)o * wpr + wi);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const __nv_bfloat16 t = __float2bfloat16_rn((float)((int)((word >> (2 * k)) & 3u) - 1));
                tile[oo][wq * 16 + k] = t;
                if (T != nullptr) T[(size_t)o * ld_i + wi * 16 + k] = t;
            }
        }
    }
    if (Tt == nullptr) return;
    __syncthreads();
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    for (int ii = ty; ii < 64; ii += 4) {
        const int i = i0 + ii, o = o0 + tx;
        if (i < I && o < O) Tt[(size_t)i * ld_o + o] = tile[tx][ii];
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 3-D map over bf16 planes [P][rows][ld]: dims {K, rows, P}, box {64, box_rows, 1}, 128-byte swizzle.
// Reads beyond K or rows return zeros, so ragged edges need no padding in memory.
bool make_map(CUtensorMap* map, const void* base, int K, int rows, int planes, int ld, size_t plane_stride,
              int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)plane_stride * 2};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int tc_pick_bn(int N) {
    // widest tile that wastes least: N = 288 -> 96 x 3, 768 -> 256 x 3, 1024.. -> 256
    int best = 256, best_waste = 1 << 30;
    for (int bn = 256; bn >= 64; bn -= 32) {
        const int tiles = (N + bn - 1) / bn;
        const int waste = tiles * bn - N;
        if (waste < best_waste) { best_waste = waste; best = bn; }
    }
    return best;
}


size_t tc_splitk_workspace_bytes(int M, int N, int K, int sm_count, int depth_limit, int* splits_out) {
    const int bn = tc_pick_bn(N);
    const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const int ktiles = (K + BK - 1) / BK;
    int splits = 1;
    if (tiles < sm_count && ktiles >= 8) {
        splits = (2 * sm_count + tiles - 1) / tiles;
        if (splits > ktiles / 4) splits = ktiles / 4;
        if (splits > 32) splits = 32;
        if (splits < 1) splits = 1;
    }
    // Accuracy: tensor-core accumulation into TMEM truncates, and the error of a product of two
    // fp32-split operands was measured to grow linearly with the accumulation depth (3e-7 relative
    // at K = 1024, 6e-6 at K = 16384).  `depth_limit` (k-tiles of 64) bounds what one accumulator
    // absorbs; deeper contractions are cut into slices that the reduction kernel adds in fp32 with
    // round-to-nearest.
    const int lim = depth_limit;
    if (lim > 0 && (ktiles + splits - 1) / splits > lim) splits = (ktiles + lim - 1) / lim;
    *splits_out = splits;
    return splits > 1 ? (size_t)splits * M * N * sizeof(float) : 0;
}

cudaError_t launch_tc_gemm(const void* a_planes, int a_nplanes, int lda, size_t a_plane_stride,
                           const void* b_planes, int b_nplanes, int ldb, size_t b_plane_stride, float* c,
                           int ldc, int M, int N, int K, const int* pa, const int* pb,
                           int nterms, const float* col_scale, float* splitk_ws, int splits, int* err_word,
                           size_t max_smem, int sm_count, cudaStream_t stream, int* launches) {
    if (nterms < 1 || nterms > 6 || (N & 3) || (ldc & 3) || (lda & 7) || (ldb & 7)) return cudaErrorInvalidValue;
    const int bn = tc_pick_bn(N);
    CUtensorMap ma, mb;
    if (!make_map(&ma, a_planes, K, M, a_nplanes, lda, a_plane_stride, BM)) return cudaErrorInvalidValue;
    if (!make_map(&mb, b_planes, K, N, b_nplanes, ldb, b_plane_stride, bn)) return cudaErrorInvalidValue;
    TcParams p;
    p.col_scale = col_scale;
    p.M = M; p.N = N; p.K = K;
    p.BN = bn;
    const size_t stage_bytes = (size_t)kATileBytes + (size_t)bn * BK * 2;
    const int ktiles = (K + BK - 1) / BK;
    int stages = (int)((max_smem - 2048) / stage_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    const int want = nterms * ((ktiles + splits - 1) / splits);   // slots one work item fills
    // Two accumulators of one CTA take 2 * pow2(BN) TMEM columns of the SM's 512.  Narrow tiles
    // (BN <= 128) with short main loops leave room for a second resident CTA, which doubles the
    // loads in flight where the loop is latency-bound; then each CTA gets half the shared memory.
    bool two_ctas = false;
    if (bn <= 128 && want <= 32) {
        const int half = (int)((((max_smem - 4096) / 2) - 1024) / stage_bytes);
        if (half >= 3) { two_ctas = true; if (half < stages) stages = half; }
    }
    if (stages > want) stages = want;
    if (stages < 2) stages = 2;
    if ((size_t)stages * stage_bytes + 1024 > max_smem) return cudaErrorInvalidConfiguration;
    if (stages < 2) return cudaErrorInvalidConfiguration;
    p.stages = stages;
    p.nterms = nterms;
    for (int t = 0; t < 6; ++t) { p.pa[t] = t < nterms ? pa[t] : 0; p.pb[t] = t < nterms ? pb[t] : 0; }
    p.splits = splits;
    p.ktiles_per_split = (ktiles + splits - 1) / splits;
    // drop empty trailing splits
    p.splits = splits = (ktiles + p.ktiles_per_split - 1) / p.ktiles_per_split;
    p.err = err_word;
    p.C = splits > 1 ? splitk_ws : c;
    p.ldc = splits > 1 ? N : ldc;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(tc_gemm_kernel), 4, max_smem);
    if (e != cudaSuccess) return e;
    const int n_items = ((N + bn - 1) / bn) * ((M + BM - 1) / BM) * splits;
    int ctas = sm_count * (two_ctas ? 2 : 1);
    if (ctas > n_items) ctas = n_items;
    tc_gemm_kernel<<<ctas, kTcThreads, smem, stream>>>(ma, mb, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ++*launches;
    if (splits > 1) {
        const size_t n4 = (size_t)M * (N / 4);
        int blocks = (int)((n4 + 255) / 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(splitk_ws, c, col_scale, M, N, ldc, splits);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        ++*launches;
    }
    return cudaSuccess;
}

// K-major use: 2-D {cols, rows}, box {32, box_outer rows}, 128-byte swizzle.  MN-major use (cols % 32 == 0):
// 3-D {32, rows, cols / 32} with the 32-column chunk as the outermost index, box {32, 32, box_outer chunks},
// 128-byte swizzle with 32-byte atoms.  Elements outside the tensor read as zero.
bool tc_encode_map_f32(void* map, const float* base, int cols, int rows, int ld, int mn_major, int box_outer) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    CUtensorMap* m = static_cast<CUtensorMap*>(map);
    void* ptr = const_cast<float*>(base);
    if (!mn_major) {
        cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
        cuuint32_t box[2] = {32, (cuuint32_t)box_outer};
        cuuint32_t estr[2] = {1, 1};
        return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (cols % 32 != 0) return false;
    cuuint64_t dims[3] = {32, (cuuint64_t)rows, (cuuint64_t)(cols / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 4, 128};
    cuuint32_t box[3] = {32, 32, (cuuint32_t)box_outer};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tc_encode_map_bf16(void* map, const void* base, int cols, int rows, int ld, int box_outer) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    return enc(static_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t launch_splitk_reduce(const float* partial, float* c, const float* col_scale, int M, int N, int ldc,
                                 int splits, cudaStream_t stream) {
    const size_t n4 = (size_t)M * (N / 4);
    int blocks = (int)((n4 + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(partial, c, col_scale, M, N, ldc, splits);
    return cudaGetLastError();
}

cudaError_t launch_split_planes(const float* src, int R, int Cc, const float* col_scale, void* planes, int ld_n,
                                int nterms, void* planes_t, int ld_t, int nterms_t, cudaStream_t stream) {
    dim3 grid((Cc + 63) / 64, (R + 63) / 64);
    if ((Cc & 3) == 0 && (R & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
        (col_scale == nullptr || (reinterpret_cast<uintptr_t>(col_scale) & 15) == 0)) {
        split_planes_vec_kernel<<<grid, 256, 0, stream>>>(src, R, Cc, col_scale, static_cast<__nv_bfloat16*>(planes),
                                                          ld_n, static_cast<__nv_bfloat16*>(planes_t), ld_t, nterms,
                                                          nterms_t);
        return cudaGetLastError();
    }
    split_planes_kernel<<<grid, 256, 0, stream>>>(src, R, Cc, col_scale, static_cast<__nv_bfloat16*>(planes), ld_n,
                                                  static_cast<__nv_bfloat16*>(planes_t), ld_t, nterms, nterms_t);
    return cudaGetLastError();
}

cudaError_t launch_expand_ternary(const uint8_t* state, int C, int O, int I, void* T, int ld_i, void* Tt, int ld_o,
                                  cudaStream_t stream) {
    dim3 grid((I + 63) / 64, (O + 63) / 64);
    expand_ternary_kernel<<<grid, 256, 0, stream>>>(state, C, O, I, static_cast<__nv_bfloat16*>(T), ld_i,
                                                    static_cast<__nv_bfloat16*>(Tt), ld_o);
    return cudaGetLastError();
}

cudaError_t launch_expand_ternary_p2(const uint32_t* packed2, int O, int I, void* T, int ld_i, void* Tt, int ld_o,
                                     cudaStream_t stream) {
    dim3 grid((I + 63) / 64, (O + 63) / 64);
    expand_ternary_p2_kernel<<<grid, 256, 0, stream>>>(packed2, O, I, static_cast<__nv_bfloat16*>(T), ld_i,
                                                       static_cast<__nv_bfloat16*>(Tt), ld_o);
    return cudaGetLastError();
}

}  // namespace mcl
