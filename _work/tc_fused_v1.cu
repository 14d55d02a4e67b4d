// Grouped tensor-core contractions with the fp32 -> bf16 term split done inside the kernel.
//
// tc_gemm.cu serves large layers from pre-split bf16 planes; every fp32 activation is then read
// once, written as 3 + 3 bf16 planes and read again by each product (28 bytes moved per 4-byte
// element).  For narrow layers (in/out features up to ~1024, many tokens) that traffic, not the
// tensor pipe, sets the step time.  Here the operands go global fp32 -> registers -> bf16 terms
// in shared memory (128-byte swizzled K-major tiles, the layout tcgen05.mma reads) -> TMEM, so
// each product reads its fp32 operands once and nothing intermediate touches HBM.  The ternary
// operand is expanded from the 2-bit packed weights on the fly.
//
// One launch runs a TABLE of problems (the three products of a step for up to 42 linears): work
// items (problem, 128-row tile, column tile, K slice) are dealt round-robin to persistent CTAs.
//   MotifCL computes the same products with scalar fp32 FMAs: kernels/compact_counter.cl:37-65
//   (forward), :207-233 (backward to input), kernels/matmul.cl:413-563 (dW = dY^T X).
//
// Problem kinds (A is [M,K], B is [N,K], C = A . B^T):
//   kFusedY   A[m][k] = a_src[m*lda + k]                  B[n][k] = T[n][k]   (packed2 row n)
//   kFusedDX  A[m][k] = a_src[m*lda + k] * a_kscale[k]    B[n][k] = T[k][n]   (packed2 row k)
//   kFusedDW  A[m][k] = a_src[k*lda + m]                  B[n][k] = b_src[k*ldb + n]
//
// CTA = 24 warps = 6 warpgroups of 80 registers per thread; setmaxnreg moves registers from the first
// two warpgroups to the converters (40 + 56 + 4 x 96 = 6 x 80: an increase can only be served from
// what the CTA itself released, so the sum must not exceed the launch allocation):
//   warp 0        allocates TMEM, one lane issues tcgen05.mma and commits (warps 1..3 idle)
//   warps 4..7    epilogue: tcgen05.ld of TMEM lane quarter (warp & 3), scale, 128-bit stores
//   warps 8..23   two converter groups of 8 warps; group g fills shared-memory stage g with the
//                 k-tiles it % 2 == g: loads go out, the group waits for its stage to be released
//                 by the MMA commit, splits, stores, fences to the async proxy and arrives
// Two accumulators in TMEM let the epilogue of one item overlap the main loop of the next.
// Every wait is bounded (see mbar_wait); on time-out the kernel records an error word and drains.
#include <cuda_bf16.h>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace mcl {
namespace {

constexpr int kFThreads = 24 * 32;
constexpr int kEpiWarp0 = 4;
constexpr int kConvWarp0 = 8;
constexpr int kATerm = 128 * 128;            // bytes of one A term tile (128 rows x 64 bf16)
constexpr int kStageB = 3 * kATerm;          // B tiles start here within a stage
constexpr int kStage = 6 * kATerm;           // 96 KiB
constexpr int kAccStride = 256;              // TMEM columns between the two accumulators

template <int CAP>
struct FusedTable {
    int n_problems, n_items, pad0, pad1;
    FusedProblem p[CAP];
};

__device__ __forceinline__ uint32_t idesc_bf16_f32(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct Item {
    int pi, mt, nt, kt0, nkt, split;
};

// item -> problem (items of a problem are contiguous; `pi` only moves forward)
template <int CAP>
__device__ __forceinline__ Item decode_item(const FusedTable<CAP>& tab, int item, int& pi) {
    while (pi + 1 < tab.n_problems && item >= tab.p[pi + 1].item_begin) ++pi;
    const FusedProblem& P = tab.p[pi];
    const int local = item - P.item_begin;
    Item it;
    it.pi = pi;
    // column tile fastest: the items that share an A slab run at the same time on neighbouring CTAs
    it.nt = local % P.tiles_n;
    const int rest = local / P.tiles_n;
    it.mt = rest % P.tiles_m;
    it.split = rest / P.tiles_m;
    const int ktiles = (P.K + 63) >> 6;
    it.kt0 = it.split * P.ktiles_per_split;
    it.nkt = min(P.ktiles_per_split, ktiles - it.kt0);
    return it;
}

__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// (lo, hi) -> term t in out[t]; lo/hi are replaced by their residuals
template <int NT>
__device__ __forceinline__ void split_pair(float lo, float hi, uint32_t (&out)[3]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const uint32_t h = pack_bf2(lo, hi);
        out[t] = h;
        if (t + 1 < NT) {
            lo -= __uint_as_float(h << 16);
            hi -= __uint_as_float(h & 0xffff0000u);
        }
    }
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
}
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// ---- converters: fp32 rows (K contiguous) -> A term tiles ------------------------------------------
// Warp w of a group owns rows 16w .. 16w+15 of the 128-row tile; a load instruction covers two rows
// of 256 contiguous bytes; every half-warp stores one full 128-byte swizzled row (conflict-free).
__device__ __forceinline__ void load_rows_a(const FusedProblem& P, int m0, int k0, int w, int l, float4 (&d)[8],
                                            float4& ksc) {
    const int c4 = l & 15, k = k0 + 4 * c4;
    const bool kin = k < P.K;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int m = m0 + 16 * w + (l >> 4) + 2 * g;
        d[g] = (kin && m < P.M) ? ldg4(P.a_src + (size_t)m * P.lda + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    ksc = (P.a_kscale != nullptr && kin) ? ldg4(P.a_kscale + k) : make_float4(1.f, 1.f, 1.f, 1.f);
}
template <int NT>
__device__ __forceinline__ void store_rows_a(uint32_t tile, int w, int l, const float4 (&d)[8], const float4 ksc,
                                             bool scaled) {
    const int c4 = l & 15;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int r = 16 * w + (l >> 4) + 2 * g;
        float4 v = d[g];
        if (scaled) {
            v.x = __fmul_rn(v.x, ksc.x); v.y = __fmul_rn(v.y, ksc.y);
            v.z = __fmul_rn(v.z, ksc.z); v.w = __fmul_rn(v.w, ksc.w);
        }
        uint32_t a[3], b[3];
        split_pair<NT>(v.x, v.y, a);
        split_pair<NT>(v.z, v.w, b);
        const uint32_t addr = tile + (uint32_t)r * 128u + ((uint32_t)((c4 >> 1) ^ (r & 7)) << 4) + (uint32_t)(c4 & 1) * 8u;
#pragma unroll
        for (int t = 0; t < NT; ++t) sts64(addr + (uint32_t)t * kATerm, a[t], b[t]);
    }
}

// ---- converters: 2-bit packed weights -> ternary B tile ------------------------------------------------
// A word holds 16 weights (field = t + 1).  0x55555555 is a word of zeros, used as the fill value.
__device__ __forceinline__ void load_p2(const FusedProblem& P, int n0, int k0, int tg, uint32_t (&words)[4]) {
    const int BN = P.BN;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int u = tg + 256 * r;
        uint32_t word = 0x55555555u;
        if (P.mode == kFusedY) {
            const int n = u >> 2, kw = (k0 >> 4) + (u & 3);
            if (n < BN && n0 + n < P.N && kw < (P.K >> 4)) word = __ldg(P.packed2 + (size_t)(n0 + n) * P.p2_stride + kw);
        } else {
            const int k = u & 63, wq = u >> 6, nw = (n0 >> 4) + wq;
            if (wq < (BN >> 4) && k0 + k < P.K && nw < (P.N >> 4)) word = __ldg(P.packed2 + (size_t)(k0 + k) * P.p2_stride + nw);
        }
        words[r] = word;
    }
}
__device__ __forceinline__ void store_p2(const FusedProblem& P, uint32_t tile, int tg, const uint32_t (&words)[4],
                                         const uint2* lut4) {
    const int BN = P.BN;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int u = tg + 256 * r;
        const uint32_t word = words[r];
        if (P.mode == kFusedY) {
            const int n = u >> 2, wq = u & 3;
            if (n < BN) {
                const uint2 e0 = lut4[word & 255u], e1 = lut4[(word >> 8) & 255u];
                const uint2 e2 = lut4[(word >> 16) & 255u], e3 = lut4[word >> 24];
                const uint32_t row = tile + (uint32_t)n * 128u;
                sts128(row + ((uint32_t)((2 * wq) ^ (n & 7)) << 4), e0.x, e0.y, e1.x, e1.y);
                sts128(row + ((uint32_t)((2 * wq + 1) ^ (n & 7)) << 4), e2.x, e2.y, e3.x, e3.y);
            }
        } else {
            const int k = u & 63, wq = u >> 6;
            if (wq < (BN >> 4)) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint2 e = lut4[(word >> (8 * q)) & 255u];
                    const int n = 16 * wq + 4 * q;       // n & 7 is 0 or 4; rows n .. n+3
                    const uint32_t base = tile + (uint32_t)n * 128u + (uint32_t)(k & 7) * 2u;
                    const uint32_t kc = (uint32_t)(k >> 3);
                    sts16(base + ((kc ^ (uint32_t)((n + 0) & 7)) << 4), e.x & 0xffffu);
                    sts16(base + 128u + ((kc ^ (uint32_t)((n + 1) & 7)) << 4), e.x >> 16);
                    sts16(base + 256u + ((kc ^ (uint32_t)((n + 2) & 7)) << 4), e.y & 0xffffu);
                    sts16(base + 384u + ((kc ^ (uint32_t)((n + 3) & 7)) << 4), e.y >> 16);
                }
            }
        }
    }
}

// ---- converters: fp32 with the FEATURE contiguous (K = token rows) -> transposed term tiles ------------------
// One pass = 32 features x 32 tokens per warp: a lane loads 4 features x 8 tokens (8 float4) and
// stores, per feature and term, one 16-byte chunk of 8 consecutive k.
__device__ __forceinline__ void load_cols(const float* src, int ld, int n_feat, int K, int f0, int k0, int pass, int l,
                                          float4 (&d)[8]) {
    const int mq = (l & 1) + 2 * (l >> 3), kc = (l >> 1) & 3;
    const int f = f0 + 32 * (pass >> 1) + 4 * mq;
    const int k = k0 + 32 * (pass & 1) + 8 * kc;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        d[j] = (f < n_feat && k + j < K) ? ldg4(src + (size_t)(k + j) * ld + f) : make_float4(0.f, 0.f, 0.f, 0.f);
}
template <int NT>
__device__ __forceinline__ void store_cols(uint32_t tile, uint32_t term_stride, int pass, int l, const float4 (&d)[8]) {
    const int mq = (l & 1) + 2 * (l >> 3), kc = (l >> 1) & 3;
    const uint32_t chunk = (uint32_t)(4 * (pass & 1) + kc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = 32 * (pass >> 1) + 4 * mq + i;
        float e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = i == 0 ? d[j].x : i == 1 ? d[j].y : i == 2 ? d[j].z : d[j].w;
        uint32_t p0[3], p1[3], p2[3], p3[3];
        split_pair<NT>(e[0], e[1], p0);
        split_pair<NT>(e[2], e[3], p1);
        split_pair<NT>(e[4], e[5], p2);
        split_pair<NT>(e[6], e[7], p3);
        const uint32_t addr = tile + (uint32_t)row * 128u + ((chunk ^ (uint32_t)(row & 7)) << 4);
#pragma unroll
        for (int t = 0; t < NT; ++t) sts128(addr + (uint32_t)t * term_stride, p0[t], p1[t], p2[t], p3[t]);
    }
}

#ifdef MCL_FUSED_PROF
__device__ long long g_fused_prof[148 * 2 * 4 + 148 * 8];
__device__ __forceinline__ long long gtime() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define PROF_T(var) const long long var = clock64()
#else
#define PROF_T(var)
#endif

template <int CAP>
__global__ void __launch_bounds__(kFThreads, 1) tc_fused_kernel(const __grid_constant__ FusedTable<CAP> tab, int* err) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[8];
    __shared__ uint2 lut4[256];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef MCL_FUSED_PROF
    if (threadIdx.x == 0) g_fused_prof[148 * 8 + blockIdx.x * 8 + 0] = gtime();
#endif
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (2 + s); };
    auto acc_full = [&](int a) { return bar0 + 8u * (4 + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (6 + a); };

    if (threadIdx.x == 0) {
        abort_flag = (*reinterpret_cast<volatile int*>(err) != 0);
        for (int s = 0; s < 2; ++s) { mbar_init(full_bar(s), 256); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 256) {
        // byte of four 2-bit fields -> four bf16 of (field - 1): -1, 0, 1, 2
        uint32_t h[4];
        for (int q = 0; q < 4; ++q) {
            const uint32_t f = (threadIdx.x >> (2 * q)) & 3u;
            h[q] = f == 0 ? 0xBF80u : f == 1 ? 0u : f == 2 ? 0x3F80u : 0x4000u;
        }
        lut4[threadIdx.x] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const int n_items = tab.n_items;
#ifdef MCL_FUSED_PROF
    if (threadIdx.x == 0) g_fused_prof[148 * 8 + blockIdx.x * 8 + 1] = gtime();
#endif

    if (warp < kEpiWarp0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 0 && lane == 0) {
            // ---- MMA issuer ------------------------------------------------------------------------
            uint32_t it = 0, n_local = 0;
            int pi = 0;
            for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x, ++n_local) {
                const Item I = decode_item(tab, item, pi);
                const FusedProblem& P = tab.p[I.pi];
                const uint32_t idesc = idesc_bf16_f32(128, P.BN);
                const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
                if (!mbar_wait(acc_empty(acc), aph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 14); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccStride;
                const uint32_t b_term = (uint32_t)P.BN * 128u;
                for (int j = 0; j < I.nkt; ++j, ++it) {
                    const int s = (int)(it & 1u);
                    if (!mbar_wait(full_bar(s), (it >> 1) & 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 12); break; }
                    tc_fence_after();
                    const uint32_t a0 = tiles + (uint32_t)s * kStage, b0 = a0 + kStageB;
                    uint32_t prod = P.prod;
                    for (int q = 0; q < P.nprod; ++q, prod >>= 4) {
                        const uint64_t da = smem_desc_k_sw128(a0 + (prod & 3u) * kATerm);
                        const uint64_t db = smem_desc_k_sw128(b0 + ((prod >> 2) & 3u) * b_term);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma_bf16(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (j | q | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));
                }
                if (abort_flag) break;
                umma_commit(acc_full(acc));
            }
        }
    } else if (warp < kConvWarp0) {
        // ---- epilogue warps ----------------------------------------------------------------------------
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        const int q = warp & 3;
        uint32_t n_local = 0;
        int pi = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n_local) {
            const Item I = decode_item(tab, item, pi);
            const FusedProblem& P = tab.p[I.pi];
            const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
            bool ok = !abort_flag;
            if (ok && !mbar_wait(acc_full(acc), aph, &abort_flag)) { abort_flag = 1; atomicExch(err, 13); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const bool scale = (P.col_scale != nullptr) && P.splits == 1;
            const int BN = P.BN, n0 = I.nt * BN;
            const int row = I.mt * 128 + q * 32 + lane;
            float* crow = P.C + ((size_t)I.split * P.M + row) * P.ldc;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= P.N) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + acc * kAccStride + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                tmem_ld_wait();
                if (row < P.M) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int col = n0 + c0 + j;
                        if (col >= P.N || c0 + j >= BN) break;
                        float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                               __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        if (scale) {
                            const float4 sc = ldg4(P.col_scale + col);
                            o.x *= sc.x; o.y *= sc.y; o.z *= sc.z; o.w *= sc.w;
                        }
                        *reinterpret_cast<float4*>(crow + col) = o;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty(acc));
        }
    } else {
        // ---- converter groups ----------------------------------------------------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 96;");
        const int cw = warp - kConvWarp0, g = cw >> 3, w = cw & 7, tg = (cw & 7) * 32 + lane;
        const uint32_t stage = tiles + (uint32_t)g * kStage;
        uint32_t it = 0, mine = 0;
        int pi = 0;
#ifdef MCL_FUSED_PROF
        long long pf_load = 0, pf_empty = 0, pf_conv = 0, pf_tiles = 0;
#endif
        for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x) {
            const Item I = decode_item(tab, item, pi);
            const FusedProblem& P = tab.p[I.pi];
            const int m0 = I.mt * 128, n0 = I.nt * P.BN;
            for (int j = 0; j < I.nkt; ++j, ++it) {
                if ((int)(it & 1u) != g) continue;
                const int k0 = (I.kt0 + j) * 64;
                bool ok = true;
                if (P.mode != kFusedDW) {
                    float4 d[8], ksc;
                    uint32_t words[4];
                    PROF_T(t0);
                    load_rows_a(P, m0, k0, w, lane, d, ksc);
                    load_p2(P, n0, k0, tg, words);
#ifdef MCL_FUSED_PROF
                    if (__float_as_uint(d[7].w) + __float_as_uint(d[0].x) + words[3] == 0x7fc12345u) atomicExch(err, 99);
#endif
                    PROF_T(t1);
                    ok = mbar_wait(empty_bar(g), (mine & 1u) ^ 1u, &abort_flag);
                    PROF_T(t2);
                    if (ok) {
                        if (P.na == 3) store_rows_a<3>(stage, w, lane, d, ksc, P.a_kscale != nullptr);
                        else store_rows_a<2>(stage, w, lane, d, ksc, P.a_kscale != nullptr);
                        store_p2(P, stage + kStageB, tg, words, lut4);
                    }
#ifdef MCL_FUSED_PROF
                    { PROF_T(t3); pf_load += t1 - t0; pf_empty += t2 - t1; pf_conv += t3 - t2; ++pf_tiles; }
#endif
                } else {
                    float4 da[8], db[8];
                    const int b_passes = (P.BN >> 5) * 2;
                    load_cols(P.a_src, P.lda, P.M, P.K, m0, k0, w, lane, da);
                    PROF_T(t0);
                    if (w < b_passes) load_cols(P.b_src, P.ldb, P.N, P.K, n0, k0, w, lane, db);
#ifdef MCL_FUSED_PROF
                    if (__float_as_uint(da[7].w) + __float_as_uint(db[7].x) == 0x7fc12345u) atomicExch(err, 99);
#endif
                    PROF_T(t1);
                    ok = mbar_wait(empty_bar(g), (mine & 1u) ^ 1u, &abort_flag);
                    PROF_T(t2);
                    if (ok) {
                        const uint32_t b_term = (uint32_t)P.BN * 128u;
                        if (P.na == 3) {
                            store_cols<3>(stage, kATerm, w, lane, da);
                            if (w < b_passes) store_cols<3>(stage + kStageB, b_term, w, lane, db);
                        } else {
                            store_cols<2>(stage, kATerm, w, lane, da);
                            if (w < b_passes) store_cols<2>(stage + kStageB, b_term, w, lane, db);
                        }
                    }
#ifdef MCL_FUSED_PROF
                    { PROF_T(t3); pf_load += t1 - t0; pf_empty += t2 - t1; pf_conv += t3 - t2; ++pf_tiles; }
#endif
                }
                if (!ok) { abort_flag = 1; atomicExch(err, 11); break; }
                fence_proxy_async();
                mbar_arrive(full_bar(g));
                ++mine;
            }
        }
#ifdef MCL_FUSED_PROF
        if (w == 0 && lane == 0 && blockIdx.x < 148) {
            long long* o = g_fused_prof + (blockIdx.x * 2 + g) * 4;
            o[0] = pf_load; o[1] = pf_empty; o[2] = pf_conv; o[3] = pf_tiles;
            g_fused_prof[148 * 8 + blockIdx.x * 8 + 2 + g] = gtime();
        }
#endif
    }
    __syncwarp();
    if (abort_flag) {
        // gave up: let MMAs that may still read shared memory finish before it is released
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 2000000ull) {}
    }
    tc_fence_before();
    __syncthreads();
#ifdef MCL_FUSED_PROF
    if (threadIdx.x == 0) g_fused_prof[148 * 8 + blockIdx.x * 8 + 4] = gtime();
#endif
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

int pick_bn(int N, int step, int lo, int hi) {
    int best = hi, best_waste = 1 << 30;
    for (int bn = hi; bn >= lo; bn -= step) {
        const int waste = ((N + bn - 1) / bn) * bn - N;
        if (waste < best_waste) { best_waste = waste; best = bn; }
    }
    return best;
}

}  // namespace

size_t fused_plan(FusedProblem* p, int target_items, int depth_limit) {
    const int ktiles = (p->K + 63) / 64;
    p->tiles_m = (p->M + 127) / 128;
    if (p->mode != kFusedDW) {
        p->BN = pick_bn(p->N, 16, 16, 256);
        p->tiles_n = (p->N + p->BN - 1) / p->BN;
        p->splits = 1;
        p->ktiles_per_split = ktiles;
        return 0;
    }
    p->BN = pick_bn(p->N, 32, 32, 128);
    p->tiles_n = (p->N + p->BN - 1) / p->BN;
    const int tiles = p->tiles_m * p->tiles_n;
    int splits = (target_items + tiles - 1) / tiles;
    if (splits > ktiles / 4) splits = ktiles / 4;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    if (depth_limit > 0 && (ktiles + splits - 1) / splits > depth_limit) splits = (ktiles + depth_limit - 1) / depth_limit;
    p->ktiles_per_split = (ktiles + splits - 1) / splits;
    p->splits = (ktiles + p->ktiles_per_split - 1) / p->ktiles_per_split;
    return p->splits > 1 ? (size_t)p->splits * p->M * p->N : 0;
}

template <int CAP>
static cudaError_t launch_fused_cap(const FusedProblem* probs, int n, int n_items, int* err_word, size_t max_smem,
                                    int sm_count, int slot, cudaStream_t stream) {
    FusedTable<CAP> tab;             // the by-value kernel argument
    tab.n_problems = n;
    tab.n_items = n_items;
    for (int i = 0; i < n; ++i) tab.p[i] = probs[i];
    const size_t smem = 2 * (size_t)kStage + 1024;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(tc_fused_kernel<CAP>), slot, max_smem);
    if (e != cudaSuccess) return e;
    const int ctas = n_items < sm_count ? n_items : sm_count;
    tc_fused_kernel<CAP><<<ctas, kFThreads, smem, stream>>>(tab, err_word);
    return cudaGetLastError();
}

cudaError_t launch_tc_fused(FusedProblem* probs, int n, int* err_word, size_t max_smem, int sm_count,
                            cudaStream_t stream, int* launches) {
    if (n < 1 || n > kFusedMaxProblems) return cudaErrorInvalidValue;
    int items = 0;
    for (int i = 0; i < n; ++i) {
        FusedProblem& p = probs[i];
        if (p.mode == kFusedDW ? (p.BN > 128 || (p.BN & 31)) : (p.BN > 256 || (p.BN & 15))) return cudaErrorInvalidValue;
        if ((p.N & 3) || (p.ldc & 3) || (p.K & 3) || (p.lda & 3)) return cudaErrorInvalidValue;
        p.item_begin = items;
        items += p.tiles_m * p.tiles_n * p.splits;
    }
    if (2 * (size_t)kStage + 1024 + 4096 > max_smem) return cudaErrorInvalidConfiguration;
    cudaError_t e = n <= 4 ? launch_fused_cap<4>(probs, n, items, err_word, max_smem, sm_count, 6, stream)
                           : launch_fused_cap<kFusedMaxProblems>(probs, n, items, err_word, max_smem, sm_count, 7, stream);
    if (e == cudaSuccess) ++*launches;
    return e;
}

#ifdef MCL_FUSED_PROF
extern "C" int mcl_debug_fused_prof(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_fused_prof, sizeof(long long) * (148 * 2 * 4 + 148 * 8));
}
#endif

}  // namespace mcl
