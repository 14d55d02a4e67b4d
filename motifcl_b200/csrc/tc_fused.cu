// Grouped tensor-core contractions for narrow layers: fp32 operands go from global memory to the
// tensor cores without an intermediate copy in HBM.
//
// tc_gemm.cu serves wide layers from pre-split bf16 planes: every fp32 activation is read once,
// written as 3 + 3 bf16 planes and read again by each product (28 bytes moved per 4-byte element).
// For narrow layers (in/out features up to ~1024, many tokens) that traffic, not the tensor pipe,
// sets the step time.  Here TMA brings the RAW fp32 tiles into shared memory and the products run
// as tcgen05.mma.kind::tf32 on two terms per fp32 operand:
//     a = hi + lo,   hi = a with the low 13 mantissa bits cleared (what the tensor core reads of a
//                         raw fp32 word),  lo = tf32_round(a - hi)   (a - hi is exact)
// so `hi` needs no work at all and `lo` is one elementwise pass over the tile in shared memory.
// a.b is taken as lo.b + hi.b for an exact (ternary) b and as lo_a.hi_b + hi_a.lo_b + hi_a.hi_b for
// two fp32 operands; the dropped lo.lo and the rounding of lo are ~2^-22 relative.
//
// One launch runs a TABLE of problems (the three products of a step for many linears): work items
// (problem, 128-row tile, column tile, K slice) are dealt round-robin to persistent CTAs.
//   MotifCL computes the same products with scalar fp32 FMAs: kernels/compact_counter.cl:37-65
//   (forward), :207-233 (backward to input), kernels/matmul.cl:413-563 (dW = dY^T X).
//
// Problem kinds (C[M,N] = A[M,K] . B[N,K]^T); every tensor is row-major fp32 behind a TMA map with
// a 32 x 32 box and the 128-byte swizzle:
//   kFusedY   A = X  [tokens,in]  K-major              B = T [out,in]  K-major   (exact)
//   kFusedDX  A = dY [tokens,out] K-major, x scale[k]  B = T [out,in]  MN-major  (exact)
//   kFusedDW  A = dY [tokens,out] MN-major             B = X [tokens,in] MN-major
// "MN-major" = the M (or N) index is the contiguous one in memory, the layout a transposed
// operand has; the tensor core reads it in place (instruction-descriptor transpose bits), so no
// transposed copy of an activation is ever made.
//
// CTA = 16 warps, 3 shared-memory stages of one 32-deep k-tile each:
//   warp 0        TMA producer (one lane): 32 x 32 boxes of A and B, mbarrier complete_tx
//   warp 1        allocates TMEM; one lane issues tcgen05.mma and commits
//   warps 4..7    epilogue: tcgen05.ld of TMEM lane quarter (warp & 3), scale, 128-bit stores
//   warps 8..15   converters: wait for the boxes, write the `lo` tiles (and the scaled `hi` tile
//                 for dX), fence to the async proxy, arrive
// Two accumulators in TMEM let the epilogue of one item overlap the main loop of the next.
// Every wait is bounded (see mbar_wait); on time-out the kernel records an error word and drains.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

#include "counter_codec.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace mcl {
namespace {

constexpr int kFThreads = 16 * 32;
constexpr int kEpiWarp0 = 4;
constexpr int kConvWarp0 = 8;
constexpr int kConvThreads = 8 * 32;
constexpr int kStages = 3;
constexpr int kBox = 32 * 32 * 4;            // bytes of one 32 x 32 fp32 box
constexpr int kALo = 4 * kBox;               // stage layout: A hi (4 boxes), A lo, B hi (<= 8 boxes) ...
constexpr int kBHi = 8 * kBox;               // ... and, for two fp32 operands, B lo at kBHi + 4 boxes
constexpr int kBLo = 12 * kBox;
constexpr int kStage = 16 * kBox;            // 64 KiB
constexpr int kAccStride = 256;              // TMEM columns between the two accumulators

template <int CAP>
struct FusedTable {
    CUtensorMap maps[2 * CAP];
    int n_problems, n_items, pad0, pad1;
    FusedProblem p[CAP];
};

// Instruction descriptor, kind::tf32: D = f32 (bits 4-5 = 1), A = B = tf32 (bits 7-9, 10-12 = 2),
// bit 15 / 16 = A / B is MN-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t idesc_tf32(int m, int n, bool a_mn, bool b_mn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Shared-memory layouts.  K-major: rows of 128 bytes (32 fp32 of k) in the 128-byte swizzle, 8-row
// groups 1024 bytes apart (stride byte offset).  MN-major: rows of 128 bytes hold 32 consecutive m (or
// n) for one k, in the 128-byte swizzle with 32-byte atoms (the form the tensor core can transpose
// 32-bit data from): 4 k-rows per 512 bytes (stride byte offset), the next 32 m one box = 4096 bytes
// further (leading byte offset).
__device__ __forceinline__ void umma_tf32(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accum) : "memory");
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
    const int ktiles = (P.K + 31) >> 5;
    it.kt0 = it.split * P.ktiles_per_split;
    it.nkt = min(P.ktiles_per_split, ktiles - it.kt0);
    return it;
}

__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// lo term of a: a minus what the tensor core reads of the raw word, rounded to tf32
__device__ __forceinline__ float lo_term(float a) {
    const float r = a - __uint_as_float(__float_as_uint(a) & 0xffffe000u);
    uint32_t t;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(r));
    return __uint_as_float(t);
}
__device__ __forceinline__ float4 lo_term4(float4 v) {
    return make_float4(lo_term(v.x), lo_term(v.y), lo_term(v.z), lo_term(v.w));
}

#ifdef MCL_FUSED_PROF
__device__ long long g_fused_prof[148 * 16];
#define PROF_T(var) const long long var = clock64()
#define PROF_ADD(acc, a, b) acc += (b) - (a)
#else
#define PROF_T(var)
#define PROF_ADD(acc, a, b)
#endif

template <int CAP>
__global__ void __launch_bounds__(kFThreads, 1) tc_fused_kernel(const __grid_constant__ FusedTable<CAP> tab, int* err) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[3 * kStages + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(bars);
    auto tma_full = [&](int s) { return bar0 + 8u * s; };
    auto conv_full = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto empty_bar = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
    auto acc_full = [&](int a) { return bar0 + 8u * (3 * kStages + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (3 * kStages + 2 + a); };

    if (threadIdx.x == 0) {
        abort_flag = (*reinterpret_cast<volatile int*>(err) != 0);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(tma_full(s), 1);
            mbar_init(conv_full(s), kConvThreads);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const int n_items = tab.n_items;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----------------------------------------------------------------------
            uint32_t it = 0;
            int pi = 0;
            long long pf_wait = 0, pf_issue = 0; (void)pf_wait; (void)pf_issue;
            PROF_T(tstart);
            for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x) {
                const Item I = decode_item(tab, item, pi);
                const FusedProblem& P = tab.p[I.pi];
                const CUtensorMap* ma = &tab.maps[P.a_map];
                const CUtensorMap* mb = &tab.maps[P.b_map];
                const int m0 = I.mt * 128, n0 = I.nt * P.BN;
                for (int j = 0; j < I.nkt; ++j, ++it) {
                    const int s = (int)(it % kStages);
                    const uint32_t ph = (it / kStages) & 1u;
                    PROF_T(t0);
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 11); break; }
                    PROF_T(t1); PROF_ADD(pf_wait, t0, t1);
                    const uint32_t st = tiles + (uint32_t)s * kStage;
                    const int k0 = (I.kt0 + j) * 32;
                    mbar_expect_tx(tma_full(s), 4u * kBox + (uint32_t)P.BN * 128u);
                    // K-major: one box of 32 k x rows; MN-major: one box of 32 m x 32 k x chunks (3-D map)
                    if (P.mode == kFusedDW) tma_load_3d(st, ma, tma_full(s), 0, k0, m0 >> 5);
                    else tma_load_2d(st, ma, tma_full(s), k0, m0);
                    if (P.mode == kFusedY) tma_load_2d(st + kBHi, mb, tma_full(s), k0, n0);
                    else tma_load_3d(st + kBHi, mb, tma_full(s), 0, k0, n0 >> 5);
                    PROF_T(t2); PROF_ADD(pf_issue, t1, t2);
                }
            }
#ifdef MCL_FUSED_PROF
            { PROF_T(tend); long long* o = g_fused_prof + blockIdx.x * 16; o[0] = pf_wait; o[1] = pf_issue; o[2] = tend - tstart; o[3] = it; }
#endif
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ------------------------------------------------------------------------
            uint32_t it = 0, n_local = 0;
            int pi = 0;
            long long pf_acc = 0, pf_full = 0, pf_issue = 0; (void)pf_acc; (void)pf_full; (void)pf_issue;
            PROF_T(tstart);
            for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x, ++n_local) {
                const Item I = decode_item(tab, item, pi);
                const FusedProblem& P = tab.p[I.pi];
                const bool a_mn = P.mode == kFusedDW, b_mn = P.mode != kFusedY;
                const uint32_t idesc = idesc_tf32(128, P.BN, a_mn, b_mn);
                // descriptor words: low = address / 16 | leading byte offset / 16 << 16, high = stride byte offset / 16 |
                // version bit | layout type << 29 (1 = 128-byte swizzle with 32-byte atoms, 2 = 128-byte swizzle)
                const uint32_t a_step = a_mn ? 64u : 2u, b_step = b_mn ? 64u : 2u;          // 16-byte units per 8 k
                const uint32_t a_lo = a_mn ? ((uint32_t)(kBox >> 4) << 16) : (1u << 16);
                const uint32_t b_lo = b_mn ? ((uint32_t)(kBox >> 4) << 16) : (1u << 16);
                const uint32_t a_hi = a_mn ? ((512u >> 4) | (1u << 14) | (1u << 29)) : ((1024u >> 4) | (1u << 14) | (2u << 29));
                const uint32_t b_hi = b_mn ? ((512u >> 4) | (1u << 14) | (1u << 29)) : ((1024u >> 4) | (1u << 14) | (2u << 29));
                const uint32_t nprod = (uint32_t)P.nprod, prod0 = P.prod;
                const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
                PROF_T(ta0);
                if (!mbar_wait(acc_empty(acc), aph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 14); break; }
                PROF_T(ta1); PROF_ADD(pf_acc, ta0, ta1);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccStride;
                uint32_t accum = 0;
                for (int j = 0; j < I.nkt; ++j, ++it) {
                    const int s = (int)(it % kStages);
                    PROF_T(t0);
                    if (!mbar_wait(conv_full(s), (it / kStages) & 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 12); break; }
                    PROF_T(t1); PROF_ADD(pf_full, t0, t1);
                    tc_fence_after();
                    const uint32_t st16 = (tiles + (uint32_t)s * kStage) >> 4;
                    uint32_t prod = prod0;
                    for (uint32_t q = 0; q < nprod; ++q, prod >>= 4) {
                        const uint32_t a16 = a_lo | (st16 + ((prod & 3u) ? (kALo >> 4) : 0u));
                        const uint32_t b16 = b_lo | (st16 + (((prod >> 2) & 3u) ? (kBLo >> 4) : (kBHi >> 4)));
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) {
                            const uint64_t da = ((uint64_t)a_hi << 32) | (uint64_t)(a16 + kk * a_step);
                            const uint64_t db = ((uint64_t)b_hi << 32) | (uint64_t)(b16 + kk * b_step);
                            umma_tf32(d_tmem, da, db, idesc, accum);
                            accum = 1u;
                        }
                    }
                    umma_commit(empty_bar(s));
                    PROF_T(t2); PROF_ADD(pf_issue, t1, t2);
                }
                if (abort_flag) break;
                umma_commit(acc_full(acc));
            }
#ifdef MCL_FUSED_PROF
            { PROF_T(tend); long long* o = g_fused_prof + blockIdx.x * 16 + 4; o[0] = pf_acc; o[1] = pf_full; o[2] = pf_issue; o[3] = tend - tstart; }
#endif
        }
    } else if (warp >= kEpiWarp0 && warp < kConvWarp0) {
        // ---- epilogue warps ----------------------------------------------------------------------------
        const int q = warp & 3;
        uint32_t n_local = 0;
        int pi = 0;
        long long pf_wait = 0, pf_store = 0; (void)pf_wait; (void)pf_store;
        PROF_T(tstart);
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n_local) {
            PROF_T(t0);
            const Item I = decode_item(tab, item, pi);
            const FusedProblem& P = tab.p[I.pi];
            const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
            bool ok = !abort_flag;
            if (ok && !mbar_wait_warp(acc_full(acc), aph, &abort_flag)) { abort_flag = 1; atomicExch(err, 13); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            PROF_T(t1); PROF_ADD(pf_wait, t0, t1);
            tc_fence_after();
            const bool scale = (P.col_scale != nullptr) && P.splits == 1;
            const int BN = P.BN, n0 = I.nt * BN;
            const int row0 = I.mt * 128 + q * 32;
            float* cbase = P.C + ((size_t)I.split * P.M + row0) * P.ldc;
            // The TMEM fragment (lane = row, 32 columns) goes through a swizzled 4 KiB tile of shared memory so
            // that a store instruction writes 4 rows x 128 contiguous bytes instead of 32 rows x 16 bytes.
            const uint32_t scratch = tiles + (uint32_t)kStages * kStage + (uint32_t)q * 4096u;
            const int rsub = lane >> 3, j4 = lane & 7;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= P.N) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + acc * kAccStride + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    sts128(scratch + (uint32_t)lane * 128u + ((uint32_t)(j ^ (lane & 7)) << 4),
                           make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                __syncwarp();
                const int col = n0 + c0 + 4 * j4;
                const bool col_ok = col < P.N && c0 + 4 * j4 < BN;
                float4 sc = make_float4(1.f, 1.f, 1.f, 1.f);
                if (scale && col_ok) sc = __ldg(reinterpret_cast<const float4*>(P.col_scale + col));
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    const int rr = p * 4 + rsub;
                    float4 o = lds128(scratch + (uint32_t)rr * 128u + ((uint32_t)(j4 ^ (rr & 7)) << 4));
                    if (col_ok && row0 + rr < P.M) {
                        o.x *= sc.x; o.y *= sc.y; o.z *= sc.z; o.w *= sc.w;
                        *reinterpret_cast<float4*>(cbase + (size_t)rr * P.ldc + col) = o;
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            mbar_arrive(acc_empty(acc));
            PROF_T(t2); PROF_ADD(pf_store, t1, t2);
        }
#ifdef MCL_FUSED_PROF
        if (warp == kEpiWarp0 && lane == 0) { PROF_T(tend); long long* o = g_fused_prof + blockIdx.x * 16 + 8; o[0] = pf_wait; o[1] = pf_store; o[2] = tend - tstart; o[3] = n_local; }
#endif
    } else if (warp >= kConvWarp0) {
        // ---- converters --------------------------------------------------------------------------------
        const int tg = threadIdx.x - kConvWarp0 * 32;
        uint32_t it = 0;
        int pi = 0;
        long long pf_wait = 0, pf_work = 0; (void)pf_wait; (void)pf_work;
        PROF_T(tstart);
        for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x) {
            const Item I = decode_item(tab, item, pi);
            const FusedProblem& P = tab.p[I.pi];
            const int nb_lo = P.mode == kFusedDW ? (P.BN >> 5) : 0;     // boxes of B that need a lo tile
            const float* ksc = P.a_kscale;
            bool ok = true;
            for (int j = 0; j < I.nkt; ++j, ++it) {
                const int s = (int)(it % kStages);
                PROF_T(t0);
                ok = mbar_wait_warp(tma_full(s), (it / kStages) & 1u, &abort_flag);
                if (!ok) break;
                PROF_T(t1); PROF_ADD(pf_wait, t0, t1);
                const uint32_t st = tiles + (uint32_t)s * kStage;
                const int k0 = (I.kt0 + j) * 32;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int idx = tg + kConvThreads * r;            // 16-byte chunk of the A tile
                    const uint32_t addr = st + (uint32_t)idx * 16u;
                    float4 v = lds128(addr);
                    if (ksc != nullptr) {
                        const int k = k0 + 4 * ((idx & 7) ^ ((idx >> 3) & 7));     // undo the swizzle: logical k of this chunk
                        if (k < P.K) {
                            const float4 sc = __ldg(reinterpret_cast<const float4*>(ksc + k));
                            v.x = __fmul_rn(v.x, sc.x); v.y = __fmul_rn(v.y, sc.y);
                            v.z = __fmul_rn(v.z, sc.z); v.w = __fmul_rn(v.w, sc.w);
                            sts128(addr, v);
                        }
                    }
                    sts128(addr + kALo, lo_term4(v));
                }
                for (int r = 0; r < nb_lo; ++r) {
                    const uint32_t addr = st + kBHi + (uint32_t)(tg + kConvThreads * r) * 16u;
                    sts128(addr + (kBLo - kBHi), lo_term4(lds128(addr)));
                }
                fence_proxy_async();
                mbar_arrive(conv_full(s));
                PROF_T(t2); PROF_ADD(pf_work, t1, t2);
            }
            if (!ok) { abort_flag = 1; atomicExch(err, 15); break; }
        }
#ifdef MCL_FUSED_PROF
        if (tg == 0) { PROF_T(tend); long long* o = g_fused_prof + blockIdx.x * 16 + 12; o[0] = pf_wait; o[1] = pf_work; o[2] = tend - tstart; o[3] = it; }
#endif
    }
    __syncwarp();
    if (abort_flag) {
        // gave up: let copies and MMAs that may still touch shared memory finish before it is released
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 2000000ull) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- ternary digits as fp32 [O][I]: the exact operand of Y (K-major) and dX (MN-major) ----------------
__global__ void __launch_bounds__(256) ternary_f32_from_state_kernel(const uint8_t* __restrict__ state, int C,
                                                                     long long n_groups, float* __restrict__ T) {
    __shared__ DecodeLut lut;
    build_decode_lut(&lut, C, threadIdx.x, blockDim.x);
    __syncthreads();
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += (long long)gridDim.x * blockDim.x) {
        const uint8_t* s = state + g * 3;
        const uint32_t w = (uint32_t)__ldg(s) | ((uint32_t)__ldg(s + 1) << 8) | ((uint32_t)__ldg(s + 2) << 16);
        reinterpret_cast<float4*>(T)[g] = make_float4(lut.e[w & 63u].x, lut.e[(w >> 6) & 63u].x, lut.e[(w >> 12) & 63u].x,
                                                      lut.e[(w >> 18) & 63u].x);
    }
}
__global__ void __launch_bounds__(256) ternary_f32_from_p2_kernel(const uint32_t* __restrict__ packed2, long long n_words,
                                                                  float* __restrict__ T) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (long long)gridDim.x * blockDim.x) {
        const uint32_t w = __ldg(packed2 + i);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t b = w >> (8 * q);
            reinterpret_cast<float4*>(T)[i * 4 + q] = make_float4((float)((int)(b & 3u) - 1), (float)((int)((b >> 2) & 3u) - 1),
                                                                  (float)((int)((b >> 4) & 3u) - 1), (float)((int)((b >> 6) & 3u) - 1));
        }
    }
}

// fewest column tiles of at most `hi` columns, then the narrowest tile (a multiple of `step`) that covers N
int pick_bn(int N, int step, int hi) {
    const int tiles = (N + hi - 1) / hi;
    const int per = (N + tiles - 1) / tiles;
    return ((per + step - 1) / step) * step;
}

bool same_operand(const FusedOperand& a, const FusedOperand& b) {
    return a.ptr == b.ptr && a.rows == b.rows && a.cols == b.cols && a.ld == b.ld && a.mn_major == b.mn_major &&
           a.box_outer == b.box_outer;
}

template <int CAP>
cudaError_t launch_fused_cap(const FusedProblem* probs, const FusedOperand* a_ops, const FusedOperand* b_ops, int n,
                             int* err_word, size_t max_smem, int sm_count, int slot, cudaStream_t stream, int* used) {
    // takes as many problems from the front as fit the table (problems and distinct tensor maps)
    FusedTable<CAP> tab;
    constexpr int kMaps = (int)(sizeof(tab.maps) / sizeof(tab.maps[0]));
    FusedOperand seen[kMaps];
    int n_maps = 0, items = 0, taken = 0;
    for (; taken < n && taken < CAP; ++taken) {
        int idx[2];
        const FusedOperand* ops[2] = {&a_ops[taken], &b_ops[taken]};
        int added = 0;
        for (int o = 0; o < 2; ++o) {
            idx[o] = -1;
            for (int m = 0; m < n_maps + added; ++m)
                if (same_operand(seen[m], *ops[o])) { idx[o] = m; break; }
            if (idx[o] < 0) {
                if (n_maps + added >= kMaps) break;
                seen[n_maps + added] = *ops[o];
                idx[o] = n_maps + added;
                ++added;
            }
        }
        if (idx[0] < 0 || idx[1] < 0) break;
        for (int m = n_maps; m < n_maps + added; ++m)
            if (!tc_encode_map_f32(&tab.maps[m], seen[m].ptr, seen[m].cols, seen[m].rows, seen[m].ld, seen[m].mn_major,
                                   seen[m].box_outer))
                return cudaErrorInvalidValue;
        n_maps += added;
        FusedProblem& p = tab.p[taken];
        p = probs[taken];
        p.a_map = idx[0];
        p.b_map = idx[1];
        p.item_begin = items;
        items += p.tiles_m * p.tiles_n * p.splits;
    }
    if (taken == 0) return cudaErrorInvalidValue;
    tab.n_problems = taken;
    tab.n_items = items;
    tab.pad0 = tab.pad1 = 0;
    if (const char* dbg = getenv("MCL_FUSED_DBG")) sscanf(dbg, "%d,%d", &tab.pad0, &tab.pad1);
    const size_t smem = (size_t)kStages * kStage + 4 * 4096 + 1024;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(tc_fused_kernel<CAP>), slot, max_smem);
    if (e != cudaSuccess) return e;
    const int ctas = items < sm_count ? items : sm_count;
    tc_fused_kernel<CAP><<<ctas, kFThreads, smem, stream>>>(tab, err_word);
    *used = taken;
    return cudaGetLastError();
}

}  // namespace

size_t fused_plan(FusedProblem* p, int target_items, int depth_limit) {
    const int ktiles = (p->K + 31) / 32;
    p->tiles_m = (p->M + 127) / 128;
    if (p->mode != kFusedDW) {
        p->BN = pick_bn(p->N, p->mode == kFusedY ? 16 : 32, 256);
        p->tiles_n = (p->N + p->BN - 1) / p->BN;
        p->splits = 1;
        p->ktiles_per_split = ktiles;
        p->nprod = 2;
        p->prod = 0x01u;              // lo.b, then hi.b
        return 0;
    }
    p->BN = pick_bn(p->N, 32, 128);
    p->tiles_n = (p->N + p->BN - 1) / p->BN;
    p->nprod = 3;
    p->prod = 0x041u;                 // lo_a.hi_b, hi_a.lo_b, hi_a.hi_b
    const int tiles = p->tiles_m * p->tiles_n;
    int splits = (target_items + tiles - 1) / tiles;
    if (splits > ktiles / 8) splits = ktiles / 8;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    if (depth_limit > 0 && (ktiles + splits - 1) / splits > depth_limit) splits = (ktiles + depth_limit - 1) / depth_limit;
    p->ktiles_per_split = (ktiles + splits - 1) / splits;
    p->splits = (ktiles + p->ktiles_per_split - 1) / p->ktiles_per_split;
    return p->splits > 1 ? (size_t)p->splits * p->M * p->N : 0;
}

cudaError_t launch_tc_fused(const FusedProblem* probs, const FusedOperand* a_ops, const FusedOperand* b_ops, int n,
                            int* err_word, size_t max_smem, int sm_count, cudaStream_t stream, int* launches) {
    if ((size_t)kStages * kStage + 4 * 4096 + 1024 + 2048 > max_smem) return cudaErrorInvalidConfiguration;
    for (int i = 0; i < n; ++i) {
        const FusedProblem& p = probs[i];
        if (p.mode == kFusedDW ? (p.BN > 128 || (p.BN & 31)) : (p.BN > 256 || (p.BN & (p.mode == kFusedY ? 15 : 31))))
            return cudaErrorInvalidValue;
        if ((p.N & 3) || (p.ldc & 3) || (a_ops[i].ld & 3) || (b_ops[i].ld & 3)) return cudaErrorInvalidValue;
    }
    int done = 0;
    while (done < n) {
        int used = 0;
        const int left = n - done;
        cudaError_t e = left <= 3
            ? launch_fused_cap<3>(probs + done, a_ops + done, b_ops + done, left, err_word, max_smem, sm_count, 6, stream, &used)
            : launch_fused_cap<kFusedMaxProblems>(probs + done, a_ops + done, b_ops + done, left, err_word, max_smem,
                                                  sm_count, 7, stream, &used);
        if (e != cudaSuccess) return e;
        ++*launches;
        done += used;
    }
    return cudaSuccess;
}

cudaError_t launch_ternary_f32(const uint8_t* state, const uint32_t* packed2, int C, int O, int I, float* T, int sm_count,
                               cudaStream_t stream) {
    if (state != nullptr) {
        const long long groups = (long long)O * (I / 4);
        long long blocks = (groups + 255) / 256;
        if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
        ternary_f32_from_state_kernel<<<(int)blocks, 256, 0, stream>>>(state, C, groups, T);
    } else {
        const long long words = (long long)O * (I / 16);
        long long blocks = (words + 255) / 256;
        if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
        ternary_f32_from_p2_kernel<<<(int)blocks, 256, 0, stream>>>(packed2, words, T);
    }
    return cudaGetLastError();
}

#ifdef MCL_FUSED_PROF
extern "C" int mcl_debug_fused_prof(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_fused_prof, sizeof(long long) * 148 * 16);
}
#endif

}  // namespace mcl
