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
// so `hi` is the raw word and `lo` one elementwise pass over the tile.
// a.b is taken as lo.b + hi.b for an exact (ternary) b and as lo_a.hi_b + hi_a.lo_b + hi_a.hi_b for
// two fp32 operands; the dropped lo.lo and the rounding of lo are ~2^-22 relative.
//
// One launch runs a TABLE of problems (the three products of a step for many linears): work items
// (problem, 128-row tile, column tile, K slice) are drawn from a global counter by persistent CTAs.
//   MotifCL computes the same products with scalar fp32 FMAs: kernels/compact_counter.cl:37-65
//   (forward), :207-233 (backward to input), kernels/matmul.cl:413-563 (dW = dY^T X).
//
// Problem kinds (C[M,N] = A[M,K] . B[N,K]^T); every tensor is row-major fp32 behind a TMA map with
// 32-float-wide boxes (K-major use: 128-byte swizzle; MN-major use: 3-D map, 32-byte-atom swizzle):
//   kFusedY   A = X  [tokens,in]  K-major              B = T [out,in]  K-major   (exact)
//   kFusedDX  A = dY [tokens,out] K-major, x scale[k]  B = T [out,in]  MN-major  (exact)
//   kFusedDW  A = dY [tokens,out] MN-major             B = X [tokens,in] MN-major
//   kFusedYB / kFusedDXB  the two row products as tcgen05.mma.kind::f16: A split into two bf16 terms
//             (hi = bf16(a), lo = bf16(a - hi), two k per TMEM column), B = the ternary digits as a K-major
//             bf16 matrix (T [out,in] for Y, its transpose [in,out] for dX), k-tiles of 64: half the MMA
//             instructions and hand-offs per unit of work; 16 mantissa bits, relative L2 ~2.5e-6
// "MN-major" = the M (or N) index is the contiguous one in memory, the layout a transposed
// operand has; the tensor core reads it in place (instruction-descriptor transpose bits), so no
// transposed copy of an activation is ever made.
//
// CTA = 16 warps.  The A operand of every product is read from TENSOR MEMORY: two converter threads share one
// row of the A tile (= one TMEM lane), read half of its k each from the raw tile in shared memory and store the
// raw words (`hi`, scaled by scale[k] for dX) and the lo terms into 64 TMEM columns (tcgen05.st).  A
// transposed A (dW) is read column-wise from the MN-major boxes, so the transpose costs nothing.  Shared
// memory holds the RAW ring (2 to 6 slots: A and B as TMA delivers them; deep, because it has to cover
// the latency of HBM) and, for dW only, a ring of B lo tiles.  Three tiles are in flight between the
// converters and the MMA lane (three A slots in TMEM, three B lo slots).
//   warp 0        one lane draws work items from a global counter and issues the TMA copies
//   warp 1        allocates TMEM; one lane issues tcgen05.mma (A from TMEM, B from shared memory) and commits
//   warp 2        one lane asks the tiles of the next work item into L2 (TMA prefetch; off by default)
//   warps 4..7    epilogue: tcgen05.ld of TMEM lane quarter (warp & 3), scale, 128-bit stores
//   warps 8..15   converters: all eight work on every k-tile, half a row of the A tile per thread
// TMEM columns: two accumulators of at most 160 columns at 0 and 160 (the epilogue of one item overlaps the
// main loop of the next), A slots of 64 columns at 320, 384, 448.
// Every wait is bounded (see mbar_wait); on time-out the kernel records an error word and drains.
#include <cuda.h>
#include <cuda_bf16.h>
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
constexpr int kBox = 32 * 32 * 4;            // bytes of one 32 x 32 fp32 box
constexpr int kABytes = 4 * kBox;            // an A tile: 128 rows (or 128 m) x 32 k
constexpr int kMaxRaw = 6;                   // slots of the raw ring (A hi + B hi as TMA delivers them)
constexpr int kLoSlots = 3;                  // tiles between converters and MMA: A (hi, lo) in tensor memory, B lo (dW) in shared memory
constexpr int kQueue = 4;                    // work items in flight between the scheduler lane and the other roles
constexpr int kQueueReaders = 1 + 1 + 4 + 8; // MMA lane, prefetch lane, epilogue warps, converter warps
constexpr int kPrefetchAhead = 12;           // k-tiles the prefetch lane may run ahead of the copies
constexpr int kScratch = 4 * 2048;           // epilogue staging, 2 KiB per warp
constexpr int kAccStride = 160;              // TMEM columns between the two accumulators (an accumulator is at most 160 wide)
constexpr int kACol = 320;                   // the A tiles follow the accumulators: 64 columns each (hi, lo)

template <int CAP>
struct FusedTable {
    CUtensorMap maps[2 * CAP];
    int n_problems, n_items;
    int n_raw, raw_slot, lo_slot, pad0;      // ring geometry (bytes), chosen by the launcher for the table's tiles
    int prefetch, pad1, pad2, pad3;          // prefetch: the prefetch lane asks tiles into L2 ahead of the copies
    FusedProblem p[CAP];
};

// Instruction descriptor, kind::tf32: D = f32 (bits 4-5 = 1), A = B = tf32 (bits 7-9, 10-12 = 2),
// bit 15 / 16 = A / B is MN-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t idesc_tf32(int m, int n, bool a_mn, bool b_mn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Shared-memory layouts (B operand; the raw A tiles use the same ones).  K-major: rows of 128 bytes (32 fp32 of k) in the 128-byte swizzle, 8-row
// groups 1024 bytes apart (stride byte offset).  MN-major: rows of 128 bytes hold 32 consecutive m (or
// n) for one k, in the 128-byte swizzle with 32-byte atoms (the form the tensor core can transpose
// 32-bit data from): 4 k-rows per 512 bytes (stride byte offset), the next 32 m one box = 4096 bytes
// further (leading byte offset).
// tf32 MMA with the A operand in tensor memory: row m of the tile = TMEM lane m, one tf32 per 32-bit column
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_c, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_c), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accum) : "memory");
}
// kind::f16 (bf16 operands, two per 32-bit TMEM column for A), A in tensor memory
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_c, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_c), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accum) : "memory");
}
// Instruction descriptor, kind::f16: D = f32, A = B = bf16 (1 at bits 7 and 10), both K-major
__device__ __forceinline__ uint32_t idesc_bf16_k(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ bool is_bf16_mode(int mode) { return mode >= kFusedYB; }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

struct Item {
    int pi, mt, nt, kt0, nkt, split;
};

// item -> problem (items of a problem are contiguous; `pi` only moves forward).  `sp` is the CTA's copy of
// the problem table in shared memory: the roles walk it at every item, and the constant bank that holds
// the kernel argument is far too small a cache for it.
__device__ __forceinline__ Item decode_item(const FusedProblem* sp, int n_problems, int item, int& pi) {
    while (pi + 1 < n_problems && item >= sp[pi + 1].item_begin) ++pi;
    const FusedProblem& P = sp[pi];
    const int local = item - P.item_begin;
    Item it;
    it.pi = pi;
    // column tile fastest: the items that share an A slab run at the same time on neighbouring CTAs
    it.nt = local % P.tiles_n;
    const int rest = local / P.tiles_n;
    it.mt = rest % P.tiles_m;
    it.split = rest / P.tiles_m;
    const int ktiles = is_bf16_mode(P.mode) ? (P.K + 63) >> 6 : (P.K + 31) >> 5;
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



template <int CAP>
__global__ void __launch_bounds__(kFThreads, 1) tc_fused_kernel(const __grid_constant__ FusedTable<CAP> tab, int* err,
                                                                int* next_item) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kMaxRaw + 2 * kLoSlots + 4 + 2 * kQueue];
    __shared__ int queue_item[kQueue], queue_next[kQueue];
    __shared__ unsigned int tiles_issued;      // progress of the TMA lane, paces the prefetch lane
    __shared__ FusedProblem sp[CAP];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_raw = tab.n_raw;
    const uint32_t raw_slot = (uint32_t)tab.raw_slot, lo_slot = (uint32_t)tab.lo_slot;
    const uint32_t raw0 = (smem_u32(smem_raw) + 1023u) & ~1023u;        // raw ring: A hi at +0, B hi at +kABytes
    const uint32_t lo0 = raw0 + (uint32_t)n_raw * raw_slot;             // lo ring:  A lo at +0, B lo at +kABytes
    const uint32_t scratch0 = lo0 + (uint32_t)kLoSlots * lo_slot;       // 2 KiB per epilogue warp
    const uint32_t bar0 = smem_u32(bars);
    auto raw_full = [&](int s) { return bar0 + 8u * s; };
    auto raw_empty = [&](int s) { return bar0 + 8u * (kMaxRaw + s); };
    auto lo_full = [&](int s) { return bar0 + 8u * (2 * kMaxRaw + s); };
    auto lo_empty = [&](int s) { return bar0 + 8u * (2 * kMaxRaw + kLoSlots + s); };
    auto acc_full = [&](int a) { return bar0 + 8u * (2 * kMaxRaw + 2 * kLoSlots + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (2 * kMaxRaw + 2 * kLoSlots + 2 + a); };
    auto a_col = [](int sl) -> uint32_t { return (uint32_t)(kACol + 64 * sl); };   // TMEM columns of A slot sl
    auto q_full = [&](int s) { return bar0 + 8u * (2 * kMaxRaw + 2 * kLoSlots + 4 + s); };
    auto q_empty = [&](int s) { return bar0 + 8u * (2 * kMaxRaw + 2 * kLoSlots + 4 + kQueue + s); };

    if (threadIdx.x == 0) {
        abort_flag = (*reinterpret_cast<volatile int*>(err) != 0);
        tiles_issued = 0;
        for (int s = 0; s < kMaxRaw; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), 1); }
        for (int s = 0; s < kLoSlots; ++s) { mbar_init(lo_full(s), kConvThreads); mbar_init(lo_empty(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 128); }
        for (int s = 0; s < kQueue; ++s) { mbar_init(q_full(s), 1); mbar_init(q_empty(s), kQueueReaders); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int n_problems = tab.n_problems;
    {
        static_assert(sizeof(FusedProblem) % 4 == 0, "FusedProblem is copied word by word");
        const uint32_t* src = reinterpret_cast<const uint32_t*>(tab.p);
        uint32_t* dst = reinterpret_cast<uint32_t*>(sp);
        const int words = n_problems * (int)(sizeof(FusedProblem) / 4);
        for (int i = threadIdx.x; i < words; i += kFThreads) dst[i] = src[i];
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

    // Work items come from a global counter (long items first), so CTAs stay busy until the table is
    // empty.  The TMA lane draws them and passes every item number, the end marker included, to the
    // other roles through a small queue in shared memory.
    uint32_t q_seq = 0;
    auto next_from_queue = [&]() -> int {       // called by converged warps (or by the single MMA lane)
        const int s = (int)(q_seq % kQueue);
        int item = n_items;
        if (mbar_wait_warp(q_full(s), (q_seq / kQueue) & 1u, &abort_flag)) {
            item = *reinterpret_cast<volatile int*>(&queue_item[s]);
            __syncwarp();
            if (lane == 0) mbar_arrive(q_empty(s));
        } else {
            abort_flag = 1;
            atomicExch(err, 16);
        }
        ++q_seq;
        return item;
    };

    if (warp == 0) {
        if (lane == 0) {
            // ---- scheduler + TMA producer --------------------------------------------------------------
            uint32_t it = 0, rs = 0, rph = 0;          // tiles issued, raw slot, its phase parity
            int pi = 0;
            // two items are drawn ahead: the next one is published with the current one (the prefetch lane asks
            // its tiles into L2), the one after is still in flight from the counter
            int drawn = atomicAdd(next_item, 1);
            int drawn2 = atomicAdd(next_item, 1);
            for (;;) {
                const int item = abort_flag ? n_items : drawn;
                drawn = drawn2;
                if (item < n_items) drawn2 = atomicAdd(next_item, 1);
                {
                    const int s = (int)(q_seq % kQueue);
                    if (!mbar_wait(q_empty(s), ((q_seq / kQueue) & 1u) ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 17); break; }
                    *reinterpret_cast<volatile int*>(&queue_item[s]) = item < n_items ? item : n_items;
                    *reinterpret_cast<volatile int*>(&queue_next[s]) = drawn < n_items ? drawn : n_items;
                    mbar_arrive(q_full(s));
                    ++q_seq;
                }
                if (item >= n_items) break;
                const Item I = decode_item(sp, n_problems, item, pi);
                const FusedProblem& P = sp[I.pi];
                const CUtensorMap* ma = &tab.maps[P.a_map];
                const CUtensorMap* mb = &tab.maps[P.b_map];
                const int m0 = I.mt * 128, n0 = I.nt * P.BN, mode = P.mode;
                const uint32_t bytes = (uint32_t)kABytes + (uint32_t)P.BN * 128u;
                for (int j = 0; j < I.nkt; ++j, ++it) {
                    const int s = (int)rs;
                    const uint32_t ph = rph;
                    if (++rs == (uint32_t)n_raw) { rs = 0; rph ^= 1u; }
                    if (!mbar_wait(raw_empty(s), ph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 11); break; }
                    const uint32_t st = raw0 + (uint32_t)s * raw_slot;
                    const int k0 = (I.kt0 + j) * 32;
                    if (is_bf16_mode(mode)) {
                        // 64 k: two fp32 boxes of A side by side, one bf16 box of the ternary operand
                        mbar_expect_tx(raw_full(s), 2u * (uint32_t)kABytes + (uint32_t)P.BN * 128u);
                        const int kb = (I.kt0 + j) * 64;
                        tma_load_2d(st, ma, raw_full(s), kb, m0);
                        tma_load_2d(st + kABytes, ma, raw_full(s), kb + 32, m0);
                        tma_load_2d(st + 2 * kABytes, mb, raw_full(s), kb, n0);
                    } else {
                        mbar_expect_tx(raw_full(s), bytes);
                        // K-major: one box of 32 k x rows; MN-major: one box of 32 m x 32 k x chunks (3-D map)
                        if (mode == kFusedDW) tma_load_3d(st, ma, raw_full(s), 0, k0, m0 >> 5);
                        else tma_load_2d(st, ma, raw_full(s), k0, m0);
                        if (mode == kFusedY) tma_load_2d(st + kABytes, mb, raw_full(s), k0, n0);
                        else tma_load_3d(st + kABytes, mb, raw_full(s), 0, k0, n0 >> 5);
                    }
                    *reinterpret_cast<volatile unsigned int*>(&tiles_issued) = it + 1;
                }
                if (abort_flag) {      // tell the other roles to stop
                    const int s = (int)(q_seq % kQueue);
                    if (mbar_wait(q_empty(s), ((q_seq / kQueue) & 1u) ^ 1u, &abort_flag)) {
                        *reinterpret_cast<volatile int*>(&queue_item[s]) = n_items;
                        *reinterpret_cast<volatile int*>(&queue_next[s]) = n_items;
                        mbar_arrive(q_full(s));
                    }
                    break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ------------------------------------------------------------------------
            uint32_t it = 0, n_local = 0, rs = 0;
            int pi = 0;
            for (;;) {
                int item = n_items;
                {   // single-lane form of next_from_queue
                    const int s = (int)(q_seq % kQueue);
                    if (mbar_wait(q_full(s), (q_seq / kQueue) & 1u, &abort_flag)) {
                        item = *reinterpret_cast<volatile int*>(&queue_item[s]);
                        mbar_arrive(q_empty(s));
                    } else { abort_flag = 1; atomicExch(err, 16); }
                    ++q_seq;
                }
                if (item >= n_items || abort_flag) break;
                const Item I = decode_item(sp, n_problems, item, pi);
                const FusedProblem& P = sp[I.pi];
                const bool bf = is_bf16_mode(P.mode);
                const bool b_mn = P.mode != kFusedY;
                const uint32_t idesc = bf ? idesc_bf16_k(128, P.BN) : idesc_tf32(128, P.BN, false, b_mn);
                // B descriptor words: low = address / 16 | leading byte offset / 16 << 16, high = stride byte offset / 16 |
                // version bit | layout type << 29 (1 = 128-byte swizzle with 32-byte atoms, 2 = 128-byte swizzle)
                const uint32_t b_step = b_mn ? 64u : 2u;                                    // 16-byte units per 8 k
                const uint32_t b_lo = b_mn ? ((uint32_t)(kBox >> 4) << 16) : (1u << 16);
                const uint32_t b_hi = b_mn ? ((512u >> 4) | (1u << 14) | (1u << 29)) : ((1024u >> 4) | (1u << 14) | (2u << 29));
                const uint32_t nprod = (uint32_t)P.nprod, prod0 = P.prod;
                if (P.flush <= 0) {
                // ---- the whole item in one accumulator ----
                const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
                if (!mbar_wait(acc_empty(acc), aph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 14); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccStride;
                uint32_t accum = 0;
                for (int j = 0; j < I.nkt; ++j, ++it) {
                    const int s = (int)rs, sl = (int)(it % kLoSlots);
                    if (++rs == (uint32_t)n_raw) rs = 0;
                    const uint32_t hi16 = (raw0 + (uint32_t)s * raw_slot + (bf ? 2u : 1u) * (uint32_t)kABytes) >> 4;     // B as TMA delivered it
                    const uint32_t lo16 = (lo0 + (uint32_t)sl * lo_slot) >> 4;                          // B lo
                    const uint32_t a_tm = tmem_base + a_col(sl);                                        // A hi, A lo at +32
                    // the converters arrive after they have seen the raw tile, so this wait covers the copies as well
                    if (!mbar_wait(lo_full(sl), (it / kLoSlots) & 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 12); break; }
                    tc_fence_after();
                    uint32_t prod = prod0;
                    if (bf) {
                        // the ternary tile is K-major bf16 in the 128-byte swizzle (rows of 64 k); A terms: hi, lo
                        const uint64_t db0 = smem_desc_k_sw128(hi16 << 4);
#pragma unroll
                        for (uint32_t t = 0; t < 2; ++t)
#pragma unroll
                            for (uint32_t kk = 0; kk < 4; ++kk) {
                                umma_bf16_ts(d_tmem, a_tm + 32u * t + kk * 8u, db0 + 2u * kk, idesc, accum);
                                accum = 1u;
                            }
                    } else
                    for (uint32_t q = 0; q < nprod; ++q, prod >>= 4) {
                        const uint32_t a_t = a_tm + ((prod & 3u) ? 32u : 0u);
                        const uint32_t b16 = b_lo | (((prod >> 2) & 3u) ? lo16 : hi16);
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) {
                            const uint64_t db = ((uint64_t)b_hi << 32) | (uint64_t)(b16 + kk * b_step);
                            umma_tf32_ts(d_tmem, a_t + kk * 8u, db, idesc, accum);
                            accum = 1u;
                        }
                    }
                    umma_commit(raw_empty(s));
                    umma_commit(lo_empty(sl));
                }
                if (abort_flag) break;
                umma_commit(acc_full(acc));
                ++n_local;
                } else {
                // An accumulator takes at most P.flush k-tiles (tensor-core accumulation truncates, and the error grows
                // with the number of instructions that add into one accumulator): a long item hands its accumulator to
                // the epilogue every P.flush k-tiles and goes on in the other one; the epilogue adds the pieces in fp32.
                const int flush = P.flush > 0 ? P.flush : I.nkt;
                for (int j0 = 0; j0 < I.nkt && !abort_flag; j0 += flush, ++n_local) {
                const int j1 = min(I.nkt, j0 + flush);
                const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
                if (!mbar_wait(acc_empty(acc), aph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 14); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccStride;
                uint32_t accum = 0;
                for (int j = j0; j < j1; ++j, ++it) {
                    const int s = (int)rs, sl = (int)(it % kLoSlots);
                    if (++rs == (uint32_t)n_raw) rs = 0;
                    const uint32_t hi16 = (raw0 + (uint32_t)s * raw_slot + (bf ? 2u : 1u) * (uint32_t)kABytes) >> 4;     // B as TMA delivered it
                    const uint32_t lo16 = (lo0 + (uint32_t)sl * lo_slot) >> 4;                          // B lo
                    const uint32_t a_tm = tmem_base + a_col(sl);                                        // A hi, A lo at +32
                    // the converters arrive after they have seen the raw tile, so this wait covers the copies as well
                    if (!mbar_wait(lo_full(sl), (it / kLoSlots) & 1u, &abort_flag)) { abort_flag = 1; atomicExch(err, 12); break; }
                    tc_fence_after();
                    uint32_t prod = prod0;
                    if (bf) {
                        // the ternary tile is K-major bf16 in the 128-byte swizzle (rows of 64 k); A terms: hi, lo
                        const uint64_t db0 = smem_desc_k_sw128(hi16 << 4);
#pragma unroll
                        for (uint32_t t = 0; t < 2; ++t)
#pragma unroll
                            for (uint32_t kk = 0; kk < 4; ++kk) {
                                umma_bf16_ts(d_tmem, a_tm + 32u * t + kk * 8u, db0 + 2u * kk, idesc, accum);
                                accum = 1u;
                            }
                    } else
                    for (uint32_t q = 0; q < nprod; ++q, prod >>= 4) {
                        const uint32_t a_t = a_tm + ((prod & 3u) ? 32u : 0u);
                        const uint32_t b16 = b_lo | (((prod >> 2) & 3u) ? lo16 : hi16);
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) {
                            const uint64_t db = ((uint64_t)b_hi << 32) | (uint64_t)(b16 + kk * b_step);
                            umma_tf32_ts(d_tmem, a_t + kk * 8u, db, idesc, accum);
                            accum = 1u;
                        }
                    }
                    umma_commit(raw_empty(s));
                    umma_commit(lo_empty(sl));
                }
                if (abort_flag) break;
                umma_commit(acc_full(acc));
                }
                }
                if (abort_flag) break;
            }
        }
    } else if (warp == 2) {
        if (lane == 0) {
            // ---- prefetch lane: asks the tiles of the NEXT item into L2 ------------------------------------
            // HBM is ~1.5 us away and the raw ring holds four tiles; a copy whose tile is already in L2 completes
            // in a third of the time.  The lane stays at most kPrefetchAhead tiles ahead of the copies.
            int pi = 0;
            unsigned int pos = 0;      // tiles of the items published so far
            for (;;) {
                int item = n_items, nxt = n_items;
                {
                    const int s = (int)(q_seq % kQueue);
                    if (mbar_wait(q_full(s), (q_seq / kQueue) & 1u, &abort_flag)) {
                        item = *reinterpret_cast<volatile int*>(&queue_item[s]);
                        nxt = *reinterpret_cast<volatile int*>(&queue_next[s]);
                        mbar_arrive(q_empty(s));
                    }
                    ++q_seq;
                }
                if (item >= n_items || abort_flag) break;
                int pc = pi;
                const Item I = decode_item(sp, n_problems, item, pc);
                pi = pc;
                pos += (unsigned int)I.nkt;
                if (nxt >= n_items || !tab.prefetch) continue;
                int pn = pi;
                const Item J = decode_item(sp, n_problems, nxt, pn);
                const FusedProblem& Q = sp[J.pi];
                const CUtensorMap* qa = &tab.maps[Q.a_map];
                const CUtensorMap* qb = &tab.maps[Q.b_map];
                const int qm = J.mt * 128, qn = J.nt * Q.BN, qmode = Q.mode;
                for (int t = 0; t < J.nkt && !abort_flag; ++t) {
                    // tile t of the next item is stream position pos + t
                    while ((int)(pos + (unsigned int)t - *reinterpret_cast<volatile unsigned int*>(&tiles_issued)) > kPrefetchAhead &&
                           !abort_flag)
                        __nanosleep(100);
                    const int k = (J.kt0 + t) * (is_bf16_mode(qmode) ? 64 : 32);
                    if (qmode == kFusedDW) {
                        tma_prefetch_3d(qa, 0, k, qm >> 5);
                        tma_prefetch_3d(qb, 0, k, qn >> 5);
                    } else {
                        tma_prefetch_2d(qa, k, qm);      // the ternary operand is small and stays in L2 by itself
                        if (is_bf16_mode(qmode)) tma_prefetch_2d(qa, k + 32, qm);
                    }
                }
            }
        }
    } else if (warp >= kEpiWarp0 && warp < kConvWarp0) {
        // ---- epilogue warps ----------------------------------------------------------------------------
        const int q = warp & 3;
        uint32_t n_local = 0;
        int pi = 0;
        bool alive = true;
        while (alive) {
            const int item = next_from_queue();
            if (item >= n_items) break;
            const Item I = decode_item(sp, n_problems, item, pi);
            const FusedProblem& P = sp[I.pi];
            if (P.flush <= 0) {
            // ---- the whole item is one accumulator: scale and store ----
            do {
            const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
            bool ok = !abort_flag;
            if (ok && !mbar_wait_warp(acc_full(acc), aph, &abort_flag)) { abort_flag = 1; atomicExch(err, 13); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            tc_fence_after();
            const bool scale = (P.col_scale != nullptr) && P.splits == 1;
            const int BN = P.BN, n0 = I.nt * BN;
            const int row0 = I.mt * 128 + q * 32;
            float* cbase = P.C + ((size_t)I.split * P.M + row0) * P.ldc;
            // The TMEM fragment (lane = row, 16 columns) goes through a swizzled 2 KiB tile of shared memory so
            // that a store instruction writes 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes.
            const uint32_t scratch = scratch0 + (uint32_t)q * 2048u;
            const int rsub = lane >> 2, j4 = lane & 3;
            {
                // software pipeline: the TMEM load of the next chunk and the scale of this one are in flight while
                // the current chunk goes through shared memory to global memory
                const uint32_t t0addr = tmem_base + acc * kAccStride + ((uint32_t)(q * 32) << 16);
                uint32_t r[16];
                int nchunks = 0;
                for (int c0 = 0; c0 < BN && n0 + c0 < P.N; c0 += 16) ++nchunks;
                if (nchunks > 0) tmem_ld16(t0addr, r);
                for (int ci = 0; ci < nchunks; ++ci) {
                    const int c0 = ci * 16;
                    const int col = n0 + c0 + 4 * j4;
                    const bool col_ok = col < P.N;
                    float4 sc = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (scale && col_ok) sc = __ldg(reinterpret_cast<const float4*>(P.col_scale + col));
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        sts128(scratch + (uint32_t)lane * 64u + ((uint32_t)(j ^ ((lane >> 1) & 3)) << 4),
                               make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                           __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                    __syncwarp();
                    if (ci + 1 < nchunks) tmem_ld16(t0addr + (uint32_t)(c0 + 16), r);
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const int rr = p * 8 + rsub;
                        float4 o = lds128(scratch + (uint32_t)rr * 64u + ((uint32_t)(j4 ^ ((rr >> 1) & 3)) << 4));
                        if (col_ok && row0 + rr < P.M) {
                            o.x *= sc.x; o.y *= sc.y; o.z *= sc.z; o.w *= sc.w;
                            *reinterpret_cast<float4*>(cbase + (size_t)rr * P.ldc + col) = o;
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty(acc));
            ++n_local;
            } while (false);
            } else {
            const int flush = P.flush > 0 ? P.flush : I.nkt;
            const int npieces = (I.nkt + flush - 1) / flush;
            for (int piece = 0; piece < npieces; ++piece, ++n_local) {
            const bool add_prev = piece > 0;       // later pieces of an item are added to what this thread stored before
            const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
            bool ok = !abort_flag;
            if (ok && !mbar_wait_warp(acc_full(acc), aph, &abort_flag)) { abort_flag = 1; atomicExch(err, 13); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { alive = false; break; }
            tc_fence_after();
            const bool scale = (P.col_scale != nullptr) && P.splits == 1;
            const int BN = P.BN, n0 = I.nt * BN;
            const int row0 = I.mt * 128 + q * 32;
            float* cbase = P.C + ((size_t)I.split * P.M + row0) * P.ldc;
            // The TMEM fragment (lane = row, 16 columns) goes through a swizzled 2 KiB tile of shared memory so
            // that a store instruction writes 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes.
            const uint32_t scratch = scratch0 + (uint32_t)q * 2048u;
            const int rsub = lane >> 2, j4 = lane & 3;
            {
                // software pipeline: the TMEM load of the next chunk and the scale of this one are in flight while
                // the current chunk goes through shared memory to global memory
                const uint32_t t0addr = tmem_base + acc * kAccStride + ((uint32_t)(q * 32) << 16);
                uint32_t r[16];
                int nchunks = 0;
                for (int c0 = 0; c0 < BN && n0 + c0 < P.N; c0 += 16) ++nchunks;
                if (nchunks > 0) tmem_ld16(t0addr, r);
                if (!add_prev) {
                    // the first (usually only) piece of an item: scale and store
                    for (int ci = 0; ci < nchunks; ++ci) {
                        const int c0 = ci * 16;
                        const int col = n0 + c0 + 4 * j4;
                        const bool col_ok = col < P.N;
                        float4 sc = make_float4(1.f, 1.f, 1.f, 1.f);
                        if (scale && col_ok) sc = __ldg(reinterpret_cast<const float4*>(P.col_scale + col));
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            sts128(scratch + (uint32_t)lane * 64u + ((uint32_t)(j ^ ((lane >> 1) & 3)) << 4),
                                   make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                        __syncwarp();
                        if (ci + 1 < nchunks) tmem_ld16(t0addr + (uint32_t)(c0 + 16), r);
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const int rr = p * 8 + rsub;
                            float4 o = lds128(scratch + (uint32_t)rr * 64u + ((uint32_t)(j4 ^ ((rr >> 1) & 3)) << 4));
                            if (col_ok && row0 + rr < P.M) {
                                o.x *= sc.x; o.y *= sc.y; o.z *= sc.z; o.w *= sc.w;
                                *reinterpret_cast<float4*>(cbase + (size_t)rr * P.ldc + col) = o;
                            }
                        }
                        __syncwarp();
                    }
                } else {
                    // a later piece: add to what this thread stored for the earlier ones (fetched one chunk ahead: an L2
                    // round trip); only unscaled outputs are cut into pieces
                    float4 prev[4], prev_next[4];
                    auto load_prev = [&](int ci, float4 (&dst)[4]) {
                        const int col = n0 + ci * 16 + 4 * j4;
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const int rr = p * 8 + rsub;
                            dst[p] = (col < P.N && row0 + rr < P.M) ? *reinterpret_cast<const float4*>(cbase + (size_t)rr * P.ldc + col)
                                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    };
                    if (nchunks > 0) load_prev(0, prev_next);
                    for (int ci = 0; ci < nchunks; ++ci) {
                        const int c0 = ci * 16;
                        const int col = n0 + c0 + 4 * j4;
                        const bool col_ok = col < P.N;
#pragma unroll
                        for (int p = 0; p < 4; ++p) prev[p] = prev_next[p];
                        if (ci + 1 < nchunks) load_prev(ci + 1, prev_next);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            sts128(scratch + (uint32_t)lane * 64u + ((uint32_t)(j ^ ((lane >> 1) & 3)) << 4),
                                   make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                        __syncwarp();
                        if (ci + 1 < nchunks) tmem_ld16(t0addr + (uint32_t)(c0 + 16), r);
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const int rr = p * 8 + rsub;
                            float4 o = lds128(scratch + (uint32_t)rr * 64u + ((uint32_t)(j4 ^ ((rr >> 1) & 3)) << 4));
                            if (col_ok && row0 + rr < P.M) {
                                o.x = __fadd_rn(prev[p].x, o.x); o.y = __fadd_rn(prev[p].y, o.y);
                                o.z = __fadd_rn(prev[p].z, o.z); o.w = __fadd_rn(prev[p].w, o.w);
                                *reinterpret_cast<float4*>(cbase + (size_t)rr * P.ldc + col) = o;
                            }
                        }
                        __syncwarp();
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty(acc));
            }
                    }
        }
    } else if (warp >= kConvWarp0) {
        // ---- converters --------------------------------------------------------------------------------
        // All eight warps work on every k-tile: a thread owns HALF a row of the A tile (its TMEM lane = the row, so
        // the two warps of a lane quarter share each row): it reads 16 k (32 k of one fp32 box for the bf16 kinds) of
        // that row from the raw tile and stores them (`hi`: the raw words, scaled for dX) and their lo terms into its
        // 16 + 16 of the slot's 64 TMEM columns.  A transposed A (dW) is read column-wise from the MN-major boxes, which
        // is the transpose the tensor core would otherwise have to make.  The B lo tile of dW stays in shared memory.
        const int half = (warp - kConvWarp0) >> 2;                           // which half of the row's k
        const int tg = (int)threadIdx.x - kConvWarp0 * 32;                   // 0..255 among the converters
        const int q = warp & 3, row = q * 32 + lane;
        uint32_t it = 0, rs = 0, rph = 0;
        int pi = 0;
        for (;;) {
            const int item = next_from_queue();
            if (item >= n_items || abort_flag) break;
            const Item I = decode_item(sp, n_problems, item, pi);
            const FusedProblem& P = sp[I.pi];
            const bool a_mn = P.mode == kFusedDW;
            const int nb_lo = a_mn ? P.BN * 8 : 0;                      // 16-byte chunks of B that need a lo part
            const float* ksc = P.a_kscale;
            const int K = P.K;
            bool ok = true;
            for (int j = 0; j < I.nkt; ++j, ++it) {
                const int s = (int)rs;
                const uint32_t ph = rph;
                if (++rs == (uint32_t)n_raw) { rs = 0; rph ^= 1u; }
                const int sl = (int)(it % kLoSlots);
                const uint32_t a_taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a_col(sl) + 16u * (uint32_t)half;
                // the slot first: once its last reader (tile it - 3) is done, every earlier tile is
                ok = mbar_wait_warp(lo_empty(sl), ((it / kLoSlots) & 1u) ^ 1u, &abort_flag) &&
                     mbar_wait_warp(raw_full(s), ph, &abort_flag);
                if (!ok) break;
                tc_fence_after();          // the MMAs that read this TMEM slot have completed
                const int k0 = (I.kt0 + j) * 32;
                const uint32_t st = raw0 + (uint32_t)s * raw_slot, sto = lo0 + (uint32_t)sl * lo_slot;
                uint32_t hi[16], lo[16];
                if (is_bf16_mode(P.mode)) {
                    // 64 k of the row lie in two boxes; this thread takes box `half`: 32 k -> two bf16 terms, two k per
                    // TMEM column (even k in the low half)
                    const int kb = (I.kt0 + j) * 64 + 32 * half;
                    const uint32_t ra = st + (uint32_t)half * (uint32_t)kABytes + (uint32_t)row * 128u;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        float4 v = lds128(ra + ((uint32_t)(c ^ (row & 7)) << 4));
                        if (ksc != nullptr) {
                            const int k = kb + 4 * c;
                            if (k < K) {
                                const float4 sc = __ldg(reinterpret_cast<const float4*>(ksc + k));
                                v.x = __fmul_rn(v.x, sc.x); v.y = __fmul_rn(v.y, sc.y);
                                v.z = __fmul_rn(v.z, sc.z); v.w = __fmul_rn(v.w, sc.w);
                            }
                        }
                        const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
                        const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - __low2float(h0), v.y - __high2float(h0));
                        const __nv_bfloat162 l1 = __floats2bfloat162_rn(v.z - __low2float(h1), v.w - __high2float(h1));
                        hi[2 * c] = *reinterpret_cast<const uint32_t*>(&h0);
                        hi[2 * c + 1] = *reinterpret_cast<const uint32_t*>(&h1);
                        lo[2 * c] = *reinterpret_cast<const uint32_t*>(&l0);
                        lo[2 * c + 1] = *reinterpret_cast<const uint32_t*>(&l1);
                    }
                } else if (!a_mn) {
                    // K-major: row `row` is 128 bytes, its 16-byte chunks XOR-swizzled by the row number; this thread
                    // takes chunks 4 half .. 4 half + 3 (16 k)
                    const uint32_t ra = st + (uint32_t)row * 128u;
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const int c = 4 * half + cc;
                        float4 v = lds128(ra + ((uint32_t)(c ^ (row & 7)) << 4));
                        if (ksc != nullptr) {
                            const int k = k0 + 4 * c;
                            if (k < K) {
                                const float4 sc = __ldg(reinterpret_cast<const float4*>(ksc + k));
                                v.x = __fmul_rn(v.x, sc.x); v.y = __fmul_rn(v.y, sc.y);
                                v.z = __fmul_rn(v.z, sc.z); v.w = __fmul_rn(v.w, sc.w);
                            }
                        }
                        const float4 l = lo_term4(v);
                        hi[4 * cc] = __float_as_uint(v.x); hi[4 * cc + 1] = __float_as_uint(v.y);
                        hi[4 * cc + 2] = __float_as_uint(v.z); hi[4 * cc + 3] = __float_as_uint(v.w);
                        lo[4 * cc] = __float_as_uint(l.x); lo[4 * cc + 1] = __float_as_uint(l.y);
                        lo[4 * cc + 2] = __float_as_uint(l.z); lo[4 * cc + 3] = __float_as_uint(l.w);
                    }
                } else {
                    // MN-major: box q holds this lane quarter's 32 rows; k-row kk is 128 bytes whose 32-byte atoms are
                    // XOR-swizzled by kk & 3.  The 32 lanes of a warp read one whole k-row per instruction; this warp
                    // takes k-rows 16 half .. 16 half + 15.
                    const uint32_t ba = st + (uint32_t)q * (uint32_t)kBox + ((uint32_t)(lane & 7) << 2);
#pragma unroll
                    for (int kc = 0; kc < 16; ++kc) {
                        const int kk = 16 * half + kc;
                        const uint32_t w = lds32(ba + (uint32_t)kk * 128u + ((uint32_t)((lane >> 3) ^ (kk & 3)) << 5));
                        hi[kc] = w;
                        lo[kc] = __float_as_uint(lo_term(__uint_as_float(w)));
                    }
                }
                tmem_st16(a_taddr, hi);
                tmem_st16(a_taddr + 32u, lo);
                for (int c = tg; c < nb_lo; c += kConvThreads) {
                    const uint32_t off = (uint32_t)c * 16u;
                    sts128(sto + off, lo_term4(lds128(st + (uint32_t)kABytes + off)));
                }
                if (nb_lo) fence_proxy_async();
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(lo_full(sl));
            }
            if (!ok) { abort_flag = 1; atomicExch(err, 15); break; }
        }
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
constexpr int kTernCap = 64;
struct TernaryGroup {
    int n, C;
    long long unit_begin[kTernCap + 1];        // units of 4 weights (one float4 of T)
    const uint8_t* state[kTernCap];            // 6-bit state of layer j, or null: then
    const uint32_t* packed2[kTernCap];         // its 2-bit words
    float* T[kTernCap];
};
__global__ void __launch_bounds__(256) ternary_f32_group_kernel(const __grid_constant__ TernaryGroup g) {
    __shared__ DecodeLut lut;
    build_decode_lut(&lut, g.C, threadIdx.x, blockDim.x);
    __syncthreads();
    const long long total = g.unit_begin[g.n];
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
        int lo = 0, hi = g.n - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (g.unit_begin[mid] <= u) lo = mid; else hi = mid - 1;
        }
        const long long q = u - g.unit_begin[lo];
        float4 t;
        if (g.state[lo] != nullptr) {
            const uint8_t* s = g.state[lo] + q * 3;
            const uint32_t w = (uint32_t)__ldg(s) | ((uint32_t)__ldg(s + 1) << 8) | ((uint32_t)__ldg(s + 2) << 16);
            t = make_float4(lut.e[w & 63u].x, lut.e[(w >> 6) & 63u].x, lut.e[(w >> 12) & 63u].x, lut.e[(w >> 18) & 63u].x);
        } else {
            const uint32_t b = __ldg(g.packed2[lo] + (q >> 2)) >> (8 * (int)(q & 3));
            t = make_float4((float)((int)(b & 3u) - 1), (float)((int)((b >> 2) & 3u) - 1), (float)((int)((b >> 4) & 3u) - 1),
                            (float)((int)((b >> 6) & 3u) - 1));
        }
        reinterpret_cast<float4*>(g.T[lo])[q] = t;
    }
}

// ---- ternary digits of several layers as bf16, both orientations --------------------------------------------
// T [O][I] (the K-major operand of Y) and Tt [I][O] (the K-major operand of dX), 64 x 64 tiles through shared memory
struct TernaryBf16Group {
    int n, C;
    int tile_begin[kTernCap + 1];
    int O[kTernCap], I[kTernCap];
    const uint8_t* state[kTernCap];            // 6-bit state of layer j, or null: then
    const uint32_t* packed2[kTernCap];         // its 2-bit words
    __nv_bfloat16* T[kTernCap];
    __nv_bfloat16* Tt[kTernCap];
};
__global__ void __launch_bounds__(256) ternary_bf16_group_kernel(const __grid_constant__ TernaryBf16Group g) {
    __shared__ DecodeLut lut;
    __shared__ __nv_bfloat16 tile[64][66];
    build_decode_lut(&lut, g.C, threadIdx.x, blockDim.x);
    __syncthreads();
    const int total = g.tile_begin[g.n];
    for (int u = blockIdx.x; u < total; u += gridDim.x) {
        int lo = 0, hi = g.n - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (g.tile_begin[mid] <= u) lo = mid; else hi = mid - 1;
        }
        const int O = g.O[lo], I = g.I[lo], tiles_i = (I + 63) >> 6;
        const int local = u - g.tile_begin[lo];
        const int o0 = (local / tiles_i) * 64, i0 = (local % tiles_i) * 64;
        const uint8_t* state = g.state[lo];
        const uint32_t* p2 = g.packed2[lo];
        __nv_bfloat16* T = g.T[lo];
        __nv_bfloat16* Tt = g.Tt[lo];
        // 64 rows x 16 groups of 4 weights per tile
        for (int e = threadIdx.x; e < 64 * 16; e += 256) {
            const int oo = e >> 4, gi = e & 15, o = o0 + oo, i = i0 + 4 * gi;
            if (o < O && i < I) {
                float t[4];
                if (state != nullptr) {
                    const uint8_t* sp = state + ((size_t)o * (I >> 2) + (i >> 2)) * 3;
                    const uint32_t w = (uint32_t)__ldg(sp) | ((uint32_t)__ldg(sp + 1) << 8) | ((uint32_t)__ldg(sp + 2) << 16);
#pragma unroll
                    for (int k = 0; k < 4; ++k) t[k] = lut.e[(w >> (6 * k)) & 63u].x;
                } else {
                    const uint32_t b = __ldg(p2 + (size_t)o * (I >> 4) + (i >> 4)) >> (2 * (i & 15));
#pragma unroll
                    for (int k = 0; k < 4; ++k) t[k] = (float)((int)((b >> (2 * k)) & 3u) - 1);
                }
                const __nv_bfloat162 t01 = __floats2bfloat162_rn(t[0], t[1]), t23 = __floats2bfloat162_rn(t[2], t[3]);
                tile[oo][4 * gi] = __low2bfloat16(t01); tile[oo][4 * gi + 1] = __high2bfloat16(t01);
                tile[oo][4 * gi + 2] = __low2bfloat16(t23); tile[oo][4 * gi + 3] = __high2bfloat16(t23);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&t01); pk.y = *reinterpret_cast<const uint32_t*>(&t23);
                *reinterpret_cast<uint2*>(T + (size_t)o * I + i) = pk;
            }
        }
        __syncthreads();
        // transposed: thread -> (row i of Tt, two consecutive o)
        for (int e = threadIdx.x; e < 64 * 32; e += 256) {
            const int ii = e >> 5, op = (e & 31) * 2, i = i0 + ii, o = o0 + op;
            if (i < I && o < O) {       // O is even
                __nv_bfloat162 v;
                v.x = tile[op][ii]; v.y = tile[op + 1][ii];
                *reinterpret_cast<__nv_bfloat162*>(Tt + (size_t)i * O + o) = v;
            }
        }
        __syncthreads();
    }
}

// ---- the split-K reduction of several layers in one launch ----------------------------------------------------
constexpr int kGroupCap = 64;
struct ReduceGroup {
    int n;
    long long unit_begin[kGroupCap + 1];       // units of one float4 of the result
    const float* partial[kGroupCap];
    float* out[kGroupCap];
    int splits[kGroupCap];
};
__device__ __forceinline__ int find_group(const long long* begin, int n, long long u) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (begin[mid] <= u) lo = mid; else hi = mid - 1;
    }
    return lo;
}
// out = sum over z (ascending: deterministic) of partial[z]; all tensors dense [rows * cols]
__global__ void __launch_bounds__(256) splitk_reduce_group_kernel(const __grid_constant__ ReduceGroup g) {
    const long long total = g.unit_begin[g.n];
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
        const int j = find_group(g.unit_begin, g.n, u);
        const long long q = u - g.unit_begin[j], n4 = g.unit_begin[j + 1] - g.unit_begin[j];
        const float4* src = reinterpret_cast<const float4*>(g.partial[j]) + q;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < g.splits[j]; ++z) {
            const float4 v = __ldg(src + (long long)z * n4);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(g.out[j])[q] = acc;
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
           a.box_outer == b.box_outer && a.bf16 == b.bf16;
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
            if (!(seen[m].bf16 ? tc_encode_map_bf16(&tab.maps[m], seen[m].ptr, seen[m].cols, seen[m].rows, seen[m].ld, seen[m].box_outer)
                               : tc_encode_map_f32(&tab.maps[m], seen[m].ptr, seen[m].cols, seen[m].rows, seen[m].ld, seen[m].mn_major,
                                                   seen[m].box_outer)))
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
    // ring geometry: a raw slot holds the A tile and the widest B tile of the table, a lo slot the A lo
    // tile and the widest B tile that needs a lo part
    int bhi = 0, blo = 0;
    for (int i = 0; i < taken; ++i) {
        const int bytes = tab.p[i].BN * 128;
        const int raw = bytes + (tab.p[i].mode >= kFusedYB ? kABytes : 0);    // bf16 kinds: a second fp32 box of A
        if (raw > bhi) bhi = raw;
        if (tab.p[i].mode == kFusedDW && bytes > blo) blo = bytes;      // only two fp32 operands need a B lo tile
    }
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, reinterpret_cast<const void*>(tc_fused_kernel<CAP>));
    if (e != cudaSuccess) return e;
    tab.raw_slot = kABytes + ((bhi + 1023) & ~1023);
    tab.lo_slot = (blo + 1023) & ~1023;
    tab.pad0 = 0;
    tab.prefetch = 0;       // asking the next item's tiles into L2 ahead of the copies measured no gain
    const long long budget = (long long)max_smem - (long long)fa.sharedSizeBytes - 1024 - kScratch - kLoSlots * (long long)tab.lo_slot;
    int n_raw = (int)(budget / tab.raw_slot);
    if (n_raw > kMaxRaw) n_raw = kMaxRaw;
    if (n_raw < 2) return cudaErrorInvalidConfiguration;
    tab.n_raw = n_raw;
    const size_t smem = (size_t)n_raw * tab.raw_slot + (size_t)kLoSlots * tab.lo_slot + kScratch + 1024;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(tc_fused_kernel<CAP>), slot, max_smem);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(err_word + 1, 0, sizeof(int), stream);          // the work-item counter
    if (e != cudaSuccess) return e;
    const int ctas = items < sm_count ? items : sm_count;
    tc_fused_kernel<CAP><<<ctas, kFThreads, smem, stream>>>(tab, err_word, err_word + 1);
    *used = taken;
    return cudaGetLastError();
}

}  // namespace

size_t fused_plan(FusedProblem* p, int target_items, int depth_limit) {
    const int ktiles = (p->K + 31) / 32;
    p->tiles_m = (p->M + 127) / 128;
    if (p->mode >= kFusedYB) {
        p->BN = pick_bn(p->N, 16, 160);
        p->tiles_n = (p->N + p->BN - 1) / p->BN;
        p->splits = 1;
        p->ktiles_per_split = (p->K + 63) / 64;
        p->nprod = 2;
        p->prod = 0x10u;
        return 0;
    }
    if (p->mode != kFusedDW) {
        // B tiles of at most 20 KiB keep the raw ring four slots deep; wider tiles (three slots) measured 1.4x slower
        p->BN = pick_bn(p->N, p->mode == kFusedY ? 16 : 32, 160);
        p->tiles_n = (p->N + p->BN - 1) / p->BN;
        p->splits = 1;
        p->ktiles_per_split = ktiles;
        p->nprod = 2;
        p->prod = 0x10u;              // hi.b, then lo.b
        return 0;
    }
    // 160-wide column tiles: an MMA instruction costs about 100 cycles whatever its width (operand feed), so fewer and
    // wider instructions win (96-wide tiles measured 1.14x slower per step)
    p->BN = pick_bn(p->N, 32, 160);
    p->tiles_n = (p->N + p->BN - 1) / p->BN;
    p->nprod = 3;
    p->prod = 0x410u;                 // hi_a.hi_b, then lo_a.hi_b, hi_a.lo_b
    const int tiles = p->tiles_m * p->tiles_n;
    int splits = (target_items + tiles - 1) / tiles;
    if (splits > ktiles / 8) splits = ktiles / 8;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    if (depth_limit > 0 && (ktiles + splits - 1) / splits > depth_limit) splits = (ktiles + depth_limit - 1) / depth_limit;
    p->ktiles_per_split = (ktiles + splits - 1) / splits;
    p->splits = (ktiles + p->ktiles_per_split - 1) / p->ktiles_per_split;
    p->flush = kFusedFlushKtiles;
    return p->splits > 1 ? (size_t)p->splits * p->M * p->N : 0;
}

cudaError_t launch_tc_fused(const FusedProblem* probs, const FusedOperand* a_ops, const FusedOperand* b_ops, int n,
                            int* err_word, size_t max_smem, int sm_count, cudaStream_t stream, int* launches) {
    for (int i = 0; i < n; ++i) {
        const FusedProblem& p = probs[i];
        if (p.mode == kFusedDW ? (p.BN > 160 || (p.BN & 31)) : (p.BN > 160 || (p.BN & (p.mode == kFusedDX ? 31 : 15))))
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


cudaError_t launch_ternary_f32_group(const uint8_t* const* state, const uint32_t* const* packed2, float* const* T, const int* O, const int* I, int n, int C,
                                     int sm_count, cudaStream_t stream, int* launches) {
    for (int done = 0; done < n;) {
        TernaryGroup g;
        const int take = n - done < kTernCap ? n - done : kTernCap;
        long long units = 0;
        for (int j = 0; j < take; ++j) {
            g.unit_begin[j] = units;
            g.state[j] = state[done + j];
            g.packed2[j] = packed2[done + j];
            g.T[j] = T[done + j];
            units += (long long)O[done + j] * (I[done + j] / 4);
        }
        g.unit_begin[take] = units;
        g.n = take; g.C = C;
        long long blocks = (units + 255) / 256;
        if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
        ternary_f32_group_kernel<<<(int)blocks, 256, 0, stream>>>(g);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        ++*launches;
        done += take;
    }
    return cudaSuccess;
}

cudaError_t launch_ternary_bf16_group(const uint8_t* const* state, const uint32_t* const* packed2, void* const* T, void* const* Tt,
                                      const int* O, const int* I, int n, int C, int sm_count, cudaStream_t stream, int* launches) {
    for (int done = 0; done < n;) {
        TernaryBf16Group g;
        const int take = n - done < kTernCap ? n - done : kTernCap;
        int tiles = 0;
        for (int j = 0; j < take; ++j) {
            g.tile_begin[j] = tiles;
            g.state[j] = state[done + j];
            g.packed2[j] = packed2[done + j];
            g.T[j] = static_cast<__nv_bfloat16*>(T[done + j]);
            g.Tt[j] = static_cast<__nv_bfloat16*>(Tt[done + j]);
            g.O[j] = O[done + j]; g.I[j] = I[done + j];
            tiles += ((O[done + j] + 63) / 64) * ((I[done + j] + 63) / 64);
        }
        g.tile_begin[take] = tiles;
        g.n = take; g.C = C;
        const int blocks = tiles < sm_count * 8 ? tiles : sm_count * 8;
        ternary_bf16_group_kernel<<<blocks, 256, 0, stream>>>(g);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        ++*launches;
        done += take;
    }
    return cudaSuccess;
}

cudaError_t launch_splitk_reduce_group(const float* const* partial, float* const* out, const int* elements, const int* splits,
                                       int n, int sm_count, cudaStream_t stream, int* launches) {
    for (int done = 0; done < n;) {
        ReduceGroup g;
        const int take = n - done < kGroupCap ? n - done : kGroupCap;
        long long units = 0;
        for (int j = 0; j < take; ++j) {
            g.unit_begin[j] = units;
            g.partial[j] = partial[done + j];
            g.out[j] = out[done + j];
            g.splits[j] = splits[done + j];
            units += elements[done + j] / 4;
        }
        g.unit_begin[take] = units;
        g.n = take;
        long long blocks = (units + 255) / 256;
        if (blocks > (long long)sm_count * 8) blocks = (long long)sm_count * 8;
        splitk_reduce_group_kernel<<<(int)blocks, 256, 0, stream>>>(g);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        ++*launches;
        done += take;
    }
    return cudaSuccess;
}


}  // namespace mcl
