// Ternary decode GEMV on tensor cores (sm_100a): y[m,o] = scale[o] * sum_k x[m,k] * t[o,k],
// M <= 16, with t read from the 2-bit packed weights.  HBM-bound on out*in/4 bytes of weights.
//
// CUDA cores cannot keep up with 4 weights per byte (one multiply-add per weight and
// activation row), so the contraction runs as integer MMA, exactly:
//   * each activation row is scaled by a power of two to |x'| < 1 and written as four signed
//     7-bit digits, x' = (q0 + q1/128 + q2/128^2 + q3/128^3) / 64, truncation error < 4e-9;
//     digit d of row m is row 4m+d of an int8 matrix Xq [N, in] (N = 16, 32, 48 or 64);
//   * a CTA streams a [128 rows x 256 weights] tile of packed 2-bit fields (f = t + 1) through
//     TMA, four warps expand the fields to int8 in the K-major 128-byte-swizzle layout that
//     tcgen05.mma reads, and one thread issues kind::i8 MMAs  acc[128, N] += F . Xq^T  into
//     int32 accumulators in TMEM;
//   * sum_k x t = sum_k x f - sum_k x, so a per-row digit sum is subtracted at the end.
// Integer accumulation is exact and order-independent, which makes split-K over atomics
// deterministic.  A finalize kernel recombines the digits in double precision.
#include <cuda.h>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace mcl {
namespace {

constexpr int GV_ROWS = 128;       // output rows per tile (UMMA M)
constexpr int GV_KB = 256;         // weights per k-block = 64 packed bytes per row
constexpr int GV_RAW = GV_ROWS * (GV_KB / 4);          // 8 KiB staging of packed bytes

constexpr int GV_THREADS = 320;
constexpr int GV_MAX_STAGES = 12;      // slots of the raw ring (packed weights + activation digits)
constexpr int GV_EXP = 4;              // expanded tiles in flight in tensor memory, 64 columns each
constexpr int GV_ACOLS = 64;           // a [128 rows x 256 int8] tile = 64 32-bit columns

struct GvParams {
    int O, I, Nq;
    int ncols;         // 4 * M: digit columns that carry data
    int kblocks, kb_per_split, splits, stages;
    int* acc;          // int32 [Nq][O]: column n of all rows contiguous, so a warp's 32 rows coalesce
    int* err;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

// Instruction descriptor, kind::i8: D = s32 (bits 4-5 = 2), A = B = signed 8-bit (bits 7-9,
// 10-12 = 1), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t idesc_i8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Expansion of one packed word (16 fields) into 16 bytes costs seven logic ops when output word i
// takes the fields 4j + i (j = byte index): (w >> 2i) & 0x03030303.  That permutes k inside every
// group of 16 (byte 4i + j of the group holds weight 4j + i); a contraction over k does not care as
// long as the activation digits are stored in the same order, which gemv_quantize_kernel does.
__device__ __forceinline__ int gv_kperm(int k) { return (k & ~15) | ((k & 3) << 2) | ((k >> 2) & 3); }


__global__ void __launch_bounds__(GV_THREADS) gemv_tc_kernel(const __grid_constant__ CUtensorMap tmP,
                                                             const __grid_constant__ CUtensorMap tmX,
                                                             const GvParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * GV_MAX_STAGES + 2 * GV_EXP + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.stages, Nq = p.Nq;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_tile = (uint32_t)Nq * 128u;
    // Shared memory holds only what TMA delivers (a raw slot = packed weights | the two digit tiles).  The
    // expanded int8 weight tile is four times larger than its packed form; it is written to TENSOR MEMORY
    // (tcgen05.st, thread = row = TMEM lane) and the MMA takes its A operand from there, so neither the
    // expansion nor the operand fetch uses shared-memory bandwidth.
    const uint32_t stage_bytes = GV_RAW + 2 * b_tile;
    const uint32_t bar0 = smem_u32(bars);
    auto raw_full = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (GV_MAX_STAGES + s); };
    auto a_full = [&](int e) { return bar0 + 8u * (2 * GV_MAX_STAGES + e); };
    auto a_empty = [&](int e) { return bar0 + 8u * (2 * GV_MAX_STAGES + GV_EXP + e); };
    auto acc_full = [&](int a) { return bar0 + 8u * (2 * GV_MAX_STAGES + 2 * GV_EXP + a); };
    auto acc_empty = [&](int a) { return bar0 + 8u * (2 * GV_MAX_STAGES + 2 * GV_EXP + 2 + a); };
    // TMEM columns: [0, 2 Nq) two accumulators, [a_col0, a_col0 + GV_EXP * 64) expanded tiles
    const uint32_t a_col0 = 128;
    const uint32_t tmem_cols = 512;

    const int row_tiles = (p.O + GV_ROWS - 1) / GV_ROWS;
    const int n_items = row_tiles * p.splits;

    if (threadIdx.x == 0) {
        abort_flag = (*reinterpret_cast<volatile int*>(p.err) != 0);
        for (int s = 0; s < S; ++s) { mbar_init(raw_full(s), 1); mbar_init(empty_bar(s), 1); }
        for (int e = 0; e < GV_EXP; ++e) { mbar_init(a_full(e), 128); mbar_init(a_empty(e), 1); }
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
            // ---- TMA producer: packed weight tile + the two activation-digit tiles of a k-block ----
            uint32_t it = 0;
            for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x) {
                const int rt = item % row_tiles, split = item / row_tiles;
                const int kb0 = split * p.kb_per_split;
                const int nkb = min(p.kb_per_split, p.kblocks - kb0);
                for (int j = 0; j < nkb; ++j, ++it) {
                    const int s = (int)(it % (uint32_t)S);
                    const uint32_t ph = (it / (uint32_t)S) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 11); break; }
                    const uint32_t st = base + (uint32_t)s * stage_bytes;
                    const int kb = kb0 + j;
                    mbar_expect_tx(raw_full(s), GV_RAW + 2 * b_tile);
                    tma_load_2d(st, &tmP, raw_full(s), kb * (GV_KB / 4), rt * GV_ROWS);
                    tma_load_2d(st + GV_RAW, &tmX, raw_full(s), kb * GV_KB, 0);
                    tma_load_2d(st + GV_RAW + b_tile, &tmX, raw_full(s), kb * GV_KB + 128, 0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer: 8 x (128 x Nq x 32) int8 MMAs per k-block ------------------------------
            const uint32_t idesc = idesc_i8(GV_ROWS, Nq);
            uint32_t it = 0, n_local = 0;
            for (int item = blockIdx.x; item < n_items && !abort_flag; item += gridDim.x, ++n_local) {
                const int split = item / row_tiles;
                const int kb0 = split * p.kb_per_split;
                const int nkb = min(p.kb_per_split, p.kblocks - kb0);
                const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
                if (!mbar_wait(acc_empty(acc), aph ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 14); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * (uint32_t)Nq;
                for (int j = 0; j < nkb; ++j, ++it) {
                    const int s = (int)(it % (uint32_t)S);
                    const int e = (int)(it % GV_EXP);
                    // the expanders arrive after they have seen the raw slot: this wait covers the digit tiles too
                    if (!mbar_wait(a_full(e), (it / GV_EXP) & 1u, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 12); break; }
                    tc_fence_after();
                    const uint32_t st = base + (uint32_t)s * stage_bytes;
                    const uint32_t a_tm = tmem_base + a_col0 + (uint32_t)e * GV_ACOLS;
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const uint64_t db = smem_desc_k_sw128(st + GV_RAW + t * b_tile);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)      // 32 int8 of k = 8 TMEM columns of A, 32 bytes (+2) of B
                            umma_i8_ts(d_tmem, a_tm + (uint32_t)(t * 32 + kk * 8), db + 2u * kk, idesc, (j | t | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(a_empty(e));
                    umma_commit(empty_bar(s));
                }
                if (abort_flag) break;
                umma_commit(acc_full(acc));
            }
        }
    } else if (warp < 6) {
        // ---- expanders: 2-bit fields -> int8, written to tensor memory; thread = tile row = TMEM lane ----
        // a warp may touch the TMEM lanes of its quarter (warp % 4) only: that quarter is its 32 tile rows
        const int r = ((warp & 3) << 5) | lane;         // 0..127
        const uint32_t rsw64 = (uint32_t)((r >> 1) & 3);
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int split = item / row_tiles;
            const int kb0 = split * p.kb_per_split;
            const int nkb = min(p.kb_per_split, p.kblocks - kb0);
            for (int j = 0; j < nkb; ++j, ++it) {
                const int s = (int)(it % (uint32_t)S);
                const uint32_t ph = (it / (uint32_t)S) & 1u;
                const int e = (int)(it % GV_EXP);
                if (abort_flag || !mbar_wait(raw_full(s), ph, &abort_flag) ||
                    !mbar_wait(a_empty(e), ((it / GV_EXP) & 1u) ^ 1u, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 13); ok = false; break; }
                tc_fence_after();      // the MMAs that read this TMEM slot have completed (a_empty)
                unsigned char* st = smem_raw + (base - smem_u32(smem_raw)) + (size_t)s * stage_bytes;
                const uint4* raw = reinterpret_cast<const uint4*>(st + r * 64);
                const uint32_t a_tm = tmem_base + lane_base + a_col0 + (uint32_t)e * GV_ACOLS;
#pragma unroll
                for (int h = 0; h < 2; ++h) {           // half a row: 32 packed bytes = 128 weights = 32 TMEM columns
                    uint32_t v[32];
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int c = 2 * h + cc;
                        const uint4 pk = raw[c ^ rsw64];    // staging was written with the 64-byte swizzle
                        const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {       // one word = 16 weights = four columns of int8
                            v[cc * 16 + q * 4 + 0] = w[q] & 0x03030303u;
                            v[cc * 16 + q * 4 + 1] = (w[q] >> 2) & 0x03030303u;
                            v[cc * 16 + q * 4 + 2] = (w[q] >> 4) & 0x03030303u;
                            v[cc * 16 + q * 4 + 3] = (w[q] >> 6) & 0x03030303u;
                        }
                    }
                    tmem_st32(a_tm + (uint32_t)(32 * h), v);
                }
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(a_full(e));
            }
        }
    } else {
        // ---- epilogue warps: int32 accumulator -> global (atomic when k is split) ---------------
        const int q = warp & 3;
        uint32_t n_local = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n_local) {
            const int rt = item % row_tiles;
            const uint32_t acc = n_local & 1u, aph = (n_local >> 1) & 1u;
            bool ok = !abort_flag;
            if (ok && !mbar_wait(acc_full(acc), aph, &abort_flag)) { abort_flag = 1; atomicExch(p.err, 15); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = rt * GV_ROWS + q * 32 + lane;
            int* dst = p.acc + row;
            for (int c0 = 0; c0 < Nq; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + acc * (uint32_t)Nq + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                tmem_ld_wait();
                if (row < p.O) {
                    // columns at and beyond 4 M are padding of the digit matrix (all zero): nothing to add
                    if (p.splits == 1) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < p.ncols) dst[(size_t)(c0 + j) * p.O] = (int)v[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < p.ncols) atomicAdd(dst + (size_t)(c0 + j) * p.O, (int)v[j]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty(acc));
        }
    }
    __syncwarp();
    if (abort_flag) {
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 2000000ull) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ---- activation rows -> four int8 digit rows each, digit sums, power-of-two scale ---------------
// grid = Nq / 4 blocks (one per activation row slot; slots >= M are written as zeros)
__global__ void __launch_bounds__(256) gemv_quantize_kernel(const float* __restrict__ x, int M, int I,
                                                            signed char* __restrict__ xq, int* __restrict__ corr,
                                                            float* __restrict__ xscale, int4* __restrict__ acc_clear,
                                                            long long clear_int4) {
    __shared__ float red[256];
    __shared__ int isum[4];
    const int m = blockIdx.x, tid = threadIdx.x;
    if (blockIdx.y > 0) {
        // the blocks of the other grid rows only zero the split-K accumulators of the contraction that follows
        const long long nthr = (long long)gridDim.x * (gridDim.y - 1) * 256;
        for (long long i = ((long long)(blockIdx.y - 1) * gridDim.x + blockIdx.x) * 256 + tid; i < clear_int4; i += nthr)
            acc_clear[i] = make_int4(0, 0, 0, 0);
        return;
    }
    signed char* q0 = xq + (size_t)(4 * m) * I;
    if (m >= M) {
        for (int k = tid; k < I; k += 256) { q0[k] = 0; q0[I + k] = 0; q0[2 * (size_t)I + k] = 0; q0[3 * (size_t)I + k] = 0; }
        return;
    }
    const float* xr = x + (size_t)m * I;
    float amax = 0.0f;
    for (int k = tid; k < I; k += 256) amax = fmaxf(amax, fabsf(__ldg(xr + k)));
    red[tid] = amax;
    if (tid < 4) isum[tid] = 0;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]);
        __syncthreads();
    }
    amax = red[0];
    int e = 0;
    if (amax > 0.0f) frexpf(amax, &e);              // amax = f * 2^e, f in [0.5, 1): 2^e > amax
    const float inv = ldexpf(64.0f, -e);            // x * inv = x' * 64 with |x'| < 1, exact scaling
    int s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    for (int k = tid; k < I; k += 256) {
        float v = __ldg(xr + k) * inv;
        const float d0 = rintf(v); v = (v - d0) * 128.0f;
        const float d1 = rintf(v); v = (v - d1) * 128.0f;
        const float d2 = rintf(v); v = (v - d2) * 128.0f;
        const float d3 = rintf(v);
        const int kp = gv_kperm(k);          // the order in which the expanded weights lie
        q0[kp] = (signed char)d0; q0[I + kp] = (signed char)d1;
        q0[2 * (size_t)I + kp] = (signed char)d2; q0[3 * (size_t)I + kp] = (signed char)d3;
        s0 += (int)d0; s1 += (int)d1; s2 += (int)d2; s3 += (int)d3;
    }
    atomicAdd(&isum[0], s0); atomicAdd(&isum[1], s1); atomicAdd(&isum[2], s2); atomicAdd(&isum[3], s3);
    __syncthreads();
    if (tid < 4) corr[4 * m + tid] = isum[tid];
    if (tid == 0) xscale[m] = ldexpf(1.0f, e) / 64.0f;
}

// y[m,o] = scale[o] * xscale[m] * sum_d 128^-d * (acc[o][4m+d] - corr[4m+d])
__global__ void gemv_finalize_kernel(const int* __restrict__ acc, const int* __restrict__ corr,
                                     const float* __restrict__ xscale, const float* __restrict__ scale,
                                     float* __restrict__ y, int M, int O, int Nq) {
    const int o = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
    if (o >= O) return;
    const int a0 = __ldg(acc + (size_t)(4 * m + 0) * O + o), a1 = __ldg(acc + (size_t)(4 * m + 1) * O + o);
    const int a2 = __ldg(acc + (size_t)(4 * m + 2) * O + o), a3 = __ldg(acc + (size_t)(4 * m + 3) * O + o);
    const double sum = (double)(a0 - corr[4 * m]) + (double)(a1 - corr[4 * m + 1]) * (1.0 / 128.0) +
                       (double)(a2 - corr[4 * m + 2]) * (1.0 / 16384.0) + (double)(a3 - corr[4 * m + 3]) * (1.0 / 2097152.0);
    y[(size_t)m * O + o] = (float)((double)__ldg(scale + o) * (double)xscale[m] * sum);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn gv_encode_tiled() {
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
bool gv_map_2d(CUtensorMap* map, const void* basep, size_t inner_bytes, size_t rows, size_t pitch_bytes,
               int box_inner, int box_rows, CUtensorMapSwizzle sw) {
    EncodeTiledFn enc = gv_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(basep), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool gemv_tc_supported(int M, int in_features, int out_features) {
    return M >= 1 && M <= 16 && in_features % 64 == 0 && in_features >= 256 && out_features >= 1;
}

// workspace: Xq [64][in] int8 | corr [64] int | xscale [16] float | acc [Nq][out] int32
size_t gemv_tc_workspace_bytes(int M, int in_features, int out_features) {
    const int Nq = 16 * ((M + 3) / 4);
    size_t o = ((size_t)64 * in_features + 1023) & ~size_t(1023);
    o += 1024;
    o += ((size_t)out_features * Nq * sizeof(int) + 1023) & ~size_t(1023);
    return o;
}

cudaError_t launch_ternary_gemv_tc(const float* x, const uint32_t* packed2, const float* scale, float* y, int M,
                                   int in_features, int out_features, void* workspace, int* err_word, int sm_count,
                                   size_t max_smem, cudaStream_t stream, int* launches) {
    const int I = in_features, O = out_features;
    const int Nq = 16 * ((M + 3) / 4);
    char* w = static_cast<char*>(workspace);
    signed char* xq = reinterpret_cast<signed char*>(w);
    size_t o = ((size_t)64 * I + 1023) & ~size_t(1023);
    int* corr = reinterpret_cast<int*>(w + o);
    float* xscale = reinterpret_cast<float*>(w + o + 512);
    int* acc = reinterpret_cast<int*>(w + o + 1024);

    GvParams p;
    p.O = O; p.I = I; p.Nq = Nq; p.ncols = 4 * M;
    p.kblocks = (I + GV_KB - 1) / GV_KB;
    const int row_tiles = (O + GV_ROWS - 1) / GV_ROWS;
    int splits = 1;
    if (row_tiles < 2 * sm_count) {
        splits = (3 * sm_count + row_tiles - 1) / row_tiles;
        if (splits > p.kblocks / 2) splits = p.kblocks / 2;
        if (splits < 1) splits = 1;
    }
    p.kb_per_split = (p.kblocks + splits - 1) / splits;
    p.splits = splits = (p.kblocks + p.kb_per_split - 1) / p.kb_per_split;
    p.acc = acc; p.err = err_word;
    const size_t stage_bytes = (size_t)GV_RAW + 2 * (size_t)Nq * 128;
    int stages = (int)((max_smem - 2048) / stage_bytes);
    if (stages > GV_MAX_STAGES) stages = GV_MAX_STAGES;
    if (stages < 2) return cudaErrorInvalidConfiguration;
    p.stages = stages;

    CUtensorMap mp, mx;
    if (!gv_map_2d(&mp, packed2, (size_t)I / 4, (size_t)O, (size_t)I / 4, GV_KB / 4, GV_ROWS, CU_TENSOR_MAP_SWIZZLE_64B))
        return cudaErrorInvalidValue;
    if (!gv_map_2d(&mx, xq, (size_t)I, 64, (size_t)I, 128, Nq, CU_TENSOR_MAP_SWIZZLE_128B)) return cudaErrorInvalidValue;

    // one launch quantizes the activations and, when k is split, zeroes the digit columns of the accumulators
    // that carry data (O * 4 M ints: O is padded to a multiple of 4 by the 1 KiB rounding of the workspace)
    const long long clear_int4 = splits > 1 ? ((long long)O * 4 * M + 3) / 4 : 0;
    int clear_rows = 0;
    if (clear_int4 > 0) {
        clear_rows = (int)((clear_int4 + (long long)(Nq / 4) * 256 * 8 - 1) / ((long long)(Nq / 4) * 256 * 8));
        if (clear_rows < 1) clear_rows = 1;
        if (clear_rows > 64) clear_rows = 64;
    }
    gemv_quantize_kernel<<<dim3(Nq / 4, 1 + clear_rows), 256, 0, stream>>>(x, M, I, xq, corr, xscale,
                                                                           reinterpret_cast<int4*>(acc), clear_int4);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ++*launches;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    e = ensure_dynamic_smem(reinterpret_cast<const void*>(gemv_tc_kernel), 5, max_smem);
    if (e != cudaSuccess) return e;
    int ctas = row_tiles * splits;
    if (ctas > sm_count) ctas = sm_count;
    gemv_tc_kernel<<<ctas, GV_THREADS, smem, stream>>>(mp, mx, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ++*launches;
    gemv_finalize_kernel<<<dim3((O + 255) / 256, M), 256, 0, stream>>>(acc, corr, xscale, scale, y, M, O, Nq);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ++*launches;
    return cudaSuccess;
}


}  // namespace mcl
