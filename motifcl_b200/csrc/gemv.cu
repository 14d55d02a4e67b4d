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


// ---- M = 1: table look-up kernels ------------------------------------------------------------------------------------
// With one multiply-add per weight the CUDA cores spend three instructions per weight (two to turn a 2-bit field into a
// float, one FMA) and cannot follow the memory.  Here the activations go into a table first: for every PAIR of
// consecutive activations (x0, x1) the 16 sums (f0 - 1) x0 + (f1 - 1) x1 over the two fields' values are stored (one
// rounding per entry, 64 bytes per pair), so a pair of weights costs one look-up with the nibble that holds its two
// fields, and one add: (word << 2) & 0x3C3C3C3C holds nibble x 4 - the entry's byte offset - in every byte, one prmt
// takes a byte out and the load is [byte + constant].  Lanes of a warp are different ROWS looking at the same pair of
// activations, so a load touches the 16 banks of one table entry set: no conflicts, whatever the data.
//
// gemv_lut_kernel (in_features > 4096): grid = (blocks of 256 rows) x (slices of KS weights along k).  A CTA copies its
// rows' words of the slice into shared memory (cp.async, coalesced) and meanwhile builds the table of the slice; then
// thread = row.  The slices of a row block meet through partial sums in global memory: every CTA stores its sums, takes
// a ticket, and the CTA that draws the last ticket adds the slices in slice order (deterministic, whichever CTA is last),
// applies the row scale, writes y and puts the ticket word back to zero for the next launch.  No CTA waits for another.
template <int KS>
__global__ void __launch_bounds__(256) gemv_lut_kernel(const float* __restrict__ x, const uint32_t* __restrict__ packed2,
                                                      const float* __restrict__ scale, float* __restrict__ y,
                                                      float* __restrict__ part, unsigned int* __restrict__ tickets, int I,
                                                      int O) {
    constexpr int G = KS / 2;                    // pairs of weights per slice
    constexpr int NV = KS / 64;                  // 16-byte pieces per row and slice (4 or 8)
    __shared__ __align__(16) float tab[G * 16];
    __shared__ __align__(16) uint4 wt[256 * NV];     // the CTA's 256 rows x KS / 4 bytes of 2-bit words
    const int slice = blockIdx.y, S = gridDim.y;
    const int row = blockIdx.x * 256 + threadIdx.x;
    // A row's pieces sit at wt[r * NV + (c ^ swz(r))]: thread r then reads its own row with 16-byte loads that spread
    // over all banks (rows that would share banks take different piece slots).
    auto swz = [](int r) { return NV == 8 ? (r & 7) : ((r >> 1) & 3); };

#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int L = j * 256 + threadIdx.x;
        const int r = L / NV, c = L % NV;            // NV consecutive threads copy one row's contiguous bytes
        const int gr = min(blockIdx.x * 256 + r, O - 1);
        const uint4* src = reinterpret_cast<const uint4*>(packed2 + (size_t)gr * (I >> 4) + (size_t)slice * (KS / 16)) + c;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(wt + r * NV + (c ^ swz(r)));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int g = threadIdx.x; g < G; g += 256) {
        const float2 xv = __ldg(reinterpret_cast<const float2*>(x + (size_t)slice * KS) + g);
        const float a[4] = {-xv.x, 0.0f, xv.x, 2.0f * xv.x};         // (f - 1) x: exact
        float4* dst = reinterpret_cast<float4*>(tab + (size_t)g * 16);
        // the four 16-byte stores go out in an order rotated by lane / 2: consecutive lanes' entry sets are 64 bytes
        // apart, so lanes 0, 2, 4, 6 would otherwise store into the same banks
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int f1 = (t + ((threadIdx.x & 31) >> 1)) & 3;
            const float bf = (float)(f1 - 1) * xv.y;                   // exact
            dst[f1] = make_float4(__fadd_rn(a[0], bf), __fadd_rn(a[1], bf), __fadd_rn(a[2], bf), __fadd_rn(a[3], bf));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};     // four chains: byte b of a word adds into chain b
    const char* tb = reinterpret_cast<const char*>(tab);
    const int sw = swz(threadIdx.x);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint4 wv = wt[threadIdx.x * NV + (i ^ sw)];
        const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t lo = (w4[q] << 2) & 0x3C3C3C3Cu;          // nibbles 0, 2, 4, 6 of the word, x 4
            const uint32_t hi = (w4[q] >> 2) & 0x3C3C3C3Cu;          // nibbles 1, 3, 5, 7
            const int g0 = (i * 4 + q) * 8;                          // first pair of this word in the slice
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t o0 = __byte_perm(lo, 0u, 0x4440u | (uint32_t)b);
                const uint32_t o1 = __byte_perm(hi, 0u, 0x4440u | (uint32_t)b);
                acc[b] += *reinterpret_cast<const float*>(tb + (size_t)(g0 + 2 * b) * 64 + o0);
                acc[b] += *reinterpret_cast<const float*>(tb + (size_t)(g0 + 2 * b + 1) * 64 + o1);
            }
        }
    }
    const float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);

    if (S == 1) {
        if (row < O) y[row] = __ldg(scale + row) * sum;
        return;
    }
    if (row < O) part[(size_t)slice * O + row] = sum;
    __threadfence();
    __syncthreads();                                 // also: every thread is done with the table
    int* is_last = reinterpret_cast<int*>(tab);      // its first word now carries the ticket's verdict
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(tickets + blockIdx.x, 1u);
        *is_last = (t == (unsigned int)(S - 1));
    }
    __syncthreads();
    if (!*is_last) return;
    __threadfence();
    if (row < O) {
        float a = 0.0f;
        for (int s0 = 0; s0 < S; s0 += 16) {         // 16 loads in flight, added in slice order
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = s0 + j < S ? __ldcg(part + (size_t)(s0 + j) * O + row) : 0.0f;
#pragma unroll
            for (int j = 0; j < 16; ++j) a += v[j];
        }
        y[row] = __ldg(scale + row) * a;
    }
    if (threadIdx.x == 0) tickets[blockIdx.x] = 0u;
}

// gemv_lutk_kernel (in_features <= 4096): ONE table for the whole row length.  The sliced kernel above spends more time
// around its look-ups than in them: every CTA builds a table, the slices of a row meet through global memory and a
// ticket.  When the table of ALL activations fits in shared memory (32 bytes per activation) none of that is needed.  One
// persistent CTA of 32 warps per SM builds the table once and owns a contiguous range of 16-row groups.  A unit of work
// is 16 rows x 256 weights (1 KB of words); a warp takes the units of its row block round-robin, fetches each with two
// 16-byte cp.async per lane two units ahead (a ring of two slots per warp), and TWO lanes share a row: lane h = 0 takes
// the even nibbles of every word, lane h = 1 the odd ones (rotate by 2 or 30, mask; bit 6 of every byte set for h = 1:
// the odd pair's entries lie 64 bytes after the even pair's, i.e. in banks 16-31 where the even pair's are in banks
// 0-15, so a load is one conflict-free pass over all 32 banks).  A lane folds the unit's table address into the byte
// it extracts (prmt takes the upper three bytes from a register that holds the 256-byte aligned base), so a look-up
// stays one prmt, one load and one add.  The 64-weight sums of a unit go to shared memory ([chunk][row]) and one thread
// per row adds a row's chunks in order: deterministic, no atomics, nothing crosses CTAs.
// One shared-memory load at [register + constant]: the table look-ups below need the constant IN the instruction (the
// register already holds base | entry offset), which the compiler does not do for addresses built from 64-bit pointers.
template <int IMM>
__device__ __forceinline__ float lds_f32_at(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(IMM));
    return v;
}

constexpr int kLkWarps = 32;
constexpr int kLkThreads = kLkWarps * 32;
constexpr int kLkRowBlock = 128;           // rows whose chunk sums are held at a time
constexpr int kLkMaxIn = 4096;
constexpr int kLkRing = 2;                 // unit slots per warp

__global__ void __launch_bounds__(kLkThreads, 1) gemv_lutk_kernel(const float* __restrict__ x,
                                                                  const uint32_t* __restrict__ packed2,
                                                                  const float* __restrict__ scale, float* __restrict__ y,
                                                                  int I, int O, int groups_q, int groups_r, int chunk_inv) {
    extern __shared__ __align__(1024) unsigned char lk_smem[];
    // table (32 I bytes, at the first 256-byte boundary: a look-up merges an entry's offset into the low byte of the
    // table's address) | ring: warps x slots x 1 KB | chunk sums: (I / 256) x 128 floats
    const int chunks = I >> 8;
    const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(lk_smem);
    const uint32_t tab32 = (smem0 + 255u) & ~255u;
    unsigned char* tabp = lk_smem + (tab32 - smem0);
    unsigned char* ring0 = tabp + (size_t)32 * I;
    float* csum = reinterpret_cast<float*>(ring0 + (size_t)kLkWarps * kLkRing * 1024);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = lane >> 4, r = lane & 15;

    // the activations first: their latency passes under the address arithmetic and the first copies
    const int pairs = I >> 1;
    float2 xv[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int g = threadIdx.x + j * kLkThreads;
        xv[j] = g < pairs ? __ldg(reinterpret_cast<const float2*>(x) + g) : make_float2(0.0f, 0.0f);
    }

    // this CTA's 16-row groups: groups_q each, the first groups_r CTAs one more
    const int g_begin = blockIdx.x * groups_q + min((int)blockIdx.x, groups_r);
    const int g_end = g_begin + groups_q + ((int)blockIdx.x < groups_r ? 1 : 0);

    unsigned char* my_ring = ring0 + (size_t)warp * kLkRing * 1024;
    const size_t wpr = (size_t)(I >> 4);
    // a warp's units of a row block are warp, warp + 32, ...; unit u = chunk u % chunks of group u / chunks, kept as a
    // (group, chunk) cursor that steps by 32 units without dividing
    // (chunk_inv = ceil(2^16 / chunks) from the host: n * chunk_inv >> 16 = n / chunks for n <= 32)
    const int step_g = (kLkWarps * chunk_inv) >> 16, step_c = kLkWarps - step_g * chunks;
    const int first_g = (warp * chunk_inv) >> 16, first_c = warp - first_g * chunks;
    auto advance = [&](int& g, int& c) {
        g += step_g; c += step_c;
        if (c >= chunks) { c -= chunks; ++g; }
    };
    const int pr0 = lane >> 2, pc = lane & 3;           // a lane copies piece pc of rows pr0 and pr0 + 8 of a unit
    auto fetch = [&](int row0, int c, int slot) {       // row0: first row of the unit's group
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int pr = pr0 + 8 * j;
            const int grow = min(row0 + pr, O - 1);
            const uint4* src = reinterpret_cast<const uint4*>(packed2 + (size_t)grow * wpr + (size_t)c * 16) + pc;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(my_ring + slot * 1024 + pr * 64 + ((pc ^ ((pr >> 1) & 3)) << 4));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
    };

    const uint32_t rot = h ? 30u : 2u;                  // rotate left by 2 (even nibbles) or right by 2 (odd nibbles)
    const uint32_t hbit = h ? 0x40404040u : 0u;         // + 64 bytes: the odd pair's table
    for (int gb = g_begin; gb < g_end; gb += kLkRowBlock / 16) {
        const int ng = min(kLkRowBlock / 16, g_end - gb);
        int fg = first_g, fc = first_c;                 // fetch cursor
#pragma unroll
        for (int k = 0; k < kLkRing; ++k) {
            if (fg < ng) fetch((gb + fg) * 16, fc, k);
            asm volatile("cp.async.commit_group;" ::: "memory");
            advance(fg, fc);
        }
        if (gb == g_begin) {
            // the table, once per CTA, while the first units travel
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int g = threadIdx.x + j * kLkThreads;
                if (g < pairs) {
                    const float a[4] = {-xv[j].x, 0.0f, xv[j].x, 2.0f * xv[j].x};         // (f - 1) x: exact
                    float4* dst = reinterpret_cast<float4*>(tabp + (size_t)g * 64);
                    // a thread's four 16-byte stores go out in an order rotated by lane / 2: consecutive lanes' entry
                    // sets are 64 bytes apart, so lanes 0, 2, 4, 6 would otherwise store into the same banks
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const int f1 = (t + (lane >> 1)) & 3;
                        const float bf = (float)(f1 - 1) * xv[j].y;                          // exact
                        dst[f1] = make_float4(__fadd_rn(a[0], bf), __fadd_rn(a[1], bf), __fadd_rn(a[2], bf), __fadd_rn(a[3], bf));
                    }
                }
            }
            __syncthreads();
        }
        int k = 0;
        for (int cg = first_g, cc = first_c; cg < ng; advance(cg, cc), ++k) {
            asm volatile("cp.async.wait_group %0;" ::"n"(kLkRing - 1) : "memory");
            __syncwarp();
            const int slot = k % kLkRing;
            const uint4* rowp = reinterpret_cast<const uint4*>(my_ring + slot * 1024 + r * 64);
            const uint32_t base = tab32 + ((uint32_t)cc << 13);        // table of this chunk: 128 pairs x 64 B = 8 KB
            const int sw = (r >> 1) & 3;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            // word WD of the unit's 16: this lane's four nibbles x 4 in the bytes of v; a look-up takes byte b of v below
            // the upper three bytes of the chunk's table address (prmt) and loads at + (pair of nibble 2 b) x 64
#define LK_WORD(WD, W)                                                                             \
    {                                                                                              \
        const uint32_t v = (__funnelshift_l((W), (W), rot) & 0x3C3C3C3Cu) | hbit;                  \
        acc[0] += lds_f32_at<((WD) * 8 + 0) * 64>(__byte_perm(v, base, 0x7650u));                  \
        acc[1] += lds_f32_at<((WD) * 8 + 2) * 64>(__byte_perm(v, base, 0x7651u));                  \
        acc[2] += lds_f32_at<((WD) * 8 + 4) * 64>(__byte_perm(v, base, 0x7652u));                  \
        acc[3] += lds_f32_at<((WD) * 8 + 6) * 64>(__byte_perm(v, base, 0x7653u));                  \
    }
#define LK_QUAD(Q)                                                                                 \
    {                                                                                              \
        const uint4 wv = rowp[(Q) ^ sw];                                                           \
        LK_WORD((Q) * 4 + 0, wv.x) LK_WORD((Q) * 4 + 1, wv.y) LK_WORD((Q) * 4 + 2, wv.z) LK_WORD((Q) * 4 + 3, wv.w) \
    }
            LK_QUAD(0) LK_QUAD(1) LK_QUAD(2) LK_QUAD(3)
#undef LK_QUAD
#undef LK_WORD
            float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            sum += __shfl_xor_sync(0xffffffffu, sum, 16);
            if (h == 0) csum[cc * kLkRowBlock + cg * 16 + r] = sum;
            __syncwarp();                                     // every lane is done with the slot
            if (fg < ng) fetch((gb + fg) * 16, fc, slot);
            asm volatile("cp.async.commit_group;" ::: "memory");
            advance(fg, fc);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if ((int)threadIdx.x < ng * 16) {
            const int row = gb * 16 + threadIdx.x;
            if (row < O) {
                float a = 0.0f;
                for (int c = 0; c < chunks; ++c) a += csum[c * kLkRowBlock + threadIdx.x];
                y[row] = __ldg(scale + row) * a;
            }
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

bool gemv_lut_supported(int M, int in_features, int out_features, const void* packed2, int ticket_words) {
    return M == 1 && in_features % 256 == 0 && reinterpret_cast<uintptr_t>(packed2) % 16 == 0 &&
           (out_features + 255) / 256 <= ticket_words;
}

// part: [slices][out] floats of the sliced kernel; at most in / 256 slices
size_t gemv_lut_workspace_bytes(int in_features, int out_features) {
    return in_features <= kLkMaxIn ? 0 : (size_t)(in_features / 256) * (size_t)out_features * sizeof(float);
}

cudaError_t launch_ternary_gemv_lut(const float* x, const uint32_t* packed2, const float* scale, float* y,
                                    int in_features, int out_features, float* part, unsigned int* tickets, int sm_count,
                                    size_t max_smem, cudaStream_t stream) {
    const int I = in_features, O = out_features;
    const size_t lk_smem = 256 + (size_t)32 * I + (size_t)kLkWarps * kLkRing * 1024 + (size_t)(I >> 8) * kLkRowBlock * sizeof(float);
    if (I <= kLkMaxIn && lk_smem <= max_smem) {
        cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(gemv_lutk_kernel), 12, max_smem);
        if (e != cudaSuccess) return e;
        const int groups = (O + 15) / 16;
        const int grid = groups < sm_count ? groups : sm_count;
        const int chunks = I >> 8;
        gemv_lutk_kernel<<<grid, kLkThreads, lk_smem, stream>>>(x, packed2, scale, y, I, O, groups / grid, groups % grid,
                                                                (65536 + chunks - 1) / chunks);
        return cudaGetLastError();
    }
    // the longest slice that still gives every SM two CTAs (measured: fewer, longer slices beat more CTAs)
    const int rb = (O + 255) / 256;
    if (I % 512 == 0 && (long long)rb * (I / 512) >= 2LL * sm_count)
        gemv_lut_kernel<512><<<dim3(rb, I / 512), 256, 0, stream>>>(x, packed2, scale, y, part, tickets, I, O);
    else
        gemv_lut_kernel<256><<<dim3(rb, I / 256), 256, 0, stream>>>(x, packed2, scale, y, part, tickets, I, O);
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
