// Fused compact-counter update for sm_100a: one pass over HBM per weight row.
//
// Replaces the reference's three launches per layer -- counter_row_stats_f32,
// counter_apply_update_f32 and copy_f32 (MotifCL src/nn/compact_counter.cpp:113-156,
// kernels/compact_counter.cl:59-139, kernels/basic.cl:6-9) -- with one kernel that reads the
// packed 6-bit state and the fp32 weight gradient once, and writes the new state, the 2-bit
// packed ternary weights and the per-row scale / RMS moment.
//
// Work decomposition.  A CTA owns a batch of ROWS weight rows at a time (persistent loop
// over batches).  For each batch:
//   load   all threads copy the rows' gradient (128-bit loads) and state bytes into
//          shared memory; when lr_scale != 0 they also store q = gw * t.
//   stats  one warp pair (64 threads) per row replays the reference's reduction order
//          exactly: 64 lanes, lane l accumulates groups l, l+64, ... with separately
//          rounded multiply and add, then the 32,16,...,1 tree (first step through shared
//          memory, the rest by warp shuffles).  Lane 0 finishes v, denom and the new scale.
//   tick   all threads run the stochastic-rounding tick, one packed group (4 weights) per
//          thread-iteration, writing the new state bytes to shared memory and emitting one
//          byte of 2-bit fields per group.  The part of the tick after the stochastic
//          rounding -- carry into the ternary digit, clamp, re-encode -- is a function of the
//          old ternary digit and the (small, integer) rounded counter only, so it is read
//          from a table built once per CTA with the reference's own float formulas; values
//          outside the table's range take the formulas directly.
//   store  all threads copy the new state and the 2-bit words back with wide stores.
// HBM traffic per weight: 0.75 B state in, 4 B gradient in, 0.75 B state out, 0.25 B
// packed weights out = 5.75 B.
#include "counter_codec.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace mcl {

namespace {

constexpr int kUpdThreads = 256;             // 4 warp pairs
constexpr int kMaxRowsPerBatch = kUpdThreads / 64;

struct UpdParams {
    uint8_t* state;          // [rows, in/4*3]
    float* scale;            // [rows]
    float* v;                // [rows]
    const float* grad_w;     // [rows, in]
    uint32_t* packed2;       // [rows, in/16] or null
    int C, in_features, rows, row_offset;
    int rows_per_batch;
    int state_align;         // 16, 4 or 1: widest access every state / packed2 row start allows
    float lr, lr_scale, rms_beta, rms_eps;
    uint32_t seed;
    const uint32_t* seed_offset;   // optional device word added to seed (a step counter for recorded batches)
};

struct RowConst {
    float dn, k_tick, k_reb, pad;
};

// Tail table: new 6-bit code and 2-bit field for (old ternary digit t in {-1,0,1,2}, rounded
// counter ccv in [-kTailK, kTailK]); entry = code | field << 8.
constexpr int kTailK = 32;
constexpr int kTailRow = 2 * kTailK + 1;

// Per-row table indexed by the OLD code: x = float(c) * (s_old / s_new) (the rebased counter),
// y = index of the tail-table row of the code's ternary digit, pre-offset by kTailK.
struct RowEntry {
    float creb;
    int tail_base;
};

// Shared-memory carve-up (per CTA), all offsets 16-byte aligned:
//   lut[64] float2 | rowc[R] RowConst | part[R][2][32] float | gw[R][I] float |
//   q[R][I] float (only WITH_Q) | st[R][sb] bytes (sb = state row bytes rounded up to 16, +16)
//   | so[R][sb] bytes (new state) | p2[R][I/4 rounded to 16] bytes
template <bool WITH_Q>
__global__ void __launch_bounds__(kUpdThreads, 3)
counter_update_dense_kernel(const UpdParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int I = p.in_features;
    const int gpr = I >> 2;
    const int row_bytes = gpr * 3;
    const int sb = ((row_bytes + 15) & ~15) + 16;
    const int pb = (gpr + 15) & ~15;
    const int R = p.rows_per_batch;

    DecodeLut* lut = reinterpret_cast<DecodeLut*>(smem);
    RowConst* rowc = reinterpret_cast<RowConst*>(smem + sizeof(DecodeLut));
    float* part = reinterpret_cast<float*>(rowc + kMaxRowsPerBatch);
    RowEntry* rowtab = reinterpret_cast<RowEntry*>(part + kMaxRowsPerBatch * 64);     // [R][64]
    unsigned short* tail = reinterpret_cast<unsigned short*>(rowtab + kMaxRowsPerBatch * 64);   // [4][kTailRow]
    float* gw_s = reinterpret_cast<float*>(tail + ((4 * kTailRow + 7) & ~7));
    float* q_s = gw_s + (size_t)R * I;
    unsigned char* st_s = reinterpret_cast<unsigned char*>(WITH_Q ? q_s + (size_t)R * I : q_s);
    unsigned char* so_s = st_s + (size_t)R * sb;
    unsigned char* p2_s = so_s + (size_t)R * sb;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int pair = tid >> 6;           // warp pair index = row slot in the stats phase
    const int vlane = tid & 63;          // the reference's work-item id within its 64-wide group
    const int lv = 2 * p.C - 1;
    const float Cf = (float)p.C;
    const float neg_lr = -p.lr;
    const bool check_t = 4 * lv < 64;      // some code values decode to a ternary digit the tail table lacks
    const uint32_t seed = p.seed + (p.seed_offset ? __ldg(p.seed_offset) : 0u);
    const bool aligned16 = p.state_align >= 16;   // state rows start and end on 16-byte boundaries
    const bool aligned4 = p.state_align >= 4;     // ... on 4-byte boundaries

    build_decode_lut(lut, p.C, tid, kUpdThreads);
    // tail table, evaluated with the reference's formulas (kernels/compact_counter.cl:129-136)
    for (int e = tid; e < 4 * kTailRow; e += kUpdThreads) {
        const int t = e / kTailRow - 1;
        const float ccv = (float)(e % kTailRow - kTailK);
        const float carry = truncf(__fdiv_rn(ccv, Cf));
        float rem = __fsub_rn(ccv, __fmul_rn(carry, Cf));
        const int nt = t + (int)carry;
        const int ct = nt < -1 ? -1 : (nt > 1 ? 1 : nt);
        if (ct != nt) rem = __fmul_rn(ccv > 0.0f ? 1.0f : (ccv < 0.0f ? -1.0f : 0.0f), __fsub_rn(Cf, 1.0f));
        int ri = (int)rem;
        ri = ri < -(p.C - 1) ? -(p.C - 1) : (ri > p.C - 1 ? p.C - 1 : ri);
        const unsigned code = (unsigned)((ct + 1) * lv + (ri + (p.C - 1))) & 0x3Fu;
        tail[e] = (unsigned short)(code | ((unsigned)(ct + 1) << 8));
    }
    __syncthreads();

    const int nbatches = (p.rows + R - 1) / R;
    for (int batch = blockIdx.x; batch < nbatches; batch += gridDim.x) {
        const int row0 = batch * R;
        const int nrows = min(R, p.rows - row0);

        // ---- load: state bytes, then gradient (and q) --------------------------------
        for (int r = 0; r < nrows; ++r) {
            const uint8_t* src = p.state + (size_t)(row0 + r) * row_bytes;
            unsigned char* dst = st_s + (size_t)r * sb;
            if (aligned16) {
                const uint4* s4 = reinterpret_cast<const uint4*>(src);
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                for (int i = tid; i < row_bytes / 16; i += kUpdThreads) d4[i] = __ldg(s4 + i);
            } else if (aligned4) {
                const uint32_t* s1 = reinterpret_cast<const uint32_t*>(src);
                uint32_t* d1 = reinterpret_cast<uint32_t*>(dst);
                for (int i = tid; i < row_bytes / 4; i += kUpdThreads) d1[i] = __ldg(s1 + i);
            } else {
                for (int i = tid; i < row_bytes; i += kUpdThreads) dst[i] = __ldg(src + i);
            }
        }
        if (WITH_Q) __syncthreads();
        for (int r = 0; r < nrows; ++r) {
            const float4* src = reinterpret_cast<const float4*>(p.grad_w + (size_t)(row0 + r) * I);
            float4* dst = reinterpret_cast<float4*>(gw_s + (size_t)r * I);
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(st_s + (size_t)r * sb);
            for (int g = tid; g < gpr; g += kUpdThreads) {
                const float4 gw = __ldg(src + g);
                dst[g] = gw;
                if (WITH_Q) {
                    const uint32_t w = load_group24(raw, (uint32_t)g * 3u);
                    float4 q;
                    q.x = __fmul_rn(gw.x, lut->e[w & 63u].x);
                    q.y = __fmul_rn(gw.y, lut->e[(w >> 6) & 63u].x);
                    q.z = __fmul_rn(gw.z, lut->e[(w >> 12) & 63u].x);
                    q.w = __fmul_rn(gw.w, lut->e[(w >> 18) & 63u].x);
                    reinterpret_cast<float4*>(q_s + (size_t)r * I)[g] = q;
                }
            }
        }
        __syncthreads();

        // ---- stats: warp pair `pair` owns row slot `pair` -------------------------------
        // kernels/compact_counter.cl:73-91: lane-strided accumulation, multiply and add
        // rounded separately, then lg[lid] += lg[lid + s] for s = 32 .. 1.
        float a = 0.0f, b = 0.0f;
        if (pair < nrows) {
            const float4* g4 = reinterpret_cast<const float4*>(gw_s + (size_t)pair * I);
            const float4* q4 = reinterpret_cast<const float4*>(q_s + (size_t)pair * I);
            for (int g = vlane; g < gpr; g += 64) {
                const float4 gw = g4[g];
                a = __fadd_rn(a, __fmul_rn(gw.x, gw.x));
                a = __fadd_rn(a, __fmul_rn(gw.y, gw.y));
                a = __fadd_rn(a, __fmul_rn(gw.z, gw.z));
                a = __fadd_rn(a, __fmul_rn(gw.w, gw.w));
                if (WITH_Q) {
                    const float4 q = q4[g];
                    b = __fadd_rn(b, q.x);
                    b = __fadd_rn(b, q.y);
                    b = __fadd_rn(b, q.z);
                    b = __fadd_rn(b, q.w);
                }
            }
            if (vlane >= 32) {
                part[pair * 64 + lane] = a;
                part[pair * 64 + 32 + lane] = b;
            }
        }
        __syncthreads();
        if (pair < nrows && vlane < 32) {
            a = __fadd_rn(a, part[pair * 64 + lane]);
            b = __fadd_rn(b, part[pair * 64 + 32 + lane]);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) {
                a = __fadd_rn(a, __shfl_down_sync(0xffffffffu, a, s));
                b = __fadd_rn(b, __shfl_down_sync(0xffffffffu, b, s));
            }
            if (lane == 0) {
                // kernels/compact_counter.cl:92-99
                const int row = row0 + pair;
                const float gsq = __fdiv_rn(a, (float)I);
                const float s_old = p.scale[row];
                float s_new;
                if (WITH_Q) {
                    const float gs = __fdiv_rn(b, __fsqrt_rn((float)I));
                    s_new = __fsub_rn(s_old, __fmul_rn(p.lr_scale, gs));
                } else {
                    s_new = s_old;   // lr_scale == 0 and finite statistics: scale - 0 = scale
                }
                s_new = fminf(fmaxf(s_new, 1e-5f), 10.0f);
                const float vv = __fadd_rn(__fmul_rn(p.rms_beta, p.v[row]),
                                           __fmul_rn(__fsub_rn(1.0f, p.rms_beta), gsq));
                p.v[row] = vv;
                RowConst rc;
                rc.dn = fmaxf(__fsqrt_rn(vv), p.rms_eps);
                rc.k_tick = __fdiv_rn(Cf, s_new);
                rc.k_reb = __fdiv_rn(s_old, s_new);
                rc.pad = 0.0f;
                rowc[pair] = rc;
                p.scale[row] = s_new;       // scale commit (kernels/basic.cl:6-9)
            }
        }
        __syncthreads();
        // per-row table of rebased counters (one entry per old code value)
        if (pair < nrows) {
            const float k_reb = rowc[pair].k_reb;
            const float2 tc = lut->e[vlane];
            RowEntry re;
            re.creb = __fmul_rn(tc.y, k_reb);
            const int ti = (int)tc.x + 1;                       // 0..3 for every code the tail table covers
            re.tail_base = (ti >= 0 && ti < 4) ? ti * kTailRow + kTailK : -(1 << 20);
            rowtab[pair * 64 + vlane] = re;
        }
        __syncthreads();

        // ---- tick: one packed group per thread-iteration --------------------------------
        for (int r = 0; r < nrows; ++r) {
            const RowConst rc = rowc[r];
            const float4* g4 = reinterpret_cast<const float4*>(gw_s + (size_t)r * I);
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(st_s + (size_t)r * sb);
            unsigned char* so = so_s + (size_t)r * sb;
            unsigned char* p2 = p2_s + (size_t)r * pb;
            const uint32_t elem_row = (uint32_t)(p.row_offset + row0 + r) * (uint32_t)I;
            const RowEntry* rt = rowtab + r * 64;
            for (int g = tid; g < gpr; g += kUpdThreads) {
                const uint32_t w = load_group24(raw, (uint32_t)g * 3u);
                const float4 gw = g4[g];
                const float gwv[4] = {gw.x, gw.y, gw.z, gw.w};
                uint32_t nw = 0, fields = 0;
                // first round of the element hash: the four indices of a group differ only in
                // their two low bits, so x >> 16 is shared (kernels/compact_counter.cl:17-21)
                const uint32_t e0 = elem_row + (uint32_t)(g * 4);
                const uint32_t e0x = e0 ^ (e0 >> 16);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t code_old = (w >> (6 * k)) & 63u;
                    const RowEntry re = rt[code_old];
                    const float tick = __fmul_rn(__fmul_rn(neg_lr, __fdiv_rn(gwv[k], rc.dn)), rc.k_tick);
                    const float val = __fadd_rn(re.creb, tick);
                    const float f = floorf(val);
                    uint32_t x = (e0x ^ (uint32_t)k) * 0x7feb352du;     // (e0 + k) ^ ((e0 + k) >> 16), e0 % 4 == 0
                    x ^= x >> 15; x *= 0x846ca68bu;
                    x = seed ^ x ^ (x >> 16);
                    const uint32_t h = cc_hash_u32(x) & 0x00ffffffu;
                    const float rnd = __fmul_rn((float)h, 1.0f / 16777216.0f);
                    const int iccv = __float2int_rn(f) + ((rnd < __fsub_rn(val, f)) ? 1 : 0);
                    uint32_t code, fld;
                    // |val| < K-1 bounds floor(val) + {0,1} to the table's range
                    if (fabsf(val) < (float)(kTailK - 1) && (!check_t || re.tail_base >= 0)) {
                        const unsigned e = tail[re.tail_base + iccv];
                        code = e & 0x3Fu;
                        fld = e >> 8;
                    } else {
                        const float2 tc = lut->e[code_old];
                        code = counter_tick(gwv[k], tc.x, tc.y, e0 + (uint32_t)k, seed, neg_lr, rc.dn, rc.k_tick,
                                            rc.k_reb, Cf, p.C, lv, &fld) & 0x3Fu;
                        fld &= 3u;
                    }
                    nw += code << (6 * k);
                    fields += fld << (2 * k);
                }
                so[g * 3 + 0] = (unsigned char)(nw & 0xFFu);
                so[g * 3 + 1] = (unsigned char)((nw >> 8) & 0xFFu);
                so[g * 3 + 2] = (unsigned char)((nw >> 16) & 0xFFu);
                p2[g] = (unsigned char)fields;
            }
        }
        __syncthreads();

        // ---- store ---------------------------------------------------------------------
        for (int r = 0; r < nrows; ++r) {
            uint8_t* dst = p.state + (size_t)(row0 + r) * row_bytes;
            const unsigned char* src = so_s + (size_t)r * sb;
            if (aligned16) {
                const uint4* s4 = reinterpret_cast<const uint4*>(src);
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                for (int i = tid; i < row_bytes / 16; i += kUpdThreads) d4[i] = s4[i];
            } else if (aligned4) {
                const uint32_t* s1 = reinterpret_cast<const uint32_t*>(src);
                uint32_t* d1 = reinterpret_cast<uint32_t*>(dst);
                for (int i = tid; i < row_bytes / 4; i += kUpdThreads) d1[i] = s1[i];
            } else {
                for (int i = tid; i < row_bytes; i += kUpdThreads) dst[i] = src[i];
            }
            if (p.packed2 != nullptr) {   // requires in_features % 16 == 0 (checked by the caller)
                uint32_t* d = p.packed2 + (size_t)(row0 + r) * (I >> 4);
                const unsigned char* s = p2_s + (size_t)r * pb;
                if (aligned16) {
                    const uint4* s4 = reinterpret_cast<const uint4*>(s);
                    uint4* d4 = reinterpret_cast<uint4*>(d);
                    for (int i = tid; i < gpr / 16; i += kUpdThreads) d4[i] = s4[i];
                } else {
                    const uint32_t* s1 = reinterpret_cast<const uint32_t*>(s);
                    for (int i = tid; i < gpr / 4; i += kUpdThreads) d[i] = s1[i];
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// Fast variant for in_features % 16 == 0 (every benchmark shape): same phases, but
//   * a batch holds up to kMaxRowsU16 rows, so narrow layers still give each CTA thousands of
//     weights between barriers; a warp pair walks its rows of the batch one after another and
//     pairs meet on their own named barrier, not a CTA-wide one;
//   * the tick works on units of 16 weights = 3 aligned state words in, 3 state words + one
//     2-bit word out, all 32-bit shared-memory accesses; units of all rows of the batch are
//     flattened over the threads;
//   * the gradient tile in shared memory is XOR-swizzled at 16-byte granularity so that the
//     unit-strided 128-bit reads are bank-conflict free;
//   * the right shifts of the integer hash are issued as mul.hi (FMA pipe) because the ALU
//     pipe is the busiest one in this kernel.
constexpr int kMaxRowsU16 = 64;
#ifndef MCL_UPD_CTAS_PER_SM
#define MCL_UPD_CTAS_PER_SM 4         // resident CTAs per SM the 16-weight kernel is compiled and sized for
#endif
constexpr int kUpdCtasPerSm = MCL_UPD_CTAS_PER_SM;
constexpr int kPairs = kUpdThreads / 64;

__device__ __forceinline__ int swz4(int f) {          // float4 index -> swizzled float4 index
    return (f & ~3) | ((f & 3) ^ ((f >> 3) & 3));
}
__device__ __forceinline__ uint32_t shr_mulhi(uint32_t x, uint32_t pow2) {   // x >> (32 - log2(pow2))
    return pow2 == 65536u ? x >> 16 : x >> 15;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
    float2 v; asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a)); return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_u32(uint32_t a, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

__device__ __forceinline__ float fmax_nan(float a, float b) {          // max that keeps a NaN operand
    float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r;
}

// Per-row constants of the tick (32 bytes).  gw / dn is formed without a division: yh = RN(1 / dn) and
// yl = RN((1 - dn * yh) * yh) make yh + yl equal 1 / dn to ~2^-47, so p = RN(gw * yh + RN(gw * yl)) is one of the
// two floats next to gw / dn, and one residual step  q = RN(p + (gw - dn * p) * yh)  (the residual is exact in an
// FMA) is the correctly rounded quotient -- the value the reference's IEEE division gives (Markstein's theorem:
// a faithful quotient, a reciprocal within 2^-24 relative, one FMA correction).  The argument needs no underflow:
// it holds for dn in [2^-32, 2^32] and |q| >= 2^-64; `qlo` is that bound for rows whose dn is in range and NaN for
// the others, and a unit whose smallest |q| fails  qmin >= qlo  is looked at again and, unless its small quotients
// are exact zeros, redone with the division.
struct RowK {
    float yh, yl, dn, k_tick, k_reb, qlo, pad0, pad1;
};

// Tick table of the 16-weight kernel: for weight position k in its group, old ternary digit t in {-1,0,1,2} and
// rounded counter ccv in [-64, 63]:  new code << 6k  |  (new digit + 1) << (24 + 2k), so that the four look-ups of
// a group ADD UP to its 24-bit state word and its byte of 2-bit fields.
constexpr int kTickN = 128;                      // entries per (k, t)
constexpr int kTickHalf = kTickN / 2;
constexpr int kTickBytes = 4 * 4 * kTickN * 4;   // 8 KiB
constexpr float kTickValMax = (float)(kTickHalf - 2);   // |counter + tick| below this stays inside the table

// The tick of one 16-weight unit (3 state words in, 3 state words and one word of 2-bit fields out), shared by the
// kernels below.  All operands are shared-memory addresses: sa_rowk the row's RowK, rt its 64-entry row table, sw the
// unit's three state words, g4 the first of its four gradient float4s (swizzled by jsw).  e_unit = global element
// index of the unit's first weight.
__device__ __forceinline__ void tick_unit16(const uint32_t sa_rowk, const uint32_t rt, const uint32_t sw, const uint32_t g4,
                                            const uint32_t jsw, const uint32_t e_unit, const uint32_t seed, const float neg_lr,
                                            const float Cf, const int C, const int lv, const uint32_t pow16,
                                            const uint32_t pow17, const DecodeLut* lut, uint32_t (&nwd)[4], uint32_t& fields) {
    const float4 rcv = lds_f4(sa_rowk);            // yh, yl, dn, k_tick
    const float2 rcw = lds_f2(sa_rowk + 16u);      // k_reb, qlo
    const float ndn = -rcv.z;
    const uint32_t s0 = lds_u32(sw), s1 = lds_u32(sw + 4), s2 = lds_u32(sw + 8);
    const uint32_t gwd[4] = {s0 & 0xFFFFFFu, (s0 >> 24) | ((s1 & 0xFFFFu) << 8),
                             (s1 >> 16) | ((s2 & 0xFFu) << 16), s2 >> 8};
    fields = 0;
    float vmax = 0.0f;                              // largest |counter + tick| of the unit (NaN if any is)
    float qmin = __int_as_float(0x7f800000);        // smallest |gw / dn| of the unit
#pragma unroll
    for (int gg = 0; gg < 4; ++gg) {
        const float4 gw = lds_f4(g4 + (((uint32_t)gg ^ jsw) << 4));
        const float gwv[4] = {gw.x, gw.y, gw.z, gw.w};
        const uint32_t w = gwd[gg];
        const uint32_t e0 = e_unit + 4u * gg;
        const uint32_t e0x = e0 ^ shr_mulhi(e0, pow16);
        uint32_t acc = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // byte offset of the row-table entry of the old code: code * 8
            const uint32_t c8 = (k == 0 ? (w << 3) : (w >> (6 * k - 3))) & 0x1F8u;
            const float2 re = lds_f2(rt + c8);            // x = rebased counter, y = tick-table address (int bits)
            const float g = gwv[k];
            const float pq = __fmaf_rn(g, rcv.x, __fmul_rn(g, rcv.y));
            const float q = __fmaf_rn(__fmaf_rn(ndn, pq, g), rcv.x, pq);      // = RN(g / dn), see RowK
            qmin = fminf(qmin, fabsf(q));
            const float tick = __fmul_rn(__fmul_rn(neg_lr, q), rcv.w);
            const float val = __fadd_rn(re.x, tick);
            vmax = fmax_nan(vmax, fabsf(val));
            uint32_t x = (e0x ^ (uint32_t)k) * 0x7feb352du;
            x ^= shr_mulhi(x, pow17);            // x >> 15
            x *= 0x846ca68bu;
            x = seed ^ x ^ shr_mulhi(x, pow16);  // seed ^ hash(elem)
            x ^= shr_mulhi(x, pow16);
            x *= 0x7feb352du;
            x ^= shr_mulhi(x, pow17);
            x *= 0x846ca68bu;
            const uint32_t h = (x ^ shr_mulhi(x, pow16)) & 0x00ffffffu;
            const float f = floorf(val);
            const float rnd = __fmul_rn((float)h, 1.0f / 16777216.0f);
            int iccv;           // saturating conversion: a wild value still gives an address inside this CTA's shared memory
            asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(iccv) : "f"(f));
            iccv += (rnd < __fsub_rn(val, f)) ? 1 : 0;
            acc += lds_u32((uint32_t)(__float_as_int(re.y) + 4 * iccv) + (uint32_t)(k * 4 * kTickN * 4));
        }
        nwd[gg] = acc & 0xFFFFFFu;
        fields |= (acc >> 24) << (8 * gg);
    }
    bool redo = !(vmax < kTickValMax);      // a rounded counter beyond the table, a code outside it, or a NaN
    if (!(qmin >= rcw.y)) {
        // a quotient below the range in which the division-free form is proven (or a row outside it): exact
        // zeros are fine, anything else goes to the formulas
        redo = redo || (rcw.y != rcw.y);
        for (int gg = 0; gg < 4 && !redo; ++gg) {
            const float4 gw = lds_f4(g4 + (((uint32_t)gg ^ jsw) << 4));
            const float gwv[4] = {gw.x, gw.y, gw.z, gw.w};
            for (int k = 0; k < 4; ++k)
                if (gwv[k] != 0.0f && !(fabsf(__fdiv_rn(gwv[k], rcv.z)) >= rcw.y)) redo = true;
        }
    }
    if (redo) {
        // rare: redo the unit with the reference formulas
        fields = 0;
        for (int gg = 0; gg < 4; ++gg) {
            const float4 gw = lds_f4(g4 + (((uint32_t)gg ^ jsw) << 4));
            const float gwv[4] = {gw.x, gw.y, gw.z, gw.w};
            uint32_t nw = 0;
            for (int k = 0; k < 4; ++k) {
                const float2 tc = lut->e[(gwd[gg] >> (6 * k)) & 63u];
                uint32_t fld;
                const uint32_t code = counter_tick(gwv[k], tc.x, tc.y, e_unit + (uint32_t)(4 * gg + k), seed,
                                                   neg_lr, rcv.z, rcv.w, rcw.x, Cf, C, lv, &fld);
                nw += (code & 0x3Fu) << (6 * k);
                fields += (fld & 3u) << (2 * (4 * gg + k));
            }
            nwd[gg] = nw;
        }
    }
}

// kernels/compact_counter.cl:129-136 evaluated for every (old digit, rounded counter) the table covers
__device__ __forceinline__ void build_tick_table(uint32_t* tick_tab, const int C, const int tid, const int nthreads) {
    const int lv = 2 * C - 1;
    const float Cf = (float)C;
    for (int e = tid; e < 4 * kTickN; e += nthreads) {
        const int t = e / kTickN - 1;
        const float ccv = (float)(e % kTickN - kTickHalf);
        const float carry = truncf(__fdiv_rn(ccv, Cf));
        float rem = __fsub_rn(ccv, __fmul_rn(carry, Cf));
        const int nt = t + (int)carry;
        const int ct = nt < -1 ? -1 : (nt > 1 ? 1 : nt);
        if (ct != nt) rem = __fmul_rn(ccv > 0.0f ? 1.0f : (ccv < 0.0f ? -1.0f : 0.0f), __fsub_rn(Cf, 1.0f));
        int ri = (int)rem;
        ri = ri < -(C - 1) ? -(C - 1) : (ri > C - 1 ? C - 1 : ri);
        const uint32_t code = (uint32_t)(((ct + 1) * lv + (ri + (C - 1))) & 0x3F);
        const uint32_t fld = (uint32_t)(ct + 1);
#pragma unroll
        for (int k = 0; k < 4; ++k) tick_tab[k * 4 * kTickN + e] = (code << (6 * k)) | (fld << (24 + 2 * k));
    }
}

// Row constants from the two row sums (kernels/compact_counter.cl:92-99); writes v and the new scale of the row.
template <bool WITH_Q>
__device__ __forceinline__ RowK finish_row_stats(const UpdParams& p, const int row, const float a, const float b, const float Cf,
                                                 const float s_old, const float v_old) {
    const int I = p.in_features;
    const float gsq = __fdiv_rn(a, (float)I);
    float s_new = s_old;
    if (WITH_Q) {
        const float gs = __fdiv_rn(b, __fsqrt_rn((float)I));
        s_new = __fsub_rn(s_old, __fmul_rn(p.lr_scale, gs));
    }
    s_new = fminf(fmaxf(s_new, 1e-5f), 10.0f);
    const float vv = __fadd_rn(__fmul_rn(p.rms_beta, v_old), __fmul_rn(__fsub_rn(1.0f, p.rms_beta), gsq));
    p.v[row] = vv;
    RowK rc;
    rc.dn = fmaxf(__fsqrt_rn(vv), p.rms_eps);
    rc.k_tick = __fdiv_rn(Cf, s_new);
    rc.k_reb = __fdiv_rn(s_old, s_new);
    rc.yh = __frcp_rn(rc.dn);
    rc.yl = __fmul_rn(__fmaf_rn(-rc.dn, rc.yh, 1.0f), rc.yh);
    const bool in_range = rc.dn >= 2.3283064365386963e-10f && rc.dn <= 4294967296.0f;     // 2^-32 .. 2^32
    rc.qlo = in_range ? 5.421010862427522e-20f : __int_as_float(0x7fc00000);                 // 2^-64 or NaN
    rc.pad0 = rc.pad1 = 0.0f;
    p.scale[row] = s_new;           // scale commit (kernels/basic.cl:6-9)
    return rc;
}

// Row-table entry of old code value `code`: the rebased counter and the shared-memory address of the tick-table entry
// of (k = 0, the code's digit, rounded counter 0).  A code whose ternary digit the tick table lacks gets an infinite
// counter, which sends its unit down the formula path.
__device__ __forceinline__ RowEntry row_entry(const DecodeLut* lut, const int code, const float k_reb, const uint32_t sa_tick) {
    const float2 tc = lut->e[code];
    const int ti = (int)tc.x + 1;
    const bool ok = ti >= 0 && ti < 4;
    RowEntry re;
    re.creb = ok ? __fmul_rn(tc.y, k_reb) : __int_as_float(0x7f800000);
    re.tail_base = (int)(sa_tick + 4u * (uint32_t)((ok ? ti : 0) * kTickN + kTickHalf));
    return re;
}

struct U16Layout {
    int sb, off_tick, off_rowc, off_part, off_rowtab, off_gw, off_st, off_so, off_p2;
    size_t total;
};
__host__ __device__ inline U16Layout u16_layout(int I, int R, bool with_q) {
    (void)with_q;
    U16Layout L;
    const int row_bytes = (I >> 2) * 3;
    L.sb = (row_bytes + 15) & ~15;
    size_t o = sizeof(DecodeLut);
    L.off_tick = (int)o; o += kTickBytes;
    L.off_rowc = (int)o; o += sizeof(RowK) * R;
    L.off_part = (int)o; o += sizeof(float) * 64 * kPairs;
    L.off_rowtab = (int)o; o += sizeof(RowEntry) * 64 * (size_t)R;
    L.off_gw = (int)o; o += sizeof(float) * (size_t)R * I;
    L.off_st = (int)o; o += (size_t)R * L.sb + 16;
    L.off_so = (int)o; o += (size_t)R * L.sb + 16;
    L.off_p2 = (int)o; o += (size_t)R * (I >> 2);
    L.total = (o + 15) & ~size_t(15);
    return L;
}

// Body shared by the single-layer and the grouped kernel: batches batch0, batch0 + batch_step, ... of the
// layer `p`.  The decode and tick tables depend on C alone; `build_tables` is false when an earlier call
// of the same CTA already built them for this C.
template <bool WITH_Q>
__device__ __forceinline__ void update_u16_body(const UpdParams& p, const uint32_t unit_magic, const uint32_t pow16,
                                                const uint32_t pow17, const int batch0, const int batch_step,
                                                const bool build_tables) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int I = p.in_features;
    const int gpr = I >> 2;               // packed groups (float4s) per row
    const int upr = I >> 4;               // 16-weight units per row
    const int row_bytes = gpr * 3;
    const int R = p.rows_per_batch;
    const U16Layout L = u16_layout(I, R, WITH_Q);

    DecodeLut* lut = reinterpret_cast<DecodeLut*>(smem);
    uint32_t* tick_tab = reinterpret_cast<uint32_t*>(smem + L.off_tick);
    RowK* rowc = reinterpret_cast<RowK*>(smem + L.off_rowc);
    float* part = reinterpret_cast<float*>(smem + L.off_part);
    RowEntry* rowtab = reinterpret_cast<RowEntry*>(smem + L.off_rowtab);
    float4* gw_s = reinterpret_cast<float4*>(smem + L.off_gw);
    unsigned char* st_s = smem + L.off_st;
    unsigned char* so_s = smem + L.off_so;
    uint32_t* p2_s = reinterpret_cast<uint32_t*>(smem + L.off_p2);
    const uint32_t sa0 = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sa_tick = sa0 + L.off_tick, sa_rowc = sa0 + L.off_rowc, sa_rowtab = sa0 + L.off_rowtab;
    const uint32_t sa_gw = sa0 + L.off_gw, sa_st = sa0 + L.off_st, sa_so = sa0 + L.off_so, sa_p2 = sa0 + L.off_p2;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int pair = tid >> 6;
    const int vlane = tid & 63;
    const int lv = 2 * p.C - 1;
    const float Cf = (float)p.C;
    const float neg_lr = -p.lr;
    const uint32_t seed = p.seed + (p.seed_offset ? __ldg(p.seed_offset) : 0u);
    const bool aligned16 = p.state_align >= 16;

    if (build_tables) {
        __syncthreads();                  // an earlier layer's batches may still read the old tables
        build_decode_lut(lut, p.C, tid, kUpdThreads);
        build_tick_table(tick_tab, p.C, tid, kUpdThreads);
    }
    __syncthreads();

    const int nbatches = (p.rows + R - 1) / R;
    for (int batch = batch0; batch < nbatches; batch += batch_step) {
        const int row0 = batch * R;
        const int nrows = min(R, p.rows - row0);

        // ---- load: the batch's rows are contiguous in global memory ------------------------
        {
            const uint8_t* src = p.state + (size_t)row0 * row_bytes;
            if (aligned16) {        // row_bytes % 16 == 0: one flat copy, smem row stride == row_bytes
                const uint4* s4 = reinterpret_cast<const uint4*>(src);
                uint4* d4 = reinterpret_cast<uint4*>(st_s);
                for (int i = tid; i < nrows * (row_bytes >> 4); i += kUpdThreads) d4[i] = __ldg(s4 + i);
            } else {                // rows are 4-byte aligned; smem rows padded to L.sb
                const uint32_t* s1 = reinterpret_cast<const uint32_t*>(src);
                const int wpr = row_bytes >> 2;
                for (int i = tid; i < nrows * wpr; i += kUpdThreads) {
                    const int r = i / wpr, w = i - r * wpr;
                    reinterpret_cast<uint32_t*>(st_s + (size_t)r * L.sb)[w] = __ldg(s1 + i);
                }
            }
            const float4* gsrc = reinterpret_cast<const float4*>(p.grad_w + (size_t)row0 * I);
            const int n4 = nrows * gpr;
            if ((gpr & 31) == 0) {  // rows start on a period of the swizzle: the flat float4 index can be swizzled as it is
                int i = tid;
                for (; i + 3 * kUpdThreads < n4; i += 4 * kUpdThreads) {       // four loads in flight per thread
                    const float4 v0 = __ldg(gsrc + i), v1 = __ldg(gsrc + i + kUpdThreads), v2 = __ldg(gsrc + i + 2 * kUpdThreads),
                                 v3 = __ldg(gsrc + i + 3 * kUpdThreads);
                    gw_s[swz4(i)] = v0; gw_s[swz4(i + kUpdThreads)] = v1;
                    gw_s[swz4(i + 2 * kUpdThreads)] = v2; gw_s[swz4(i + 3 * kUpdThreads)] = v3;
                }
                for (; i < n4; i += kUpdThreads) gw_s[swz4(i)] = __ldg(gsrc + i);
            } else {                // flat over the batch; row = i / gpr by multiply-high (gpr = 4 * units per row)
                for (int i = tid; i < n4; i += kUpdThreads) {
                    const int r = unit_magic ? (int)__umulhi((uint32_t)i >> 2, unit_magic) : (i >> 2);
                    const int g = i - r * gpr;
                    gw_s[r * gpr + swz4(g)] = __ldg(gsrc + i);
                }
            }
        }
        __syncthreads();

        // ---- stats: warp pair `pair` walks rows pair, pair + kPairs, ... ---------------------
        for (int r = pair; r < nrows; r += kPairs) {
            float a = 0.0f, b = 0.0f;
            const float4* g4 = gw_s + r * gpr;
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(st_s + (size_t)r * L.sb);
            for (int g = vlane; g < gpr; g += 64) {
                const float4 gw = g4[swz4(g)];
                a = __fadd_rn(a, __fmul_rn(gw.x, gw.x));
                a = __fadd_rn(a, __fmul_rn(gw.y, gw.y));
                a = __fadd_rn(a, __fmul_rn(gw.z, gw.z));
                a = __fadd_rn(a, __fmul_rn(gw.w, gw.w));
                if (WITH_Q) {
                    const uint32_t w = load_group24(raw, (uint32_t)g * 3u);
                    b = __fadd_rn(b, __fmul_rn(gw.x, lut->e[w & 63u].x));
                    b = __fadd_rn(b, __fmul_rn(gw.y, lut->e[(w >> 6) & 63u].x));
                    b = __fadd_rn(b, __fmul_rn(gw.z, lut->e[(w >> 12) & 63u].x));
                    b = __fadd_rn(b, __fmul_rn(gw.w, lut->e[(w >> 18) & 63u].x));
                }
            }
            if (vlane >= 32) {
                part[pair * 64 + lane] = a;
                part[pair * 64 + 32 + lane] = b;
            }
            asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
            if (vlane < 32) {
                a = __fadd_rn(a, part[pair * 64 + lane]);
                b = __fadd_rn(b, part[pair * 64 + 32 + lane]);
#pragma unroll
                for (int s = 16; s > 0; s >>= 1) {
                    a = __fadd_rn(a, __shfl_down_sync(0xffffffffu, a, s));
                    b = __fadd_rn(b, __shfl_down_sync(0xffffffffu, b, s));
                }
                if (lane == 0) rowc[r] = finish_row_stats<WITH_Q>(p, row0 + r, a, b, Cf, p.scale[row0 + r], p.v[row0 + r]);
            }
            asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
            rowtab[r * 64 + vlane] = row_entry(lut, vlane, rowc[r].k_reb, sa_tick);     // one entry per old code value
        }
        __syncthreads();

        // ---- tick: 16 weights per thread-iteration, units of the whole batch flattened --------
        // Shared memory is addressed with 32-bit shared-space addresses (ld.shared / st.shared), which
        // keeps the address arithmetic of the data-dependent table look-ups to one add each.
        const int nunits = nrows * upr;
        for (int u = tid; u < nunits; u += kUpdThreads) {
            const int r = unit_magic ? (int)__umulhi((uint32_t)u, unit_magic) : u;       // u / upr (magic 0: upr == 1)
            const int j = u - r * upr;
            const uint32_t g4 = sa_gw + ((uint32_t)(r * gpr + 4 * j) << 4);
            const uint32_t e_unit = (uint32_t)(p.row_offset + row0 + r) * (uint32_t)I + (uint32_t)(16 * j);
            uint32_t nwd[4], fields;
            tick_unit16(sa_rowc + (uint32_t)r * 32u, sa_rowtab + (uint32_t)r * 512u,
                        sa_st + (uint32_t)r * (uint32_t)L.sb + 12u * (uint32_t)j, g4, (uint32_t)((j >> 1) & 3), e_unit, seed,
                        neg_lr, Cf, p.C, lv, pow16, pow17, lut, nwd, fields);
            const uint32_t so = sa_so + (uint32_t)r * (uint32_t)L.sb + 12u * (uint32_t)j;
            sts_u32(so, nwd[0] | (nwd[1] << 24));
            sts_u32(so + 4, (nwd[1] >> 8) | (nwd[2] << 16));
            sts_u32(so + 8, (nwd[2] >> 16) | (nwd[3] << 8));
            sts_u32(sa_p2 + 4u * (uint32_t)(r * upr + j), fields);
        }
        __syncthreads();

        // ---- store (the next batch's loads follow without a barrier: they touch other arrays) ------------
        {
            uint8_t* dst = p.state + (size_t)row0 * row_bytes;
            if (aligned16) {
                const uint4* s4 = reinterpret_cast<const uint4*>(so_s);
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                for (int i = tid; i < nrows * (row_bytes >> 4); i += kUpdThreads) d4[i] = s4[i];
            } else {
                uint32_t* d1 = reinterpret_cast<uint32_t*>(dst);
                const int wpr = row_bytes >> 2;
                for (int i = tid; i < nrows * wpr; i += kUpdThreads) {
                    const int r = i / wpr, w = i - r * wpr;
                    d1[i] = reinterpret_cast<const uint32_t*>(so_s + (size_t)r * L.sb)[w];
                }
            }
            if (p.packed2 != nullptr) {
                uint32_t* d = p.packed2 + (size_t)row0 * upr;
                if (aligned16) {
                    const uint4* s4 = reinterpret_cast<const uint4*>(p2_s);
                    uint4* d4 = reinterpret_cast<uint4*>(d);
                    for (int i = tid; i < (nrows * upr) >> 2; i += kUpdThreads) d4[i] = s4[i];
                } else {
                    for (int i = tid; i < nrows * upr; i += kUpdThreads) d[i] = p2_s[i];
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Wide rows (in_features >= 1024, a multiple of 64): one persistent CTA per SM whose warps have ROLES, so that the
// latency of HBM, the row statistics (64 lanes of parallelism per row, by the reference's reduction order) and the
// tick (everything else) overlap instead of taking turns between CTA-wide barriers.
//   ring     D row slots in shared memory: gradient row (XOR-swizzled float4s), state row, row table, row constants
//   stats    every fourth warp (one scheduler's worth).  Stats warp s owns the CTA's rows s, s + S, ...  For a row it
//            waits until the slot's previous row has been ticked, copies gradient, state, scale and v into the slot with
//            cp.async, replays the 64-lane reduction with two virtual lanes per thread, writes v / scale / the row's
//            constants and its table, and marks the slot ready.  The warps take turns, so S rows are in flight.
//   tick     the other warps: chunks of 32 consecutive 16-weight units, dealt round-robin across rows.  A lane ticks
//            one unit, writes the new state words over the old ones in the slot, the warp copies its 384 bytes out
//            with 16-byte stores and stores its 32 words of 2-bit fields; a warp that has passed a row releases its slot.
// Measured on B200 (8192 x 4096 fp32 gradient, CUDA events): 1.95 TB/s = 0.30 of the copy bandwidth; the kernel issues
// ~55 instructions per weight (two 32-bit hashes, the quotient, floor / compare / two table look-ups), which at four
// instructions per clock and SM bounds it near 0.55 whatever the memory system does.
// Every wait is bounded: on time-out the kernel sets *err (when given) and all roles leave.
constexpr int kWsThreads = 512;
// Every fourth warp is a stats warp: warps are dealt to the SM's four schedulers by warp number, so the stats warps
// share ONE scheduler among themselves and their short dependent instruction chains do not queue behind the tick
// warps' long independent ones.
constexpr int kWsStatsWarps = kWsThreads / 128;
constexpr int kWsTickWarps = kWsThreads / 32 - kWsStatsWarps;
constexpr int kWsMaxSlots = 16;
constexpr int kWsErrCode = 21;

struct WsLayout {
    int off_tick, off_bars, off_ring, slot_bytes, off_st, off_rowtab, off_rowk, off_sv, nslots;
    size_t total;
};
__host__ __device__ inline WsLayout ws_layout(int I, size_t max_smem) {
    WsLayout L;
    size_t o = sizeof(DecodeLut);
    L.off_tick = (int)o; o += kTickBytes;
    L.off_bars = (int)o; o += 8 * 2 * kWsMaxSlots + 16;
    o = (o + 127) & ~size_t(127);
    L.off_ring = (int)o;
    const int row_bytes = (I >> 2) * 3;
    L.off_st = 4 * I;
    L.off_rowtab = L.off_st + ((row_bytes + 15) & ~15) + 16;      // 16 readable bytes after the state row (24-bit group loads)
    L.off_rowk = L.off_rowtab + 64 * (int)sizeof(RowEntry);
    L.off_sv = L.off_rowk + (int)sizeof(RowK);          // the row's old scale and v, copied in with the row
    L.slot_bytes = (L.off_sv + 16 + 127) & ~127;
    long long n = ((long long)max_smem - 1024 - (long long)o) / L.slot_bytes;
    L.nslots = n > kWsMaxSlots ? kWsMaxSlots : (int)n;
    L.total = o + (size_t)(L.nslots > 0 ? L.nslots : 0) * L.slot_bytes;
    return L;
}

// Bounded wait of a whole warp on an mbarrier phase, polled by one lane that SLEEPS between polls: the waiting roles of
// this kernel share their schedulers with the warps that do the arithmetic, and a hot poll loop costs those warps
// issue slots.  Returns false after ~0.5 s or once another role has flagged an abort.
__device__ __forceinline__ bool ws_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0 && !mbar_try_wait(bar, parity)) {
        const unsigned long long t0 = clock64();
        unsigned spins = 0;
        for (;;) {
            __nanosleep(spins < 8 ? 64 : 256);
            if (mbar_try_wait(bar, parity)) break;
            if ((++spins & 0x3Fu) == 0 && (*abort_flag || clock64() - t0 > kWaitCycles)) { ok = false; break; }
        }
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (ok) ok = mbar_try_wait(bar, parity);      // completed phase: every lane takes its own acquire
    return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}


template <bool WITH_Q>
__global__ void __launch_bounds__(kWsThreads, 1)
counter_update_ws_kernel(const UpdParams p, const uint32_t pow16, const uint32_t pow17, const int nslots, int* err) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int I = p.in_features;
    const int gpr = I >> 2, upr = I >> 4, row_bytes = gpr * 3;
    const WsLayout L = ws_layout(I, 0);
    DecodeLut* lut = reinterpret_cast<DecodeLut*>(smem);
    uint32_t* tick_tab = reinterpret_cast<uint32_t*>(smem + L.off_tick);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.off_bars + 8 * 2 * kWsMaxSlots);
    const uint32_t sa0 = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sa_tick = sa0 + L.off_tick, sa_ring = sa0 + L.off_ring, bar0 = sa0 + L.off_bars;
    auto ready_bar = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto free_bar = [&](int s) { return bar0 + 8u * (uint32_t)(kWsMaxSlots + s); };

    const int tid = threadIdx.x, hw_warp = tid >> 5, lane = tid & 31;
    const bool is_stats = (hw_warp & 3) == 0;
    const int warp = is_stats ? (hw_warp >> 2) : kWsStatsWarps + hw_warp - (hw_warp >> 2) - 1;     // role index: stats warps first
    const int lv = 2 * p.C - 1;
    const float Cf = (float)p.C;
    const float neg_lr = -p.lr;
    const uint32_t seed = p.seed + (p.seed_offset ? __ldg(p.seed_offset) : 0u);
    const int D = nslots;

    // this CTA's rows: a contiguous block
    const int r_begin = (int)(((long long)p.rows * blockIdx.x) / gridDim.x);
    const int r_end = (int)(((long long)p.rows * (blockIdx.x + 1)) / gridDim.x);
    const int nrows = r_end - r_begin;

    if (tid == 0) {
        *abort_flag = (err != nullptr && *reinterpret_cast<volatile int*>(err) != 0) ? 1 : 0;
        for (int s = 0; s < D; ++s) { mbar_init(ready_bar(s), 32); mbar_init(free_bar(s), kWsTickWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    build_decode_lut(lut, p.C, tid, kWsThreads);
    build_tick_table(tick_tab, p.C, tid, kWsThreads);
    __syncthreads();
    auto give_up = [&]() {
        *abort_flag = 1;
        if (err != nullptr) atomicExch(err, kWsErrCode);
    };

    // A slot is refilled by whichever stats warp owns the row D rows later; the wait on the slot's "free" barrier tells
    // apart only two consecutive uses, so a warp must never get two uses ahead of the ring: with S warps striding the
    // rows by S, that holds when S <= D.  Fewer slots than stats warps (very wide rows): the surplus warps sit out.
    const int S = kWsStatsWarps < D ? kWsStatsWarps : D;
    if (warp < kWsStatsWarps) {
        // ---- stats warps ---------------------------------------------------------------------------
        auto issue = [&](int n) -> bool {       // copies of local row n into its slot; false: gave up
            const int slot = n % D;
            if (!ws_wait(free_bar(slot), (((uint32_t)(n / D)) & 1u) ^ 1u, abort_flag)) return false;
            const uint32_t base = sa_ring + (uint32_t)slot * (uint32_t)L.slot_bytes;
            const float4* gsrc = reinterpret_cast<const float4*>(p.grad_w + (size_t)(r_begin + n) * I);
            for (int g = lane; g < gpr; g += 32) cp_async16(base + ((uint32_t)swz4(g) << 4), gsrc + g);
            const uint4* ssrc = reinterpret_cast<const uint4*>(p.state + (size_t)(r_begin + n) * row_bytes);
            for (int c = lane; c < (row_bytes >> 4); c += 32) cp_async16(base + (uint32_t)L.off_st + ((uint32_t)c << 4), ssrc + c);
            if (lane < 2) {
                const float* src = (lane == 0 ? p.scale : p.v) + (r_begin + n);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(base + (uint32_t)L.off_sv + 4u * (uint32_t)lane), "l"(src) : "memory");
            }
            return true;
        };
        // Several rows are in flight per SM because the stats warps take turns; a warp itself copies one row in, waits
        // for it and works on it (issuing the next row's copies earlier was measured no faster: the warp would then
        // wait for a free slot while its current row keeps the tick warps waiting).
        bool ok = true;
        for (int n = warp < S ? warp : nrows; n < nrows && ok; n += S) {
            ok = issue(n);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (!ok) break;
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
            const int slot = n % D;
            unsigned char* sbase = smem + L.off_ring + (size_t)slot * L.slot_bytes;
            const float4* g4 = reinterpret_cast<const float4*>(sbase);
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(sbase + L.off_st);
            // lane l stands for the reference's work-items l and l + 32 (kernels/compact_counter.cl:73-91): item l walks
            // groups l, l + 64, ..., item l + 32 walks l + 32, l + 96, ...
            float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
            for (int g = lane; g < gpr; g += 64) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int gg = g + 32 * h;
                    if (gg < gpr) {
                        const float4 gw = g4[swz4(gg)];
                        float& a = h ? a1 : a0;
                        a = __fadd_rn(a, __fmul_rn(gw.x, gw.x));
                        a = __fadd_rn(a, __fmul_rn(gw.y, gw.y));
                        a = __fadd_rn(a, __fmul_rn(gw.z, gw.z));
                        a = __fadd_rn(a, __fmul_rn(gw.w, gw.w));
                        if (WITH_Q) {
                            const uint32_t w = load_group24(raw, (uint32_t)gg * 3u);
                            float& b = h ? b1 : b0;
                            b = __fadd_rn(b, __fmul_rn(gw.x, lut->e[w & 63u].x));
                            b = __fadd_rn(b, __fmul_rn(gw.y, lut->e[(w >> 6) & 63u].x));
                            b = __fadd_rn(b, __fmul_rn(gw.z, lut->e[(w >> 12) & 63u].x));
                            b = __fadd_rn(b, __fmul_rn(gw.w, lut->e[(w >> 18) & 63u].x));
                        }
                    }
                }
            }
            float a = __fadd_rn(a0, a1), b = __fadd_rn(b0, b1);       // tree step 32
#pragma unroll
            for (int s2 = 16; s2 > 0; s2 >>= 1) {
                a = __fadd_rn(a, __shfl_down_sync(0xffffffffu, a, s2));
                b = __fadd_rn(b, __shfl_down_sync(0xffffffffu, b, s2));
            }
            RowK rc;
            if (lane == 0) {
                const float* sv = reinterpret_cast<const float*>(sbase + L.off_sv);
                rc = finish_row_stats<WITH_Q>(p, r_begin + n, a, b, Cf, sv[0], sv[1]);
                *reinterpret_cast<RowK*>(sbase + L.off_rowk) = rc;
            }
            const float k_reb = __shfl_sync(0xffffffffu, rc.k_reb, 0);
            RowEntry* rowtab = reinterpret_cast<RowEntry*>(sbase + L.off_rowtab);
            rowtab[lane] = row_entry(lut, lane, k_reb, sa_tick);
            rowtab[lane + 32] = row_entry(lut, lane + 32, k_reb, sa_tick);
            mbar_arrive(ready_bar(slot));          // 32 arrivals complete the phase: each lane publishes its own writes
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (!ok && lane == 0) give_up();
    } else {
        // ---- tick warps ------------------------------------------------------------------------------
        const int tw = warp - kWsStatsWarps;
        const int cpr = (upr + 31) >> 5;                     // chunks of 32 units per row
        int released = 0;                                    // rows [0, released) this warp has let go
        bool ok = true;
        // chunk number G = tw, tw + T, ... as (row n, chunk c of the row), advanced without a division
        const int step_n = kWsTickWarps / cpr, step_c = kWsTickWarps - step_n * cpr;
        int n = tw / cpr, c = tw - n * cpr;
        for (; n < nrows && ok; n += step_n, c += step_c) {
            if (c >= cpr) { c -= cpr; ++n; if (n >= nrows) break; }
            if (released < n) {
                __syncwarp();
                if (lane == 0)
                    for (; released < n; ++released) mbar_arrive(free_bar(released % D));
                released = n;
            }
            const int slot = n % D;
            if (!ws_wait(ready_bar(slot), ((uint32_t)(n / D)) & 1u, abort_flag)) { ok = false; break; }
            const uint32_t base = sa_ring + (uint32_t)slot * (uint32_t)L.slot_bytes;
            const int j = c * 32 + lane;
            const int row = r_begin + n;
            uint32_t fields = 0;
            if (j < upr) {
                uint32_t nwd[4];
                const uint32_t sw = base + (uint32_t)L.off_st + 12u * (uint32_t)j;
                tick_unit16(base + (uint32_t)L.off_rowk, base + (uint32_t)L.off_rowtab, sw, base + ((uint32_t)(4 * j) << 4),
                            (uint32_t)((j >> 1) & 3), (uint32_t)(p.row_offset + row) * (uint32_t)I + (uint32_t)(16 * j), seed,
                            neg_lr, Cf, p.C, lv, pow16, pow17, lut, nwd, fields);
                sts_u32(sw, nwd[0] | (nwd[1] << 24));            // over the old words: only this lane reads them
                sts_u32(sw + 4, (nwd[1] >> 8) | (nwd[2] << 16));
                sts_u32(sw + 8, (nwd[2] >> 16) | (nwd[3] << 8));
                if (p.packed2 != nullptr) p.packed2[(size_t)row * upr + j] = fields;
            }
            __syncwarp();
            // the chunk's 384 bytes of state, 16 bytes per lane
            const int nbytes = min(32, upr - c * 32) * 12;
            if (lane * 16 < nbytes) {
                const uint4 v = *reinterpret_cast<const uint4*>(smem + L.off_ring + (size_t)slot * L.slot_bytes + L.off_st +
                                                                (size_t)c * 384 + (size_t)lane * 16);
                *reinterpret_cast<uint4*>(p.state + (size_t)row * row_bytes + (size_t)c * 384 + (size_t)lane * 16) = v;
            }
        }
        __syncwarp();
        if (ok) {
            if (lane == 0)
                for (; released < nrows; ++released) mbar_arrive(free_bar(released % D));
        } else if (lane == 0) {
            give_up();
        }
    }
}

template <bool WITH_Q>
__global__ void __launch_bounds__(kUpdThreads, kUpdCtasPerSm)
counter_update_u16_kernel(const UpdParams p, const uint32_t unit_magic, const uint32_t pow16, const uint32_t pow17) {
    update_u16_body<WITH_Q>(p, unit_magic, pow16, pow17, blockIdx.x, gridDim.x, true);
}

// Several layers in one launch: their batches form one sequence that is dealt round-robin to the CTAs.
constexpr int kUpdGroupCap = 64;
struct UpdGroup {
    int n;
    int batch_begin[kUpdGroupCap + 1];
    uint32_t magic[kUpdGroupCap];
    UpdParams p[kUpdGroupCap];
};
template <bool WITH_Q>
__global__ void __launch_bounds__(kUpdThreads, kUpdCtasPerSm)
counter_update_u16_group_kernel(const __grid_constant__ UpdGroup g, const uint32_t pow16, const uint32_t pow17) {
    const int grid = (int)gridDim.x, b = (int)blockIdx.x;
    int built_c = -1;
    for (int j = 0; j < g.n; ++j) {
        // first batch of layer j whose global index is congruent to this CTA
        int first = (b - g.batch_begin[j]) % grid;
        if (first < 0) first += grid;
        if (first >= g.batch_begin[j + 1] - g.batch_begin[j]) continue;
        update_u16_body<WITH_Q>(g.p[j], g.magic[j], pow16, pow17, first, grid, g.p[j].C != built_c);
        built_c = g.p[j].C;
    }
}

size_t upd_smem_bytes(int I, int R, bool with_q) {
    const int gpr = I / 4;
    const size_t sb = (size_t)((gpr * 3 + 15) & ~15) + 16;
    const size_t pb = (size_t)((gpr + 15) & ~15);
    return sizeof(DecodeLut) + sizeof(RowConst) * kMaxRowsPerBatch + sizeof(float) * 64 * kMaxRowsPerBatch +
           sizeof(RowEntry) * 64 * kMaxRowsPerBatch + sizeof(unsigned short) * ((4 * kTailRow + 7) & ~7) +
           (size_t)R * I * sizeof(float) * (with_q ? 2 : 1) + (size_t)R * (2 * sb + pb);
}

// ---- decode to dense fp32 (kernels/compact_counter.cl:39-55) and 2-bit pack --------------
__global__ void decode_weight_kernel(const uint8_t* __restrict__ state, const float* __restrict__ scale,
                                     float* __restrict__ w, int C, int in_features, long long n_groups) {
    __shared__ DecodeLut lut;
    build_decode_lut(&lut, C, threadIdx.x, blockDim.x);
    __syncthreads();
    const int gpr = in_features >> 2;
    for (long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x; gid < n_groups;
         gid += (long long)gridDim.x * blockDim.x) {
        const long long row = gid / gpr;
        const uint8_t* s = state + gid * 3;
        const uint32_t wd = (uint32_t)__ldg(s) | ((uint32_t)__ldg(s + 1) << 8) | ((uint32_t)__ldg(s + 2) << 16);
        const float sc = __ldg(scale + row);
        float4 o;
        o.x = __fmul_rn(sc, lut.e[wd & 63u].x);
        o.y = __fmul_rn(sc, lut.e[(wd >> 6) & 63u].x);
        o.z = __fmul_rn(sc, lut.e[(wd >> 12) & 63u].x);
        o.w = __fmul_rn(sc, lut.e[(wd >> 18) & 63u].x);
        reinterpret_cast<float4*>(w)[gid] = o;
    }
}

// packed2 word j of a row holds weights 16j .. 16j+15, field = t + 1, LSB first.
__global__ void pack2_kernel(const uint8_t* __restrict__ state, uint32_t* __restrict__ packed2, int C,
                             long long n_words) {
    __shared__ DecodeLut lut;
    build_decode_lut(&lut, C, threadIdx.x, blockDim.x);
    __syncthreads();
    for (long long wid = (long long)blockIdx.x * blockDim.x + threadIdx.x; wid < n_words;
         wid += (long long)gridDim.x * blockDim.x) {
        // 16 weights = 4 groups = 12 state bytes, 4-byte aligned because in % 16 == 0.
        const uint32_t* s = reinterpret_cast<const uint32_t*>(state + wid * 12);
        const uint32_t a = __ldg(s), b = __ldg(s + 1), c = __ldg(s + 2);
        const uint32_t g0 = a & 0xFFFFFFu, g1 = (a >> 24) | ((b & 0xFFFFu) << 8),
                       g2 = (b >> 16) | ((c & 0xFFu) << 16), g3 = c >> 8;
        const uint32_t gs[4] = {g0, g1, g2, g3};
        uint32_t word = 0;
#pragma unroll
        for (int gg = 0; gg < 4; ++gg)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int t = (int)lut.e[(gs[gg] >> (6 * k)) & 63u].x;
                word |= (uint32_t)((t + 1) & 3) << (2 * (gg * 4 + k));
            }
        packed2[wid] = word;
    }
}

}  // namespace

// Opt a kernel in to the device's full dynamic shared memory, once per device and kernel slot.
cudaError_t ensure_dynamic_smem(const void* kern, int slot, size_t max_smem) {
    static bool done[64][16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && slot < 16 && done[dev][slot]) return cudaSuccess;
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) return e;
    // the opt-in limit covers static + dynamic shared memory
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(max_smem - fa.sharedSizeBytes));
    if (e == cudaSuccess && dev >= 0 && dev < 64 && slot < 16) done[dev][slot] = true;
    return e;
}

cudaError_t launch_counter_update_dense(uint8_t* state, float* scale, float* v, const float* grad_w,
                                        uint32_t* packed2, int C, int in_features, int rows,
                                        int row_offset, float lr, float lr_scale, float rms_beta,
                                        float rms_eps, uint32_t seed, const uint32_t* seed_offset, int* err_word,
                                        int sm_count, size_t max_smem, cudaStream_t stream) {
    const bool with_q = (lr_scale != 0.0f);
    const uintptr_t sp0 = reinterpret_cast<uintptr_t>(state), pp0 = reinterpret_cast<uintptr_t>(packed2);
    if (in_features >= 1024 && in_features % 64 == 0 && sp0 % 16 == 0 && pp0 % 4 == 0 &&
        reinterpret_cast<uintptr_t>(grad_w) % 16 == 0) {
        // wide rows: the warp-specialised kernel, one persistent CTA per SM
        const WsLayout L = ws_layout(in_features, max_smem);
        if (L.nslots >= 2) {
            UpdParams p;
            p.state = state; p.scale = scale; p.v = v; p.grad_w = grad_w; p.packed2 = packed2;
            p.C = C; p.in_features = in_features; p.rows = rows; p.row_offset = row_offset;
            p.rows_per_batch = 1; p.state_align = 16;
            p.lr = lr; p.lr_scale = lr_scale; p.rms_beta = rms_beta; p.rms_eps = rms_eps;
            p.seed = seed; p.seed_offset = seed_offset;
            auto kern = with_q ? counter_update_ws_kernel<true> : counter_update_ws_kernel<false>;
            cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), with_q ? 10 : 11, max_smem);
            if (e != cudaSuccess) return e;
            const int grid = rows < sm_count ? rows : sm_count;
            kern<<<grid, kWsThreads, L.total, stream>>>(p, 1u << 16, 1u << 17, L.nslots, err_word);
            return cudaGetLastError();
        }
    }
    if (in_features % 16 == 0 && sp0 % 4 == 0) {
        // fast variant: rows per batch sized for four CTAs per SM when a row allows it
        const size_t target = (max_smem - 4096) / kUpdCtasPerSm;
        int Ru = kMaxRowsU16;
        while (Ru > 1 && u16_layout(in_features, Ru, with_q).total > target) --Ru;
        const U16Layout L = u16_layout(in_features, Ru, with_q);
        if (L.total <= max_smem - 1024) {
            UpdParams p;
            p.state = state; p.scale = scale; p.v = v; p.grad_w = grad_w; p.packed2 = packed2;
            p.C = C; p.in_features = in_features; p.rows = rows; p.row_offset = row_offset;
            p.rows_per_batch = Ru;
            p.state_align = (in_features % 64 == 0 && sp0 % 16 == 0 && pp0 % 16 == 0) ? 16 : 4;
            p.lr = lr; p.lr_scale = lr_scale; p.rms_beta = rms_beta; p.rms_eps = rms_eps;
            p.seed = seed; p.seed_offset = seed_offset;
            const int nb = (rows + Ru - 1) / Ru;
            int per_sm = (int)((max_smem - 1024) / L.total);
            if (per_sm > kUpdCtasPerSm) per_sm = kUpdCtasPerSm;
            if (per_sm < 1) per_sm = 1;
            int grid = sm_count * per_sm;
            if (grid > nb) grid = nb;
            const uint32_t upr = (uint32_t)(in_features / 16);
            const uint32_t magic = upr == 1 ? 0u : (uint32_t)((0x100000000ull + upr - 1) / upr);   // u / upr = mulhi(u, magic), u * upr < 2^32
            auto kern = with_q ? counter_update_u16_kernel<true> : counter_update_u16_kernel<false>;
            cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), with_q ? 2 : 3, max_smem);
            if (e != cudaSuccess) return e;
            kern<<<grid, kUpdThreads, L.total, stream>>>(p, magic, 1u << 16, 1u << 17);
            return cudaGetLastError();
        }
    }
    int R = kMaxRowsPerBatch;
    while (R > 1 && upd_smem_bytes(in_features, R, with_q) > (max_smem - 3072) / 3) --R;   // three CTAs per SM (the register limit)
    const size_t smem = upd_smem_bytes(in_features, R, with_q);
    if (smem > max_smem) return cudaErrorInvalidConfiguration;   // row too long for shared memory
    UpdParams p;
    p.state = state; p.scale = scale; p.v = v; p.grad_w = grad_w; p.packed2 = packed2;
    p.C = C; p.in_features = in_features; p.rows = rows; p.row_offset = row_offset;
    p.rows_per_batch = R;
    const uintptr_t sp = reinterpret_cast<uintptr_t>(state), pp = reinterpret_cast<uintptr_t>(packed2);
    p.state_align = (in_features % 64 == 0 && sp % 16 == 0 && pp % 16 == 0) ? 16
                    : (in_features % 16 == 0 && sp % 4 == 0) ? 4 : 1;
    p.lr = lr; p.lr_scale = lr_scale; p.rms_beta = rms_beta; p.rms_eps = rms_eps; p.seed = seed; p.seed_offset = seed_offset;
    const int nbatches = (rows + R - 1) / R;
    int ctas_per_sm = (int)(max_smem / smem);
    if (ctas_per_sm > 2048 / kUpdThreads) ctas_per_sm = 2048 / kUpdThreads;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int grid = sm_count * ctas_per_sm;
    if (grid > nbatches) grid = nbatches;
    auto kern = with_q ? counter_update_dense_kernel<true> : counter_update_dense_kernel<false>;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), with_q ? 0 : 1, max_smem);
    if (e != cudaSuccess) return e;
    kern<<<grid, kUpdThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

static cudaError_t launch_update_group_narrow(const UpdateDesc* d, int n, int C, float lr, float lr_scale, float rms_beta,
                                              float rms_eps, uint32_t seed, const uint32_t* seed_offset, int sm_count,
                                              size_t max_smem, cudaStream_t stream, int* launches);

// The fused update of several layers in one launch (same C and hyper-parameters).  Returns
// cudaErrorNotSupported, having launched nothing, when a layer does not qualify for the 16-weight
// kernel; the caller then updates layer by layer.
cudaError_t launch_counter_update_group(const UpdateDesc* d, int n, int C, float lr, float lr_scale, float rms_beta,
                                        float rms_eps, uint32_t seed, const uint32_t* seed_offset, int* err_word, int sm_count,
                                        size_t max_smem, cudaStream_t stream, int* launches) {
    const bool with_q = (lr_scale != 0.0f);
    for (int i = 0; i < n; ++i) {
        if (d[i].in_features % 16 != 0 || reinterpret_cast<uintptr_t>(d[i].state) % 4 != 0) return cudaErrorNotSupported;
        if (u16_layout(d[i].in_features, 1, with_q).total > max_smem - 1024) return cudaErrorNotSupported;
    }
    // wide layers are whole launches of their own (the per-layer launcher picks the kernel); the narrow ones share launches
    UpdateDesc narrow[kUpdGroupCap];
    int nn = 0;
    auto flush_narrow = [&]() -> cudaError_t {
        if (nn == 0) return cudaSuccess;
        cudaError_t e = launch_update_group_narrow(narrow, nn, C, lr, lr_scale, rms_beta, rms_eps, seed, seed_offset, sm_count, max_smem,
                                                   stream, launches);
        nn = 0;
        return e;
    };
    for (int i = 0; i < n; ++i) {
        if (d[i].in_features >= 1024) {
            cudaError_t e = launch_counter_update_dense(d[i].state, d[i].scale, d[i].v, d[i].grad_w, d[i].packed2, C, d[i].in_features,
                                                        d[i].rows, d[i].row_offset, lr, lr_scale, rms_beta, rms_eps, seed, seed_offset,
                                                        err_word, sm_count, max_smem, stream);
            if (e != cudaSuccess) return e;
            ++*launches;
            continue;
        }
        narrow[nn++] = d[i];
        if (nn == kUpdGroupCap) {
            cudaError_t e = flush_narrow();
            if (e != cudaSuccess) return e;
        }
    }
    return flush_narrow();
}

static cudaError_t launch_update_group_narrow(const UpdateDesc* d, int n, int C, float lr, float lr_scale, float rms_beta,
                                              float rms_eps, uint32_t seed, const uint32_t* seed_offset, int sm_count,
                                              size_t max_smem, cudaStream_t stream, int* launches) {
    const bool with_q = (lr_scale != 0.0f);
    const size_t target = (max_smem - 4096) / kUpdCtasPerSm;
    for (int done = 0; done < n;) {
        UpdGroup g;
        const int take = n - done < kUpdGroupCap ? n - done : kUpdGroupCap;
        size_t smem = 0;
        int batches = 0;
        for (int j = 0; j < take; ++j) {
            const UpdateDesc& u = d[done + j];
            int Ru = kMaxRowsU16;
            while (Ru > 1 && u16_layout(u.in_features, Ru, with_q).total > target) --Ru;
            const U16Layout L = u16_layout(u.in_features, Ru, with_q);
            if (L.total > smem) smem = L.total;
            UpdParams& p = g.p[j];
            p.state = u.state; p.scale = u.scale; p.v = u.v; p.grad_w = u.grad_w; p.packed2 = u.packed2;
            p.C = C; p.in_features = u.in_features; p.rows = u.rows; p.row_offset = u.row_offset;
            p.rows_per_batch = Ru;
            const uintptr_t sp = reinterpret_cast<uintptr_t>(u.state), pp = reinterpret_cast<uintptr_t>(u.packed2);
            p.state_align = (u.in_features % 64 == 0 && sp % 16 == 0 && pp % 16 == 0) ? 16 : 4;
            p.lr = lr; p.lr_scale = lr_scale; p.rms_beta = rms_beta; p.rms_eps = rms_eps;
            p.seed = seed; p.seed_offset = seed_offset;
            const uint32_t upr = (uint32_t)(u.in_features / 16);
            g.magic[j] = upr == 1 ? 0u : (uint32_t)((0x100000000ull + upr - 1) / upr);
            g.batch_begin[j] = batches;
            batches += (u.rows + Ru - 1) / Ru;
        }
        g.batch_begin[take] = batches;
        g.n = take;
        int per_sm = (int)((max_smem - 1024) / smem);
        if (per_sm > kUpdCtasPerSm) per_sm = kUpdCtasPerSm;
        if (per_sm < 1) per_sm = 1;
        int grid = sm_count * per_sm;
        if (grid > batches) grid = batches;
        if (grid > 0) {
            auto kern = with_q ? counter_update_u16_group_kernel<true> : counter_update_u16_group_kernel<false>;
            cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), with_q ? 8 : 9, max_smem);
            if (e != cudaSuccess) return e;
            kern<<<grid, kUpdThreads, smem, stream>>>(g, 1u << 16, 1u << 17);
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
            ++*launches;
        }
        done += take;
    }
    return cudaSuccess;
}

cudaError_t launch_decode_weight(const uint8_t* state, const float* scale, float* w, int C,
                                 int in_features, int out_features, int sm_count, cudaStream_t stream) {
    const long long n_groups = (long long)out_features * (in_features / 4);
    long long blocks = (n_groups + 255) / 256;
    if (blocks > (long long)sm_count * 16) blocks = (long long)sm_count * 16;
    decode_weight_kernel<<<(int)blocks, 256, 0, stream>>>(state, scale, w, C, in_features, n_groups);
    return cudaGetLastError();
}

cudaError_t launch_pack2(const uint8_t* state, uint32_t* packed2, int C, int in_features,
                         int out_features, int sm_count, cudaStream_t stream) {
    const long long n_words = (long long)out_features * (in_features / 16);
    long long blocks = (n_words + 255) / 256;
    if (blocks > (long long)sm_count * 16) blocks = (long long)sm_count * 16;
    pack2_kernel<<<(int)blocks, 256, 0, stream>>>(state, packed2, C, n_words);
    return cudaGetLastError();
}

}  // namespace mcl
