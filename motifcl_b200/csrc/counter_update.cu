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
//          thread-iteration, rewriting the state bytes in shared memory and emitting one
//          byte of 2-bit fields per group.
//   store  all threads copy the new state and the 2-bit words back with wide stores.
// HBM traffic per weight: 0.75 B state in, 4 B gradient in, 0.75 B state out, 0.25 B
// packed weights out = 5.75 B.
#include "counter_codec.cuh"
#include "kernels.h"

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

// Shared-memory carve-up (per CTA), all offsets 16-byte aligned:
//   lut[64] float2 | rowc[R] RowConst | part[R][2][32] float | gw[R][I] float |
//   q[R][I] float (only WITH_Q) | st[R][sb] bytes (sb = state row bytes rounded up to 16, +16)
//   | so[R][sb] bytes (new state) | p2[R][I/4 rounded to 16] bytes
template <bool WITH_Q>
__global__ void __launch_bounds__(kUpdThreads)
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
    float* gw_s = part + kMaxRowsPerBatch * 64;
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
    const uint32_t seed = p.seed + (p.seed_offset ? __ldg(p.seed_offset) : 0u);
    const bool aligned16 = p.state_align >= 16;   // state rows start and end on 16-byte boundaries
    const bool aligned4 = p.state_align >= 4;     // ... on 4-byte boundaries

    build_decode_lut(lut, p.C, tid, kUpdThreads);
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

        // ---- tick: one packed group per thread-iteration --------------------------------
        for (int r = 0; r < nrows; ++r) {
            const RowConst rc = rowc[r];
            const float4* g4 = reinterpret_cast<const float4*>(gw_s + (size_t)r * I);
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(st_s + (size_t)r * sb);
            unsigned char* so = so_s + (size_t)r * sb;
            unsigned char* p2 = p2_s + (size_t)r * pb;
            const uint32_t elem_row = (uint32_t)(p.row_offset + row0 + r) * (uint32_t)I;
            for (int g = tid; g < gpr; g += kUpdThreads) {
                const uint32_t w = load_group24(raw, (uint32_t)g * 3u);
                const float4 gw = g4[g];
                const float gwv[4] = {gw.x, gw.y, gw.z, gw.w};
                uint32_t nw = 0, fields = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 tc = lut->e[(w >> (6 * k)) & 63u];
                    uint32_t fld;
                    const uint32_t code =
                        counter_tick(gwv[k], tc.x, tc.y, elem_row + (uint32_t)(g * 4 + k), seed,
                                     neg_lr, rc.dn, rc.k_tick, rc.k_reb, Cf, p.C, lv, &fld);
                    nw |= (code & 0x3Fu) << (6 * k);
                    fields |= (fld & 3u) << (2 * k);
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

size_t upd_smem_bytes(int I, int R, bool with_q) {
    const int gpr = I / 4;
    const size_t sb = (size_t)((gpr * 3 + 15) & ~15) + 16;
    const size_t pb = (size_t)((gpr + 15) & ~15);
    return sizeof(DecodeLut) + sizeof(RowConst) * kMaxRowsPerBatch + sizeof(float) * 64 * kMaxRowsPerBatch +
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
    static bool done[64][4] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && slot < 4 && done[dev][slot]) return cudaSuccess;
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) return e;
    // the opt-in limit covers static + dynamic shared memory
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(max_smem - fa.sharedSizeBytes));
    if (e == cudaSuccess && dev >= 0 && dev < 64 && slot < 4) done[dev][slot] = true;
    return e;
}

cudaError_t launch_counter_update_dense(uint8_t* state, float* scale, float* v, const float* grad_w,
                                        uint32_t* packed2, int C, int in_features, int rows,
                                        int row_offset, float lr, float lr_scale, float rms_beta,
                                        float rms_eps, uint32_t seed, const uint32_t* seed_offset, int sm_count,
                                        size_t max_smem, cudaStream_t stream) {
    const bool with_q = (lr_scale != 0.0f);
    int R = kMaxRowsPerBatch;
    while (R > 1 && upd_smem_bytes(in_features, R, with_q) > max_smem / 2) --R;
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
