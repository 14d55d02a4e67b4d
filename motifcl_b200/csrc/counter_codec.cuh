// Device-side pieces of the counter-synapse state code shared by every kernel here.
//
// State layout (MotifCL kernels/compact_counter.cl:2-3,25-36): each weight is a 6-bit code,
// four codes per 3 bytes, i.e. one little-endian 24-bit word  c0 | c1<<6 | c2<<12 | c3<<18;
// the tensor is [out, in/4, 3] bytes.  code = (t+1)*(2C-1) + (c + C-1)
// (kernels/compact_counter.cl:7-16) with ternary digit t and counter c in [-(C-1), C-1].
//
// All floating-point steps that must agree bit-for-bit with the reference use the
// explicitly rounded intrinsics (__fmul_rn, __fadd_rn, __fdiv_rn, __fsqrt_rn): nvcc never
// contracts those into FMAs, which is the rounding the CPU checker is built with.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mcl {

// kernels/compact_counter.cl:17-21
__device__ __forceinline__ uint32_t cc_hash_u32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}

// Decode table for all 64 code values, built once per CTA with the reference's integer
// formulas (kernels/compact_counter.cl:7-12), so every byte value -- including codes that a
// trained layer never reaches, such as 63 for C = 11 (t = +2) -- decodes exactly as the
// reference does.  x = float(t), y = float(c).
struct DecodeLut {
    float2 e[64];
};

__device__ __forceinline__ void build_decode_lut(DecodeLut* lut, int C, int tid, int nthreads) {
    const int lv = 2 * C - 1;
    for (int code = tid; code < 64; code += nthreads) {
        const int t = code / lv - 1;
        const int c = code % lv - (C - 1);
        lut->e[code] = make_float2((float)t, (float)c);
    }
}

// 24-bit group word starting at byte offset `byte_off` of a shared-memory byte area that is
// 4-byte aligned and padded by at least 4 readable bytes.
__device__ __forceinline__ uint32_t load_group24(const uint32_t* raw, uint32_t byte_off) {
    const uint32_t w = byte_off >> 2;
    const uint32_t lo = raw[w], hi = raw[w + 1];
    return __funnelshift_r(lo, hi, (byte_off & 3u) * 8u) & 0x00FFFFFFu;
}

// One stochastic-rounding counter tick, kernels/compact_counter.cl:119-136.
//   gw      weight gradient of this element
//   tf, cf  decoded ternary digit and counter (as floats, exact small integers)
//   elem    32-bit global element index (row * in_features + i)
//   neg_lr  -lr;  k_tick = C / s_new;  k_reb = s_old / s_new;  dn = denom;  Cf = float(C)
// Returns the new 6-bit code; *field receives the new ternary digit + 1 (2-bit field).
__device__ __forceinline__ uint32_t counter_tick(float gw, float tf, float cf, uint32_t elem,
                                                 uint32_t seed, float neg_lr, float dn, float k_tick,
                                                 float k_reb, float Cf, int C, int lv,
                                                 uint32_t* field) {
    const float tick = __fmul_rn(__fmul_rn(neg_lr, __fdiv_rn(gw, dn)), k_tick);
    const float c_reb = __fmul_rn(cf, k_reb);
    const float val = __fadd_rn(c_reb, tick);
    const float f = floorf(val);
    const uint32_t h = cc_hash_u32(seed ^ cc_hash_u32(elem)) & 0x00ffffffu;
    const float rnd = __fmul_rn((float)h, 1.0f / 16777216.0f);
    const float ccv = __fadd_rn(f, (rnd < __fsub_rn(val, f)) ? 1.0f : 0.0f);
    const float carry = truncf(__fdiv_rn(ccv, Cf));
    float rem = __fsub_rn(ccv, __fmul_rn(carry, Cf));
    const int nt = (int)tf + (int)carry;
    const int ct = nt < -1 ? -1 : (nt > 1 ? 1 : nt);
    if (ct != nt) rem = __fmul_rn(ccv > 0.0f ? 1.0f : (ccv < 0.0f ? -1.0f : 0.0f), __fsub_rn(Cf, 1.0f));
    int ri = (int)rem;
    ri = ri < -(C - 1) ? -(C - 1) : (ri > C - 1 ? C - 1 : ri);
    *field = (uint32_t)(ct + 1);
    return (uint32_t)((ct + 1) * lv + (ri + (C - 1))) & 0xFFu;
}

}  // namespace mcl
