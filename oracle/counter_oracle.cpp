// CPU oracle for the counter-synapse linear path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain C++, the arithmetic of the reference's counter-linear
// kernels so that the CUDA path can be checked against it.  It is never part of the
// shipped library: only tests, the smoke check and the benchmark's CPU-baseline leg
// load it.  Every function names the reference source it follows (paths are relative
// to the MotifCL tree).
//
// Definition of "the reference result": OpenCL C / GLSL leave FMA contraction and
// the rounding of '/' and sqrt to the implementation.  This oracle fixes them to
// IEEE-754 round-to-nearest with NO contraction (build: -O2 -ffp-contract=off, no
// -ffast-math, x86-64 SSE2 scalar math).  Parity status: pinned -- see
// oracle/ref_shim.cpp, which compiles the reference's own kernels/compact_counter.cl
// and is compared against this file by tests/test_oracle_vs_ref.py, and
// tests/golden/, which stores outputs of that compiled reference.
//
// Float->int conversions of values outside int range are undefined in C; like the
// reference, this oracle only defines results for finite inputs with |val| < 2^31.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include <algorithm>
#include <thread>

namespace {

int g_threads = 1;

// Static-chunk parallel loop over [0, n) on g_threads host threads (std::thread, so the
// checker needs no OpenMP runtime).  Iterations are independent in every use below.
template <class F>
void parallel_for(int n, F body) {
    const int nt = std::max(1, std::min(g_threads, n));
    if (nt == 1) {
        for (int i = 0; i < n; ++i) body(i);
        return;
    }
    std::vector<std::thread> th;
    th.reserve(nt);
    for (int t = 0; t < nt; ++t)
        th.emplace_back([=] {
            const int lo = (int)((int64_t)n * t / nt), hi = (int)((int64_t)n * (t + 1) / nt);
            for (int i = lo; i < hi; ++i) body(i);
        });
    for (auto& x : th) x.join();
}

// kernels/compact_counter.cl:7-16 (cc_decode / cc_encode)
inline void cc_decode(int code, int C, int* t, int* c) {
    const int lv = 2 * C - 1;
    *t = code / lv - 1;
    *c = code % lv - (C - 1);
}
inline int cc_encode(int t, int c, int C) {
    const int lv = 2 * C - 1;
    return (t + 1) * lv + (c + (C - 1));
}
// kernels/compact_counter.cl:17-24 (cc_hash_u32 / cc_uniform01)
inline uint32_t cc_hash_u32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    x ^= x >> 16; return x;
}
inline float cc_uniform01(uint32_t x) {
    return (float)(cc_hash_u32(x) & 0x00ffffffu) * (1.0f / 16777216.0f);
}
// kernels/compact_counter.cl:25-36 (cc_unpack4 / cc_pack4): four 6-bit codes in 3 bytes,
// i.e. a little-endian 24-bit word c0 | c1<<6 | c2<<12 | c3<<18.
inline void cc_unpack4(const uint8_t* p, int cc[4]) {
    const int b0 = p[0], b1 = p[1], b2 = p[2];
    cc[0] = b0 & 0x3F;
    cc[1] = ((b0 >> 6) | (b1 << 2)) & 0x3F;
    cc[2] = ((b1 >> 4) | (b2 << 4)) & 0x3F;
    cc[3] = (b2 >> 2) & 0x3F;
}
inline void cc_pack4(uint8_t* p, const int c[4]) {
    p[0] = (uint8_t)((c[0] & 0x3F) | ((c[1] & 0x03) << 6));
    p[1] = (uint8_t)(((c[1] >> 2) & 0x0F) | ((c[2] & 0x0F) << 4));
    p[2] = (uint8_t)(((c[2] >> 4) & 0x03) | ((c[3] & 0x3F) << 2));
}

inline float clampf(float x, float lo, float hi) { return std::fmin(std::fmax(x, lo), hi); }

// One row of kernels/compact_counter.cl:59-100 (counter_row_stats_f32): 64 lanes, lane l
// walks groups l, l+64, ... accumulating g_sq += gw*gw and grad_s += gw*t, then the
// shared-memory tree s = 32,16,...,1 with lane[l] += lane[l+s], then the five scalar
// lines of lane 0.  `gw` is the row's dense gradient (in_features floats).
inline void row_stats_one(const uint8_t* state_row, const float* gw, int C, int in_features,
                          float scale_old, float* v_io, float* scale_new, float* denom,
                          float lr_scale, float rms_beta, float rms_eps) {
    const int gpr = in_features / 4;
    float lg[64], lgs[64];
    for (int lid = 0; lid < 64; ++lid) {
        float g_sq = 0.0f, grad_s = 0.0f;
        for (int g = lid; g < gpr; g += 64) {
            int cc[4];
            cc_unpack4(state_row + (size_t)g * 3, cc);
            for (int k = 0; k < 4; ++k) {
                const float w = gw[g * 4 + k];
                g_sq += w * w;
                int t, c;
                cc_decode(cc[k], C, &t, &c);
                grad_s += w * (float)t;
            }
        }
        lg[lid] = g_sq;
        lgs[lid] = grad_s;
    }
    for (int s = 32; s > 0; s >>= 1)
        for (int lid = 0; lid < s; ++lid) {
            lg[lid] += lg[lid + s];
            lgs[lid] += lgs[lid + s];
        }
    const float gsq = lg[0] / (float)in_features;
    const float gs = lgs[0] / std::sqrt((float)in_features);
    const float vv = rms_beta * (*v_io) + (1.0f - rms_beta) * gsq;
    *v_io = vv;
    *denom = std::fmax(std::sqrt(vv), rms_eps);
    *scale_new = clampf(scale_old - lr_scale * gs, 1e-5f, 10.0f);
}

// One packed group of kernels/compact_counter.cl:104-139 (counter_apply_update_f32).
// `elem0` is the 32-bit global element index of the group's first weight.
inline void apply_group(uint8_t* p, const float gw[4], int C, uint32_t elem0, float s_old,
                        float s_new, float dn, float lr, uint32_t seed, int field_out[4]) {
    int cc[4], nc[4];
    cc_unpack4(p, cc);
    const float Cf = (float)C;
    for (int k = 0; k < 4; ++k) {
        const uint32_t elem = elem0 + (uint32_t)k;
        int t, c;
        cc_decode(cc[k], C, &t, &c);
        const float tick = -lr * (gw[k] / dn) * (Cf / s_new);
        const float c_reb = (float)c * (s_old / s_new);
        const float val = c_reb + tick;
        const float f = std::floor(val);
        const float rnd = cc_uniform01(seed ^ cc_hash_u32(elem));
        const float ccv = f + (rnd < (val - f) ? 1.0f : 0.0f);
        const float carry = std::trunc(ccv / Cf);
        float rem = ccv - carry * Cf;
        const int nt = t + (int)carry;
        const int ct = nt < -1 ? -1 : (nt > 1 ? 1 : nt);
        if (ct != nt) rem = (ccv > 0.0f ? 1.0f : (ccv < 0.0f ? -1.0f : 0.0f)) * (Cf - 1.0f);
        int ri = (int)rem;
        ri = ri < -(C - 1) ? -(C - 1) : (ri > C - 1 ? C - 1 : ri);
        nc[k] = cc_encode(ct, ri, C) & 0xFF;
        field_out[k] = ct + 1;
    }
    cc_pack4(p, nc);
}

}  // namespace

extern "C" {

void orc_set_threads(int n) { g_threads = n > 0 ? n : 1; }
int orc_get_threads() { return g_threads; }

// Pack one code per weight (codes[out*in], values 0..63) into the [out, in/4, 3] layout
// of src/nn/compact_counter.cpp:64-78, and the inverse.
void orc_pack_codes(const uint8_t* codes, uint8_t* state, int64_t n_weights) {
    for (int64_t g = 0; g < n_weights / 4; ++g) {
        int c[4] = {codes[4 * g], codes[4 * g + 1], codes[4 * g + 2], codes[4 * g + 3]};
        cc_pack4(state + 3 * g, c);
    }
}
void orc_unpack_codes(const uint8_t* state, uint8_t* codes, int64_t n_weights) {
    for (int64_t g = 0; g < n_weights / 4; ++g) {
        int c[4];
        cc_unpack4(state + 3 * g, c);
        for (int k = 0; k < 4; ++k) codes[4 * g + k] = (uint8_t)c[k];
    }
}

// kernels/compact_counter.cl:39-55 (decode_counter_state_weight_f32): w = scale[row] * t.
void orc_decode_weight(const uint8_t* state, const float* scale, float* w, int C, int in_features,
                       int out_features) {
    const int gpr = in_features / 4;
    parallel_for(out_features, [=](int row) {
        for (int g = 0; g < gpr; ++g) {
            int cc[4];
            cc_unpack4(state + ((size_t)row * gpr + g) * 3, cc);
            const float s = scale[row];
            for (int k = 0; k < 4; ++k) {
                int t, c;
                cc_decode(cc[k], C, &t, &c);
                w[(size_t)row * in_features + g * 4 + k] = s * (float)t;
            }
        }
    });
}

// Derived artifact (no reference kernel): 2-bit packed ternary weights.  Word m/16 of a
// row holds weight m in bits [2(m%16)+1 : 2(m%16)], field = t + 1 with t from cc_decode
// (kernels/compact_counter.cl:7-12); layout of docs/BITNET_TERNARY_VULKAN_PLAN.md:97.
// Requires in_features % 16 == 0.
void orc_pack2(const uint8_t* state, uint32_t* packed2, int C, int in_features, int out_features) {
    const int gpr = in_features / 4, wpr = in_features / 16;
    parallel_for(out_features, [=](int row) {
        for (int wd = 0; wd < wpr; ++wd) {
            uint32_t word = 0;
            for (int gg = 0; gg < 4; ++gg) {
                int cc[4];
                cc_unpack4(state + ((size_t)row * gpr + wd * 4 + gg) * 3, cc);
                for (int k = 0; k < 4; ++k) {
                    int t, c;
                    cc_decode(cc[k], C, &t, &c);
                    word |= (uint32_t)((t + 1) & 3) << (2 * (gg * 4 + k));
                }
            }
            packed2[(size_t)row * wpr + wd] = word;
        }
    });
}

// kernels/compact_counter.cl:59-100 for all rows of a shard; writes v in place.
void orc_row_stats(const uint8_t* state, const float* scale, float* v, const float* grad_w,
                   float* scale_new, float* denom, int C, int in_features, int rows,
                   float lr_scale, float rms_beta, float rms_eps) {
    const size_t row_bytes = (size_t)(in_features / 4) * 3;
    parallel_for(rows, [=](int row) {
        row_stats_one(state + row * row_bytes, grad_w + (size_t)row * in_features, C, in_features,
                      scale[row], &v[row], &scale_new[row], &denom[row], lr_scale, rms_beta, rms_eps);
    });
}

// Dense update = src/nn/compact_counter.cpp:113-156 (apply_update_seed): row stats, tick,
// scale commit.  `rows` rows starting at global row `row_offset` (the hash index of a
// weight is (row_offset+row)*in + i, so a row shard updates exactly like the same rows
// of the full matrix).  packed2 may be null; if given it receives field ct+1 per weight
// (requires in_features % 16 == 0).
void orc_update_dense(uint8_t* state, float* scale, float* v, const float* grad_w,
                      uint32_t* packed2, int C, int in_features, int rows, int row_offset, float lr,
                      float lr_scale, float rms_beta, float rms_eps, uint32_t seed) {
    const int gpr = in_features / 4;
    const size_t row_bytes = (size_t)gpr * 3;
    std::vector<float> scale_new_v(rows), denom_v(rows);
    float* scale_new = scale_new_v.data();
    float* denom = denom_v.data();
    orc_row_stats(state, scale, v, grad_w, scale_new, denom, C, in_features, rows, lr_scale,
                  rms_beta, rms_eps);
    parallel_for(rows, [=](int row) {
        uint8_t* srow = state + row * row_bytes;
        const float* gw = grad_w + (size_t)row * in_features;
        const uint32_t base = (uint32_t)(row_offset + row) * (uint32_t)in_features;
        for (int g = 0; g < gpr; ++g) {
            int field[4];
            apply_group(srow + (size_t)g * 3, gw + g * 4, C, base + (uint32_t)(g * 4), scale[row],
                        scale_new[row], denom[row], lr, seed, field);
            if (packed2) {
                uint32_t* wp = packed2 + (size_t)row * (in_features / 16) + g / 4;
                const int sh = 8 * (g & 3);
                uint32_t bits = 0;
                for (int k = 0; k < 4; ++k) bits |= (uint32_t)(field[k] & 3) << (2 * k);
                *wp = (*wp & ~(0xFFu << sh)) | (bits << sh);
            }
        }
    });
    for (int row = 0; row < rows; ++row) scale[row] = scale_new[row];  // kernels/basic.cl:6-9
}

// dW[o,i] = sum_r dY[r,o] * x[r,i], r ascending, separate multiply and add: the value the
// fused kernels recompute per weight (kernels/compact_counter.cl:175,221) and what
// matmul_transa_rb4_f32 produces per element (kernels/matmul.cl:452-465).
void orc_grad_w(const float* grad_out, const float* x, float* grad_w, int N, int in_features,
                int out_features) {
    parallel_for(out_features, [=](int o) {
        float* dst = grad_w + (size_t)o * in_features;
        for (int i = 0; i < in_features; ++i) dst[i] = 0.0f;
        for (int r = 0; r < N; ++r) {
            const float go = grad_out[(size_t)r * out_features + o];
            const float* xr = x + (size_t)r * in_features;
            for (int i = 0; i < in_features; ++i) dst[i] += go * xr[i];
        }
    });
}

// Memory-native update = src/nn/compact_counter.cpp:158-231 (apply_update_backward):
// identical to the dense update with grad_w recomputed as above.
void orc_update_fused(uint8_t* state, float* scale, float* v, const float* grad_out, const float* x,
                      uint32_t* packed2, int C, int in_features, int out_features, int N, float lr,
                      float lr_scale, float rms_beta, float rms_eps, uint32_t seed) {
    std::vector<float> gw((size_t)out_features * in_features);
    orc_grad_w(grad_out, x, gw.data(), N, in_features, out_features);
    orc_update_dense(state, scale, v, gw.data(), packed2, C, in_features, out_features, 0, lr,
                     lr_scale, rms_beta, rms_eps, seed);
}

// Forward: src/nn/compact_counter.cpp:287-293 (decode_weight then matmul_transpose_b);
// each y[r,o] is the k-ascending fp32 sum of x[r,k] * (scale[o]*t[o,k])
// (kernels/matmul.cl:509-541 per element).
void orc_forward(const float* x, const uint8_t* state, const float* scale, float* y, int N,
                 int in_features, int out_features, int C) {
    std::vector<float> wv((size_t)out_features * in_features);
    orc_decode_weight(state, scale, wv.data(), C, in_features, out_features);
    const float* w = wv.data();
    parallel_for(N, [=](int r) {
        for (int o = 0; o < out_features; ++o) {
            const float* xr = x + (size_t)r * in_features;
            const float* wo = w + (size_t)o * in_features;
            float acc = 0.0f;
            for (int k = 0; k < in_features; ++k) acc += xr[k] * wo[k];
            y[(size_t)r * out_features + o] = acc;
        }
    });
}

// kernels/compact_counter.cl:248-269 (counter_backward_input_f32):
// grad_x[r,i] = sum_o (grad_out[r,o] * scale[o]) * t[o,i], o ascending.
void orc_backward_input(const float* grad_out, const uint8_t* state, const float* scale,
                        float* grad_x, int N, int in_features, int out_features, int C) {
    std::vector<float> tfv((size_t)out_features * in_features);
    std::vector<float> ones(out_features, 1.0f);
    orc_decode_weight(state, ones.data(), tfv.data(), C, in_features, out_features);
    const float* tf = tfv.data();
    parallel_for(N, [=](int r) {
        float* dst = grad_x + (size_t)r * in_features;
        for (int i = 0; i < in_features; ++i) dst[i] = 0.0f;
        for (int o = 0; o < out_features; ++o) {
            const float gs = grad_out[(size_t)r * out_features + o] * scale[o];
            const float* to = tf + (size_t)o * in_features;
            for (int i = 0; i < in_features; ++i) dst[i] += gs * to[i];
        }
    });
}

// Generic f32 matmul as the naive kernel computes it (kernels/matmul.cl:405-411): k-ascending
// fp32 accumulation.  C[M,N] = op(A) op(B); transA: A stored [K,M]; transB: B stored [N,K].
void orc_matmul_f32(const float* A, const float* B, float* Cm, int M, int K, int N, int transA,
                    int transB) {
    parallel_for(M, [=](int row) {
        for (int col = 0; col < N; ++col) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) {
                const float av = transA ? A[(size_t)k * M + row] : A[(size_t)row * K + k];
                const float bv = transB ? B[(size_t)col * K + k] : B[(size_t)k * N + col];
                acc += av * bv;
            }
            Cm[(size_t)row * N + col] = acc;
        }
    });
}

// float64-accumulate variant of the same product, for error budgets of the split GEMMs.
void orc_matmul_f64acc(const float* A, const float* B, double* Cm, int M, int K, int N, int transA,
                       int transB) {
    parallel_for(M, [=](int row) {
        for (int col = 0; col < N; ++col) {
            double acc = 0.0;
            for (int k = 0; k < K; ++k) {
                const double av = transA ? A[(size_t)k * M + row] : A[(size_t)row * K + k];
                const double bv = transB ? B[(size_t)col * K + k] : B[(size_t)k * N + col];
                acc += av * bv;
            }
            Cm[(size_t)row * N + col] = acc;
        }
    });
}

// src/runtime/native_matmul.cpp:51-71,110-133 (native::matmul_f32_m1): out[n] = sum_k a[k]*b[k,n],
// k ascending, multiply then add (the SSE form does four columns per vector, same order).
void orc_matmul_f32_m1(const float* a, const float* b, float* out, int64_t k, int64_t n) {
    for (int64_t col = 0; col < n; ++col) {
        float acc = 0.0f;
        for (int64_t kk = 0; kk < k; ++kk) acc += a[kk] * b[kk * n + col];
        out[col] = acc;
    }
}

// Ternary decode GEMV semantics (derived): y[m,o] = sum_k x[m,k] * (scale[o] * t[o,k]) with t
// read from the 2-bit words; same summation as orc_forward.  float64 accumulate variant too.
void orc_ternary_gemv(const float* x, const uint32_t* packed2, const float* scale, float* y, int M,
                      int in_features, int out_features) {
    const int wpr = in_features / 16;
    parallel_for(out_features, [=](int o) {
        for (int m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int k = 0; k < in_features; ++k) {
                const int f = (packed2[(size_t)o * wpr + k / 16] >> (2 * (k % 16))) & 3;
                acc += x[(size_t)m * in_features + k] * (scale[o] * (float)(f - 1));
            }
            y[(size_t)m * out_features + o] = acc;
        }
    });
}
void orc_ternary_gemv_f64(const float* x, const uint32_t* packed2, const float* scale, double* y,
                          int M, int in_features, int out_features) {
    const int wpr = in_features / 16;
    parallel_for(out_features, [=](int o) {
        for (int m = 0; m < M; ++m) {
            double acc = 0.0;
            for (int k = 0; k < in_features; ++k) {
                const int f = (packed2[(size_t)o * wpr + k / 16] >> (2 * (k % 16))) & 3;
                acc += (double)x[(size_t)m * in_features + k] * (double)(f - 1);
            }
            y[(size_t)m * out_features + o] = acc * (double)scale[o];
        }
    });
}

}  // extern "C"
