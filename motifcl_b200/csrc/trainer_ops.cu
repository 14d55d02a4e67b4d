// The fp32 ops MotifCL's ternary15m block stack runs between its counter layers: rmsnorm and its
// two backward kernels, swiglu and its backward, mean softmax cross-entropy and its backward, and
// batched grouped-query attention forward/backward.  Semantics follow MotifCL's Vulkan shaders
// (kernels/vulkan/rmsnorm_f32.comp, rmsnorm_bwd_x_f32.comp, rmsnorm_row_inv_f32.comp,
// rmsnorm_bwd_w_f32.comp, swiglu_f32.comp, swiglu_bwd_f32.comp, ce_fwd_rows_f32.comp,
// ce_bwd_f32.comp, mean_reduce_f32.comp, gqa_fwd_general_f32.comp, gqa_bwd_probs_f32.comp,
// gqa_bwd_dkv_f32.comp); the reductions run in a different order (warp shuffles instead of a
// 64-lane shared-memory tree), so results agree to fp32 rounding, not bit for bit.  The row ops are
// HBM-bound: one block (or warp) per row, coalesced loads.  Attention runs as batched, shared-memory-
// tiled fp32 products around a softmax row pass instead of the shaders' one workgroup per query.
#include "kernels.h"

#include <cfloat>

namespace mcl {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Every thread of the block receives the result; `red` holds 32 floats.  Safe to call repeatedly.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : 0.0f;
    return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : -FLT_MAX;
    return warp_max(r);
}

// ---- rmsnorm -------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                      float* __restrict__ out, float* __restrict__ row_inv,
                                                      size_t rows, int cols, float eps) {
    __shared__ float red[32];
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + row * (size_t)cols;
        float ss = 0.0f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) ss += xr[c] * xr[c];
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)cols + eps);
        if (row_inv != nullptr) {
            if (threadIdx.x == 0) row_inv[row] = inv;
        } else {
            float* o = out + row * (size_t)cols;
            for (int c = threadIdx.x; c < cols; c += blockDim.x) o[c] = xr[c] * inv * w[c];
        }
    }
}

__global__ void __launch_bounds__(128) rmsnorm_bwd_x_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                            const float* __restrict__ dy, float* __restrict__ dx,
                                                            size_t rows, int cols, float eps) {
    __shared__ float red[32];
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + row * (size_t)cols;
        const float* gr = dy + row * (size_t)cols;
        float ss = 0.0f, dot = 0.0f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            const float xv = xr[c];
            ss += xv * xv;
            dot += gr[c] * w[c] * xv;
        }
        ss = block_sum(ss, red);
        dot = block_sum(dot, red);
        const float inv = rsqrtf(ss / (float)cols + eps);
        const float k = inv * inv * inv * dot / (float)cols;
        float* o = dx + row * (size_t)cols;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) o[c] = gr[c] * w[c] * inv - xr[c] * k;
    }
}

// dw[c] += sum over this block's rows of dy*x*row_inv; dw is zeroed before the launch.
__global__ void __launch_bounds__(256) rmsnorm_bwd_w_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                            const float* __restrict__ row_inv, float* __restrict__ dw,
                                                            size_t rows, int cols, size_t rows_per_block) {
    __shared__ float part[8][33];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + cx;
    const size_t r0 = (size_t)blockIdx.y * rows_per_block;
    const size_t r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
    float acc = 0.0f;
    if (col < cols)
        for (size_t r = r0 + ry; r < r1; r += 8) acc += dy[r * cols + col] * x[r * cols + col] * row_inv[r];
    part[ry][cx] = acc;
    __syncthreads();
    if (ry == 0 && col < cols) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += part[j][cx];
        atomicAdd(dw + col, s);
    }
}

// ---- swiglu ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ packed, float* __restrict__ out,
                                                     size_t rows, int hidden) {
    const size_t n = rows * (size_t)hidden;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / hidden;
        const int col = (int)(i - row * hidden);
        const float gate = packed[row * 2 * hidden + col];
        const float up = packed[row * 2 * hidden + hidden + col];
        const float sig = 1.0f / (1.0f + expf(-gate));
        out[i] = gate * sig * up;
    }
}
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const float* __restrict__ packed, const float* __restrict__ dy,
                                                         float* __restrict__ dpacked, size_t rows, int hidden) {
    const size_t n = rows * (size_t)hidden;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / hidden;
        const int col = (int)(i - row * hidden);
        const size_t base = row * 2 * hidden;
        const float gate = packed[base + col];
        const float up = packed[base + hidden + col];
        const float go = dy[i];
        const float sig = 1.0f / (1.0f + expf(-gate));
        dpacked[base + col] = go * up * (sig + gate * sig * (1.0f - sig));
        dpacked[base + hidden + col] = go * gate * sig;
    }
}

// ---- mean softmax cross-entropy --------------------------------------------------------------
// A row of logits is read from HBM once: each of the 256 threads keeps its strided share (up to kCeHold values,
// i.e. rows of up to 32768 classes; longer rows re-read the tail from memory) in registers for the max, sum
// and gradient passes.
constexpr int kCeHold = 128;

template <bool BACKWARD>
__global__ void __launch_bounds__(256) ce_kernel(const float* __restrict__ logits, const int* __restrict__ targets,
                                                 float* __restrict__ partial, const float* __restrict__ grad_out,
                                                 float* __restrict__ grad_logits, size_t rows, int cols) {
    __shared__ float red[32];
    const float gscale = BACKWARD ? grad_out[0] / (float)rows : 0.0f;
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* l = logits + row * (size_t)cols;
        float hold[kCeHold];
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < kCeHold; ++j) {
            const int c = threadIdx.x + j * 256;
            hold[j] = c < cols ? l[c] : -FLT_MAX;
            m = fmaxf(m, hold[j]);
        }
        for (int c = threadIdx.x + kCeHold * 256; c < cols; c += 256) m = fmaxf(m, l[c]);
        m = block_max(m, red);
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < kCeHold; ++j) {
            const int c = threadIdx.x + j * 256;
            if (c < cols) {
                hold[j] = expf(hold[j] - m);
                s += hold[j];
            }
        }
        for (int c = threadIdx.x + kCeHold * 256; c < cols; c += 256) s += expf(l[c] - m);
        s = block_sum(s, red);
        const int t = targets[row];
        if (!BACKWARD) {
            if (threadIdx.x == 0) partial[row] = (t < 0 || t >= cols) ? 0.0f : logf(s) + m - l[t];
        } else {
            const float inv = 1.0f / s;
            float* g = grad_logits + row * (size_t)cols;
#pragma unroll
            for (int j = 0; j < kCeHold; ++j) {
                const int c = threadIdx.x + j * 256;
                if (c < cols) g[c] = gscale * (hold[j] * inv - (c == t ? 1.0f : 0.0f));
            }
            for (int c = threadIdx.x + kCeHold * 256; c < cols; c += 256)
                g[c] = gscale * (expf(l[c] - m) * inv - (c == t ? 1.0f : 0.0f));
        }
    }
}
__global__ void __launch_bounds__(256) mean_kernel(const float* __restrict__ in, float* __restrict__ out, size_t n,
                                                   size_t denom) {
    __shared__ float red[32];
    float s = 0.0f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) s += in[i];
    s = block_sum(s, red);
    if (threadIdx.x == 0) out[0] = denom > 0 ? s / (float)denom : 0.0f;
}
// ---- batched grouped-query attention ---------------------------------------------------------
// q [B*Tq, n_head*hd], k [B*key_stride, n_kv*hd], v [B*key_stride, n_kv*vhd], out [B*Tq, n_head*vhd].
struct GqaDims {
    int batch, tq, tk, key_stride, n_head, n_kv, hd, vhd, causal, q_off, window;
    float scale;
};
// first and one-past-last key a query may attend to
__device__ __forceinline__ void key_range(const GqaDims& p, int tq, int& k0, int& k1) {
    const int abs_q = p.q_off + tq;
    k1 = p.causal ? (abs_q + 1 < p.tk ? abs_q + 1 : p.tk) : p.tk;
    k0 = 0;
    if (p.window != 0 && abs_q + 1 > p.window) k0 = abs_q + 1 - p.window;
    if (k0 > k1) k0 = k1;
}

// ---- attention as batched fp32 products + a row pass ------------------------------------------
// The seven products of attention forward and backward (S = scale*Q K^T, O = P V, dP = dO V^T,
// dq = scale*dS K, dv = P^T dO, dk = scale*dS^T Q) are one batched, strided, shared-memory-tiled
// SIMT fp32 product; exact fp32 FMAs, no tensor cores (tf32 would not hold the reference's fp32
// accuracy).  An element (r, k) of an operand of batch z = (b, hz) lives at
//     base + b*bs + (hz / hdiv)*hs + r*rs + (k / K0)*s1 + (k % K0)*s0
// which covers row- and column-major tiles, grouped heads (several query heads reading one kv
// head) and the sum over the heads of a group (k runs over (head in group, query)).
struct BOperand {
    const float* base;
    long long bs, hs, rs, s0, s1;
    int hdiv, K0, contig_k;          // contig_k: k is the unit-stride index (else the row index is)
};
struct BGemm {
    BOperand a, b;
    float* c;
    long long c_bs, c_hs, c_rs;
    int M, N, K, Hz;
    float alpha;
    int causal_mode, q_off;          // 0 none; 1 skip tiles above the diagonal (m = query, n = key);
};                                   // 2 k (= key) ends at the tile's last query; 3 k (= query) starts at the tile's first key
constexpr int kBT = 64, kBK = 16;

// A 64 x 16 tile moves through registers (4 elements per thread) so that the next tile's global loads are in
// flight while the current one is multiplied.
__device__ __forceinline__ void fetch_tile(const BOperand& o, const float* zbase, int r0, int rmax, int k0, int kend,
                                           float (&reg)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + i * 256;
        const int r = o.contig_k ? idx >> 4 : idx & 63;
        const int kk = o.contig_k ? idx & 15 : idx >> 6;
        const int row = r0 + r, k = k0 + kk;
        float v = 0.0f;
        if (row < rmax && k < kend) {
            const long long off = o.K0 > 0 ? (long long)(k / o.K0) * o.s1 + (long long)(k % o.K0) * o.s0 : (long long)k * o.s0;
            v = zbase[(long long)row * o.rs + off];
        }
        reg[i] = v;
    }
}
__device__ __forceinline__ void store_tile(const BOperand& o, const float (&reg)[4], float (*dst)[kBT + 4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + i * 256;
        const int r = o.contig_k ? idx >> 4 : idx & 63;
        const int kk = o.contig_k ? idx & 15 : idx >> 6;
        dst[kk][r] = reg[i];
    }
}

__global__ void __launch_bounds__(256) batched_gemm_kernel(BGemm g) {
    __shared__ __align__(16) float As[kBK][kBT + 4];
    __shared__ __align__(16) float Bs[kBK][kBT + 4];
    const int n0 = blockIdx.x * kBT, m0 = blockIdx.y * kBT;
    const int b = blockIdx.z / g.Hz, hz = blockIdx.z % g.Hz;
    int kbeg = 0, kend = g.K;
    if (g.causal_mode == 1 && n0 > m0 + kBT - 1 + g.q_off) return;
    if (g.causal_mode == 2) kend = min(g.K, m0 + kBT + g.q_off);
    if (g.causal_mode == 3 && m0 > g.q_off) kbeg = ((m0 - g.q_off) / kBK) * kBK;
    const float* za = g.a.base + (long long)b * g.a.bs + (long long)(hz / g.a.hdiv) * g.a.hs;
    const float* zb = g.b.base + (long long)b * g.b.bs + (long long)(hz / g.b.hdiv) * g.b.hs;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    float ra[4], rb[4];
    fetch_tile(g.a, za, m0, g.M, kbeg, kend, ra);
    fetch_tile(g.b, zb, n0, g.N, kbeg, kend, rb);
    for (int k0 = kbeg; k0 < kend; k0 += kBK) {
        store_tile(g.a, ra, As);
        store_tile(g.b, rb, Bs);
        __syncthreads();
        if (k0 + kBK < kend) {
            fetch_tile(g.a, za, m0, g.M, k0 + kBK, kend, ra);
            fetch_tile(g.b, zb, n0, g.N, k0 + kBK, kend, rb);
        }
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float a[4] = {av.x, av.y, av.z, av.w}, bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* zc = g.c + (long long)b * g.c_bs + (long long)hz * g.c_hs;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < g.N) zc[(long long)m * g.c_rs + n] = acc[i][j] * g.alpha;
        }
    }
}

// One warp per (batch, head, query) row of scores.  Forward: s <- softmax over the allowed keys, zeros elsewhere.
// Backward (dp != nullptr): s holds scores and dp holds dO.V^T on entry; on exit s = P and dp = dS = P*(dP - sum(P*dP)).
__global__ void __launch_bounds__(256) gqa_rows_kernel(float* __restrict__ s, float* __restrict__ dp, GqaDims p, size_t rows) {
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const int tq = (int)(row % p.tq);
    int k0, k1;
    key_range(p, tq, k0, k1);
    float* sr = s + row * (size_t)p.tk;
    float mx = -FLT_MAX;
    for (int t = k0 + lane; t < k1; t += 32) mx = fmaxf(mx, sr[t]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int t = k0 + lane; t < k1; t += 32) sum += expf(sr[t] - mx);
    sum = warp_sum(sum);
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    if (dp == nullptr) {
        for (int t = lane; t < p.tk; t += 32) sr[t] = (t >= k0 && t < k1) ? expf(sr[t] - mx) * inv : 0.0f;
        return;
    }
    float* dr = dp + row * (size_t)p.tk;
    float dot = 0.0f;
    for (int t = k0 + lane; t < k1; t += 32) dot += expf(sr[t] - mx) * inv * dr[t];
    dot = warp_sum(dot);
    for (int t = lane; t < p.tk; t += 32) {
        float prob = 0.0f, ds = 0.0f;
        if (t >= k0 && t < k1) {
            prob = expf(sr[t] - mx) * inv;
            ds = prob * (dr[t] - dot);
        }
        sr[t] = prob;
        dr[t] = ds;
    }
}

cudaError_t run_bgemm(const BGemm& g, int batch, cudaStream_t stream) {
    dim3 grid((g.N + kBT - 1) / kBT, (g.M + kBT - 1) / kBT, batch * g.Hz);
    batched_gemm_kernel<<<grid, 256, 0, stream>>>(g);
    return cudaGetLastError();
}

// ---- embeddings, rope, adam (kernels/vulkan/token_position_embedding_f32_i32.comp, embedding_gather_f32_i32.comp,
// embedding_weight_backward_f32_i32_scatter.comp, position_embedding_backward_f32_i32.comp, rope_f32.comp,
// rope_split_half_f32.comp, adam_update_fast_f32.comp) ------------------------------------------------------------
// out[t, d] = token_weight[ids[t], d] (0 for an id outside the table) + pos_weight[t % seq_len, d]; pos_weight may be
// NULL (plain gather).
__global__ void __launch_bounds__(256) embedding_kernel(const float* __restrict__ token_weight, const float* __restrict__ pos_weight,
                                                        const int* __restrict__ ids, float* __restrict__ out, size_t tokens,
                                                        int vocab, int seq_len, int dim) {
    const size_t n = tokens * (size_t)dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / dim;
        const int d = (int)(i - t * dim);
        const int id = ids[t];
        float v = (id >= 0 && id < vocab) ? token_weight[(size_t)id * dim + d] : 0.0f;
        if (pos_weight != nullptr) v += pos_weight[(size_t)(t % seq_len) * dim + d];
        out[i] = v;
    }
}
// grad_weight[ids[t], d] += grad_out[t, d]; grad_weight is zeroed by the caller.
__global__ void __launch_bounds__(256) embedding_scatter_kernel(const int* __restrict__ ids, const float* __restrict__ grad_out,
                                                                float* __restrict__ grad_weight, size_t tokens, int vocab,
                                                                int dim) {
    const size_t n = tokens * (size_t)dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / dim;
        const int id = ids[t];
        if (id < 0 || id >= vocab) continue;
        atomicAdd(grad_weight + (size_t)id * dim + (i - t * dim), grad_out[i]);
    }
}
// grad_position[pos, d] = sum over the batch of grad_out[(b*seq_len + pos), d]
__global__ void __launch_bounds__(256) position_backward_kernel(const float* __restrict__ grad_out, float* __restrict__ grad_position,
                                                                int batch, int seq_len, int dim) {
    const size_t n = (size_t)seq_len * dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (int b = 0; b < batch; ++b) acc += grad_out[(size_t)b * n + i];
        grad_position[i] = acc;
    }
}
// Rotary embedding on x [batch*tokens, channels] with n_head heads of head_dim at the front of each row; one thread
// per rotated pair.  split_half pairs (i, i + head_dim/2), otherwise (2i, 2i+1).  inverse negates the angle.
__global__ void __launch_bounds__(256) rope_kernel(const float* __restrict__ x, float* __restrict__ out, size_t rows, int tokens,
                                                   int channels, int n_head, int head_dim, int rotary_dim, int token_offset,
                                                   float theta, int inverse, int split_half) {
    const size_t n = rows * (size_t)channels;
    int rd = rotary_dim <= 0 ? head_dim : rotary_dim;
    rd = rd < head_dim ? rd : head_dim;
    rd -= rd & 1;
    const int half = head_dim >> 1;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / channels;
        const int c = (int)(i - row * channels);
        const int head = c / head_dim, d = c - head * head_dim;
        if (head >= n_head) continue;                 // the shaders leave such channels unwritten
        int pair, lo, hi;                             // pair index and the two channels it rotates
        bool first;
        if (split_half) {
            if (half <= 0 || d >= half * 2) { out[i] = x[i]; continue; }
            pair = d < half ? d : d - half;
            if (pair >= (rd >> 1)) { out[i] = x[i]; continue; }
            lo = pair; hi = half + pair; first = d < half;
        } else {
            if (d >= rd) { out[i] = x[i]; continue; }
            pair = d >> 1;
            lo = d & ~1; hi = lo + 1; first = d == lo;
        }
        const int token = (int)(row % tokens);
        const float exponent = (float)(2 * pair) / (float)head_dim;
        float angle = (float)(token_offset + token) / powf(theta, exponent);
        if (inverse) angle = -angle;
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const size_t base = row * (size_t)channels + (size_t)head * head_dim;
        const float a = x[base + lo], b = x[base + hi];
        out[i] = first ? a * cs - b * sn : (split_half ? b * cs + a * sn : a * sn + b * cs);
    }
}
__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ param, const float* __restrict__ grad, float* __restrict__ m,
                                                   float* __restrict__ v, size_t n, float lr, float beta1, float beta2, float eps,
                                                   float weight_decay, float c1, float c2) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float g = grad[i];
        const float mn = beta1 * m[i] + (1.0f - beta1) * g;
        const float vn = beta2 * v[i] + (1.0f - beta2) * g * g;
        m[i] = mn;
        v[i] = vn;
        const float pv = param[i];
        param[i] = pv - lr * (mn * c1 / (sqrtf(vn * c2) + eps) + weight_decay * pv);
    }
}

int flat_grid(size_t n, int sm_count) {
    size_t blocks = (n + 255) / 256;
    const size_t cap = (size_t)sm_count * 16;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

int row_grid(size_t rows, int sm_count) {
    const size_t cap = (size_t)sm_count * 16;
    return (int)(rows < cap ? rows : cap);
}

}  // namespace

cudaError_t launch_rmsnorm(const float* x, const float* w, float* out, size_t rows, int cols, float eps, int sm_count,
                           cudaStream_t stream) {
    rmsnorm_kernel<<<row_grid(rows, sm_count), 128, 0, stream>>>(x, w, out, nullptr, rows, cols, eps);
    return cudaGetLastError();
}
cudaError_t launch_rmsnorm_backward_x(const float* x, const float* w, const float* dy, float* dx, size_t rows, int cols,
                                      float eps, int sm_count, cudaStream_t stream) {
    rmsnorm_bwd_x_kernel<<<row_grid(rows, sm_count), 128, 0, stream>>>(x, w, dy, dx, rows, cols, eps);
    return cudaGetLastError();
}
cudaError_t launch_rmsnorm_backward_weight(const float* x, const float* dy, float* row_inv, float* dw, size_t rows,
                                           int cols, float eps, int sm_count, cudaStream_t stream) {
    rmsnorm_kernel<<<row_grid(rows, sm_count), 128, 0, stream>>>(x, nullptr, nullptr, row_inv, rows, cols, eps);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(dw, 0, (size_t)cols * sizeof(float), stream);
    if (e != cudaSuccess) return e;
    const int col_blocks = (cols + 31) / 32;
    size_t splits = ((size_t)sm_count * 4 + col_blocks - 1) / col_blocks;
    if (splits > (rows + 63) / 64) splits = (rows + 63) / 64;
    if (splits < 1) splits = 1;
    const size_t rows_per_block = (rows + splits - 1) / splits;
    rmsnorm_bwd_w_kernel<<<dim3(col_blocks, (unsigned)splits), 256, 0, stream>>>(x, dy, row_inv, dw, rows, cols,
                                                                                 rows_per_block);
    return cudaGetLastError();
}
cudaError_t launch_swiglu(const float* packed, float* out, size_t rows, int hidden, int sm_count, cudaStream_t stream) {
    const size_t n = rows * (size_t)hidden;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)sm_count * 16) blocks = (size_t)sm_count * 16;
    swiglu_kernel<<<(int)blocks, 256, 0, stream>>>(packed, out, rows, hidden);
    return cudaGetLastError();
}
cudaError_t launch_swiglu_backward(const float* packed, const float* dy, float* dpacked, size_t rows, int hidden,
                                   int sm_count, cudaStream_t stream) {
    const size_t n = rows * (size_t)hidden;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)sm_count * 16) blocks = (size_t)sm_count * 16;
    swiglu_bwd_kernel<<<(int)blocks, 256, 0, stream>>>(packed, dy, dpacked, rows, hidden);
    return cudaGetLastError();
}
cudaError_t launch_softmax_cross_entropy(const float* logits, const int* targets, float* partial, float* out, size_t rows,
                                         int cols, int sm_count, cudaStream_t stream) {
    ce_kernel<false><<<row_grid(rows, sm_count), 256, 0, stream>>>(logits, targets, partial, nullptr, nullptr, rows, cols);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    mean_kernel<<<1, 256, 0, stream>>>(partial, out, rows, rows);
    return cudaGetLastError();
}
cudaError_t launch_softmax_cross_entropy_backward(const float* logits, const int* targets, const float* grad_out,
                                                  float* grad_logits, size_t rows, int cols, int sm_count,
                                                  cudaStream_t stream) {
    ce_kernel<true><<<row_grid(rows, sm_count), 256, 0, stream>>>(logits, targets, nullptr, grad_out, grad_logits, rows, cols);
    return cudaGetLastError();
}

cudaError_t launch_embedding(const float* token_weight, const float* pos_weight, const int* ids, float* out, size_t tokens,
                             int vocab, int seq_len, int dim, int sm_count, cudaStream_t stream) {
    embedding_kernel<<<flat_grid(tokens * (size_t)dim, sm_count), 256, 0, stream>>>(token_weight, pos_weight, ids, out, tokens,
                                                                                    vocab, seq_len, dim);
    return cudaGetLastError();
}
cudaError_t launch_embedding_scatter(const int* ids, const float* grad_out, float* grad_weight, size_t tokens, int vocab, int dim,
                                     int sm_count, cudaStream_t stream) {
    embedding_scatter_kernel<<<flat_grid(tokens * (size_t)dim, sm_count), 256, 0, stream>>>(ids, grad_out, grad_weight, tokens,
                                                                                            vocab, dim);
    return cudaGetLastError();
}
cudaError_t launch_position_backward(const float* grad_out, float* grad_position, int batch, int seq_len, int dim, int sm_count,
                                     cudaStream_t stream) {
    position_backward_kernel<<<flat_grid((size_t)seq_len * dim, sm_count), 256, 0, stream>>>(grad_out, grad_position, batch,
                                                                                             seq_len, dim);
    return cudaGetLastError();
}
cudaError_t launch_rope(const float* x, float* out, size_t rows, int tokens, int channels, int n_head, int head_dim,
                        int rotary_dim, int token_offset, float theta, int inverse, int split_half, int sm_count,
                        cudaStream_t stream) {
    rope_kernel<<<flat_grid(rows * (size_t)channels, sm_count), 256, 0, stream>>>(x, out, rows, tokens, channels, n_head, head_dim,
                                                                                  rotary_dim, token_offset, theta, inverse,
                                                                                  split_half);
    return cudaGetLastError();
}
cudaError_t launch_adam(float* param, const float* grad, float* m, float* v, size_t n, float lr, float beta1, float beta2,
                        float eps, float weight_decay, float c1, float c2, int sm_count, cudaStream_t stream) {
    adam_kernel<<<flat_grid(n, sm_count), 256, 0, stream>>>(param, grad, m, v, n, lr, beta1, beta2, eps, weight_decay, c1, c2);
    return cudaGetLastError();
}

// scores_ws: batch*n_head*tq*tk floats of scratch.
cudaError_t launch_gqa_forward(const float* q, const float* k, const float* v, float* out, int batch, int tq, int tk,
                               int key_stride, int n_head, int n_kv, int hd, int vhd, int causal, int q_off, int window,
                               float scale, float* scores_ws, cudaStream_t stream, int* launches) {
    GqaDims p{batch, tq, tk, key_stride, n_head, n_kv, hd, vhd, causal, q_off, window, scale};
    const int group = n_head / n_kv;
    const long long qc = (long long)n_head * hd, kc = (long long)n_kv * hd, vc = (long long)n_kv * vhd, oc = (long long)n_head * vhd;
    const long long plane = (long long)tq * tk;
    BGemm s{};
    s.a = BOperand{q, tq * qc, hd, qc, 1, 0, 1, 0, 1};
    s.b = BOperand{k, key_stride * kc, hd, kc, 1, 0, group, 0, 1};
    s.c = scores_ws; s.c_bs = n_head * plane; s.c_hs = plane; s.c_rs = tk;
    s.M = tq; s.N = tk; s.K = hd; s.Hz = n_head; s.alpha = scale; s.causal_mode = causal ? 1 : 0; s.q_off = q_off;
    cudaError_t e = run_bgemm(s, batch, stream);
    if (e != cudaSuccess) return e;
    const size_t rows = (size_t)batch * n_head * tq;
    gqa_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(scores_ws, nullptr, p, rows);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    BGemm o{};
    o.a = BOperand{scores_ws, n_head * plane, plane, tk, 1, 0, 1, 0, 1};
    o.b = BOperand{v, key_stride * vc, vhd, 1, vc, 0, group, 0, 0};
    o.c = out; o.c_bs = tq * oc; o.c_hs = vhd; o.c_rs = oc;
    o.M = tq; o.N = vhd; o.K = tk; o.Hz = n_head; o.alpha = 1.0f; o.causal_mode = causal ? 2 : 0; o.q_off = q_off;
    *launches += 3;
    return run_bgemm(o, batch, stream);
}

// probs and ds (batch*n_head*tq*tk floats each) receive the probabilities and dS, as in the reference.
cudaError_t launch_gqa_backward(const float* q, const float* k, const float* v, const float* dout, float* probs, float* ds,
                                float* dq, float* dk, float* dv, int batch, int tq, int tk, int n_head, int n_kv, int hd,
                                int causal, int q_off, float scale, cudaStream_t stream, int* launches) {
    GqaDims p{batch, tq, tk, tk, n_head, n_kv, hd, hd, causal, q_off, 0, scale};
    const int group = n_head / n_kv;
    const long long qc = (long long)n_head * hd, kc = (long long)n_kv * hd;
    const long long plane = (long long)tq * tk;
    cudaError_t e;
    BGemm g{};
    // scores and dP
    g.a = BOperand{q, tq * qc, hd, qc, 1, 0, 1, 0, 1};
    g.b = BOperand{k, tk * kc, hd, kc, 1, 0, group, 0, 1};
    g.c = probs; g.c_bs = n_head * plane; g.c_hs = plane; g.c_rs = tk;
    g.M = tq; g.N = tk; g.K = hd; g.Hz = n_head; g.alpha = scale; g.causal_mode = causal ? 1 : 0; g.q_off = q_off;
    if ((e = run_bgemm(g, batch, stream)) != cudaSuccess) return e;
    g.a.base = dout; g.b.base = v; g.c = ds; g.alpha = 1.0f;
    if ((e = run_bgemm(g, batch, stream)) != cudaSuccess) return e;
    const size_t rows = (size_t)batch * n_head * tq;
    gqa_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(probs, ds, p, rows);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    // dq = scale * dS K
    BGemm d{};
    d.a = BOperand{ds, n_head * plane, plane, tk, 1, 0, 1, 0, 1};
    d.b = BOperand{k, tk * kc, hd, 1, kc, 0, group, 0, 0};
    d.c = dq; d.c_bs = tq * qc; d.c_hs = hd; d.c_rs = qc;
    d.M = tq; d.N = hd; d.K = tk; d.Hz = n_head; d.alpha = scale; d.causal_mode = causal ? 2 : 0; d.q_off = q_off;
    if ((e = run_bgemm(d, batch, stream)) != cudaSuccess) return e;
    // dv = P^T dO and dk = scale * dS^T Q, summed over the query heads of each kv head
    BGemm t{};
    t.a = BOperand{probs, n_head * plane, group * plane, 1, tk, plane, 1, tq, 0};
    t.b = BOperand{dout, tq * qc, (long long)group * hd, 1, qc, hd, 1, tq, 0};
    t.c = dv; t.c_bs = tk * kc; t.c_hs = hd; t.c_rs = kc;
    t.M = tk; t.N = hd; t.K = group * tq; t.Hz = n_kv; t.alpha = 1.0f; t.causal_mode = causal ? 3 : 0; t.q_off = q_off;
    if ((e = run_bgemm(t, batch, stream)) != cudaSuccess) return e;
    t.a.base = ds; t.b.base = q; t.c = dk; t.alpha = scale;
    *launches += 6;
    return run_bgemm(t, batch, stream);
}

// ---- mean squared error: the three kernels of MotifCL's OpenCL loss (kernels/loss.cl:1-43, src/ops/loss.cpp:21-95) ----
// The summation orders are the reference's own, so the loss is the same float: a partial sum per chunk of 256 elements,
// left to right; then 256 lanes that stride over the partial sums, a 128..1 tree, and one division.
namespace {
__global__ void mse_partial_kernel(const float* __restrict__ pred, const float* __restrict__ target,
                                   float* __restrict__ partial, long long n, long long chunks) {
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= chunks) return;
    const long long start = g * 256;
    float acc = 0.0f;
    for (int i = 0; i < 256; ++i) {
        const long long idx = start + i;
        if (idx < n) {
            const float d = __fsub_rn(pred[idx], target[idx]);
            acc = __fadd_rn(acc, __fmul_rn(d, d));
        }
    }
    partial[g] = acc;
}
__global__ void __launch_bounds__(256) mean_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                          int count, int denominator) {
    __shared__ float scratch[256];
    const int lid = threadIdx.x;
    float acc = 0.0f;
    for (int i = lid; i < count; i += 256) acc = __fadd_rn(acc, partial[i]);
    scratch[lid] = acc;
    __syncthreads();
    for (int stride = 128; stride > 0; stride >>= 1) {
        if (lid < stride) scratch[lid] = __fadd_rn(scratch[lid], scratch[lid + stride]);
        __syncthreads();
    }
    if (lid == 0) out[0] = denominator > 0 ? __fdiv_rn(scratch[0], (float)denominator) : 0.0f;
}
__global__ void mse_backward_kernel(const float* __restrict__ pred, const float* __restrict__ target,
                                    const float* __restrict__ grad_out, float* __restrict__ grad_pred, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
        grad_pred[i] = __fdiv_rn(__fmul_rn(__fmul_rn(grad_out[0], 2.0f), __fsub_rn(pred[i], target[i])), (float)n);
}
}  // namespace

cudaError_t launch_mse_loss_partial(const float* pred, const float* target, float* partial, size_t n, cudaStream_t stream) {
    const long long chunks = (long long)((n + 255) / 256);
    mse_partial_kernel<<<(unsigned)((chunks + 127) / 128), 128, 0, stream>>>(pred, target, partial, (long long)n, chunks);
    return cudaGetLastError();
}
cudaError_t launch_mean_reduce(const float* partial, float* out, int count, int denominator, cudaStream_t stream) {
    mean_reduce_kernel<<<1, 256, 0, stream>>>(partial, out, count, denominator);
    return cudaGetLastError();
}
cudaError_t launch_mse_backward(const float* pred, const float* target, const float* grad_out, float* grad_pred, size_t n,
                                cudaStream_t stream) {
    mse_backward_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(pred, target, grad_out, grad_pred, (long long)n);
    return cudaGetLastError();
}

}  // namespace mcl
