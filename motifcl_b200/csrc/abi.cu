// C-ABI layer of libmotifcl_cuda.so: contexts, argument checks, dispatch to the kernels.
// The declarations and the reference interfaces they replace are in include/motifcl_cuda.h.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>

#include "kernels.h"
#include "motifcl_cuda.h"

struct mcl_cuda_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int sm_count = 0;
    size_t max_smem = 0;
    std::string name;
    std::string error;
    uint64_t launches = 0;
    // grow-only workspace used by entry points that need scratch (row tiles of grad_w, ...)
    void* ws = nullptr;
    size_t ws_bytes = 0;
};

namespace {

thread_local std::string g_error;   // errors raised before a context exists

int fail(mcl_cuda_ctx* ctx, int code, const std::string& msg) {
    if (ctx) ctx->error = msg; else g_error = msg;
    return code;
}
int fail_cuda(mcl_cuda_ctx* ctx, const char* what, cudaError_t e) {
    return fail(ctx, MCL_CUDA_ECUDA, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// Shared checks, worded after the reference's wrappers (src/runtime/vulkan_backend.cpp:8497-8521).
int check_counter_dims(mcl_cuda_ctx* ctx, const char* op, size_t C, size_t in_features,
                       size_t out_features) {
    const std::string o(op);
    if (C == 0 || in_features == 0 || out_features == 0)
        return fail(ctx, MCL_CUDA_EINVAL, o + " requires non-zero dimensions");
    if (in_features % 4 != 0) return fail(ctx, MCL_CUDA_EINVAL, o + " requires in_features % 4 == 0");
    if (C > 32 || 3 * (2 * C - 1) > 64)
        return fail(ctx, MCL_CUDA_EINVAL, o + ": C too large for 6-bit packed state encoding");
    if (in_features > 0x7fffffffull || out_features > 0x7fffffffull ||
        in_features * out_features > 0x7fffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, o + ": out_features * in_features exceeds 32-bit element indexing");
    return MCL_CUDA_OK;
}
int check_ptr(mcl_cuda_ctx* ctx, const char* op, const char* name, const void* p, size_t align) {
    if (p == nullptr) return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + ": " + name + " is NULL");
    if (reinterpret_cast<uintptr_t>(p) % align != 0)
        return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + ": " + name + " must be " + std::to_string(align) + "-byte aligned");
    return MCL_CUDA_OK;
}
int check_hypers(mcl_cuda_ctx* ctx, const char* op, float lr, float lr_scale, float rms_beta, float rms_eps) {
    const std::string o(op);
    if (!std::isfinite(lr)) return fail(ctx, MCL_CUDA_EINVAL, o + " requires finite lr");
    if (!std::isfinite(lr_scale)) return fail(ctx, MCL_CUDA_EINVAL, o + " requires finite lr_scale");
    if (!std::isfinite(rms_beta)) return fail(ctx, MCL_CUDA_EINVAL, o + " requires finite rms_beta");
    if (!std::isfinite(rms_eps) || rms_eps < 0.0f)
        return fail(ctx, MCL_CUDA_EINVAL, o + " requires non-negative finite rms_eps");
    return MCL_CUDA_OK;
}

int ws_reserve(mcl_cuda_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->ws_bytes) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return fail_cuda(ctx, "workspace sync", e);
        if (ctx->ws) cudaFree(ctx->ws);
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
        e = cudaMalloc(&ctx->ws, bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(ctx, MCL_CUDA_ENOMEM, "workspace allocation of " + std::to_string(bytes) + " bytes failed");
        }
        ctx->ws_bytes = bytes;
    }
    *out = ctx->ws;
    return MCL_CUDA_OK;
}

#define MCL_TRY(expr) do { int _rc = (expr); if (_rc != MCL_CUDA_OK) return _rc; } while (0)
#define MCL_NEED_CTX(ctx) do { if (!(ctx)) return fail(nullptr, MCL_CUDA_EINVAL, "context is NULL"); } while (0)
#define MCL_LAUNCH(ctx, what, call) do { cudaError_t _e = (call); if (_e != cudaSuccess) return fail_cuda(ctx, what, _e); ++(ctx)->launches; } while (0)

int create_impl(int device, cudaStream_t stream, bool own, mcl_cuda_ctx** out_ctx) {
    if (!out_ctx) return fail(nullptr, MCL_CUDA_EINVAL, "out_ctx is NULL");
    *out_ctx = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return fail(nullptr, MCL_CUDA_ENODEVICE, "no CUDA device available");
    }
    if (device < 0 || device >= n) return fail(nullptr, MCL_CUDA_EINVAL, "device index out of range");
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail_cuda(nullptr, "cudaGetDeviceProperties", e);
    if (prop.major != 10)
        return fail(nullptr, MCL_CUDA_EUNSUPPORTED,
                    std::string("this library is built for sm_100a only; device is ") + prop.name +
                        " (sm_" + std::to_string(prop.major) + std::to_string(prop.minor) + ")");
    mcl_cuda_ctx* ctx = new (std::nothrow) mcl_cuda_ctx();
    if (!ctx) return fail(nullptr, MCL_CUDA_ENOMEM, "out of host memory");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->max_smem = prop.sharedMemPerBlockOptin;
    ctx->name = prop.name;
    DeviceGuard guard(device);
    if (own) {
        e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) { delete ctx; return fail_cuda(nullptr, "cudaStreamCreate", e); }
        ctx->own_stream = true;
    } else {
        ctx->stream = stream;
    }
    *out_ctx = ctx;
    return MCL_CUDA_OK;
}

}  // namespace

extern "C" {

int mcl_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}
int mcl_cuda_create(int device, mcl_cuda_ctx** out_ctx) { return create_impl(device, nullptr, true, out_ctx); }
int mcl_cuda_create_on_stream(int device, void* cuda_stream, mcl_cuda_ctx** out_ctx) {
    return create_impl(device, static_cast<cudaStream_t>(cuda_stream), false, out_ctx);
}
void mcl_cuda_destroy(mcl_cuda_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}
const char* mcl_cuda_last_error(mcl_cuda_ctx* ctx) { return ctx ? ctx->error.c_str() : g_error.c_str(); }
const char* mcl_cuda_device_name(mcl_cuda_ctx* ctx) { return ctx ? ctx->name.c_str() : ""; }
int mcl_cuda_sm_count(mcl_cuda_ctx* ctx) { return ctx ? ctx->sm_count : 0; }
uint64_t mcl_cuda_launch_count(mcl_cuda_ctx* ctx) { return ctx ? ctx->launches : 0; }

int mcl_cuda_finish(mcl_cuda_ctx* ctx) {
    MCL_NEED_CTX(ctx);
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "finish", e);
    return MCL_CUDA_OK;
}
int mcl_cuda_alloc(mcl_cuda_ctx* ctx, size_t bytes, void** out_dptr) {
    MCL_NEED_CTX(ctx);
    if (!out_dptr) return fail(ctx, MCL_CUDA_EINVAL, "alloc: out_dptr is NULL");
    *out_dptr = nullptr;
    if (bytes == 0) return fail(ctx, MCL_CUDA_EINVAL, "alloc: zero-size buffer");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaMalloc(out_dptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, MCL_CUDA_ENOMEM, "alloc of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e));
    }
    return MCL_CUDA_OK;
}
int mcl_cuda_free(mcl_cuda_ctx* ctx, void* dptr) {
    MCL_NEED_CTX(ctx);
    if (!dptr) return MCL_CUDA_OK;
    DeviceGuard guard(ctx->device);
    // Work that still uses the buffer may be queued: wait for the stream first, which keeps
    // the reference's "free while pending is safe" behaviour.
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "free", e);
    e = cudaFree(dptr);
    if (e != cudaSuccess) return fail_cuda(ctx, "free", e);
    return MCL_CUDA_OK;
}
int mcl_cuda_upload(mcl_cuda_ctx* ctx, void* dst, const void* src_host, size_t bytes) {
    MCL_NEED_CTX(ctx);
    if (bytes == 0) return MCL_CUDA_OK;
    if (!dst || !src_host) return fail(ctx, MCL_CUDA_EINVAL, "upload: NULL pointer");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "upload", e);
    // pageable sources are staged before the call returns; pinned ones are read later, so
    // wait to give upload the reference's synchronous semantics (src/tensor/tensor.cpp:311-348)
    e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "upload", e);
    return MCL_CUDA_OK;
}
int mcl_cuda_download(mcl_cuda_ctx* ctx, void* dst_host, const void* src, size_t bytes) {
    MCL_NEED_CTX(ctx);
    if (bytes == 0) return MCL_CUDA_OK;
    if (!dst_host || !src) return fail(ctx, MCL_CUDA_EINVAL, "download: NULL pointer");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "download", e);
    e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "download", e);
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_decode_weight(mcl_cuda_ctx* ctx, const uint8_t* state, const float* scale,
                                   float* weight, size_t in_features, size_t out_features, size_t C) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter decode_weight";
    MCL_TRY(check_counter_dims(ctx, op, C, in_features, out_features));
    MCL_TRY(check_ptr(ctx, op, "state", state, 1));
    MCL_TRY(check_ptr(ctx, op, "scale", scale, 4));
    MCL_TRY(check_ptr(ctx, op, "weight", weight, 16));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_decode_weight(state, scale, weight, (int)C, (int)in_features,
                                                  (int)out_features, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_pack2(mcl_cuda_ctx* ctx, const uint8_t* state, uint32_t* packed2,
                           size_t in_features, size_t out_features, size_t C) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter pack2";
    MCL_TRY(check_counter_dims(ctx, op, C, in_features, out_features));
    if (in_features % 16 != 0) return fail(ctx, MCL_CUDA_EINVAL, "counter pack2 requires in_features % 16 == 0");
    MCL_TRY(check_ptr(ctx, op, "state", state, 4));
    MCL_TRY(check_ptr(ctx, op, "packed2", packed2, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_pack2(state, packed2, (int)C, (int)in_features, (int)out_features,
                                          ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_forward(mcl_cuda_ctx* ctx, const float* x, const uint8_t* state,
                             const float* scale, float* y, size_t batch, size_t in_features,
                             size_t out_features, size_t C) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter forward";
    MCL_TRY(check_counter_dims(ctx, op, C, in_features, out_features));
    if (batch == 0 || batch > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "counter forward requires 0 < batch < 2^31");
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "state", state, 1));
    MCL_TRY(check_ptr(ctx, op, "scale", scale, 4));
    MCL_TRY(check_ptr(ctx, op, "y", y, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_simt_counter_forward(x, state, scale, y, (int)batch, (int)in_features,
                                                         (int)out_features, (int)C, ctx->stream));
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_backward_input(mcl_cuda_ctx* ctx, const uint8_t* state, const float* scale,
                                    const float* grad_out, float* grad_x, size_t batch,
                                    size_t in_features, size_t out_features, size_t C) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter backward_input";
    MCL_TRY(check_counter_dims(ctx, op, C, in_features, out_features));
    if (batch == 0 || batch > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "counter backward_input requires 0 < batch < 2^31");
    MCL_TRY(check_ptr(ctx, op, "state", state, 1));
    MCL_TRY(check_ptr(ctx, op, "scale", scale, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_x", grad_x, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_simt_counter_backward_input(state, scale, grad_out, grad_x, (int)batch,
                                                                (int)in_features, (int)out_features,
                                                                (int)C, ctx->stream));
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_update_dense(mcl_cuda_ctx* ctx, uint8_t* state, float* scale, float* v,
                                  const float* grad_w, uint32_t* packed2_out, size_t C,
                                  size_t in_features, size_t rows, size_t row_offset, float lr,
                                  float lr_scale, float rms_beta, float rms_eps, uint32_t seed) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter update";
    MCL_TRY(check_counter_dims(ctx, op, C, in_features, rows));
    MCL_TRY(check_hypers(ctx, op, lr, lr_scale, rms_beta, rms_eps));
    if ((row_offset + rows) * in_features > 0xffffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, "counter update: (row_offset + rows) * in_features exceeds 32-bit element indexing");
    MCL_TRY(check_ptr(ctx, op, "state", state, 1));
    MCL_TRY(check_ptr(ctx, op, "scale", scale, 4));
    MCL_TRY(check_ptr(ctx, op, "v", v, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_w", grad_w, 16));
    if (packed2_out) {
        if (in_features % 16 != 0) return fail(ctx, MCL_CUDA_EINVAL, "counter update: packed2 output requires in_features % 16 == 0");
        MCL_TRY(check_ptr(ctx, op, "packed2_out", packed2_out, 4));
    }
    DeviceGuard guard(ctx->device);
    cudaError_t e = mcl::launch_counter_update_dense(state, scale, v, grad_w, packed2_out, (int)C,
                                                     (int)in_features, (int)rows, (int)row_offset, lr,
                                                     lr_scale, rms_beta, rms_eps, seed, ctx->sm_count,
                                                     ctx->max_smem, ctx->stream);
    if (e == cudaErrorInvalidConfiguration)
        return fail(ctx, MCL_CUDA_EUNSUPPORTED, "counter update: in_features too large for one row in shared memory");
    if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    ++ctx->launches;
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_update_fused(mcl_cuda_ctx* ctx, uint8_t* state, float* scale, float* v,
                                  const float* grad_out, const float* x, float* scale_new_scratch,
                                  float* denom_scratch, uint32_t* packed2_out, size_t C,
                                  size_t in_features, size_t out_features, size_t batch, float lr,
                                  float lr_scale, float rms_beta, float rms_eps, uint32_t seed) {
    (void)scale_new_scratch; (void)denom_scratch;
    MCL_NEED_CTX(ctx);
    const char* op = "counter update";
    MCL_TRY(check_counter_dims(ctx, op, C, in_features, out_features));
    if (batch == 0 || batch > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "counter update requires 0 < batch < 2^31");
    MCL_TRY(check_hypers(ctx, op, lr, lr_scale, rms_beta, rms_eps));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "state", state, 1));
    if (packed2_out && in_features % 16 != 0)
        return fail(ctx, MCL_CUDA_EINVAL, "counter update: packed2 output requires in_features % 16 == 0");
    // Row tile of grad_w: at most 1/8 of the dense [out,in] gradient (and at most 32 MiB),
    // at least one row; rounded to a multiple of 64 rows when that fits.
    const size_t row_b = in_features * sizeof(float);
    size_t budget = out_features * row_b / 8;
    if (budget > (32u << 20)) budget = 32u << 20;
    size_t tile_rows = budget / row_b;
    if (tile_rows < 1) tile_rows = 1;
    if (tile_rows > 64) tile_rows &= ~size_t(63);
    if (tile_rows > out_features) tile_rows = out_features;
    void* wsp = nullptr;
    DeviceGuard guard(ctx->device);
    MCL_TRY(ws_reserve(ctx, tile_rows * row_b, &wsp));
    float* gw = static_cast<float*>(wsp);
    const size_t state_row = in_features / 4 * 3;
    for (size_t r0 = 0; r0 < out_features; r0 += tile_rows) {
        const size_t nr = (out_features - r0 < tile_rows) ? out_features - r0 : tile_rows;
        MCL_LAUNCH(ctx, "counter update (grad_w tile)",
                   mcl::launch_simt_grad_w(grad_out, x, gw, (int)batch, (int)in_features,
                                           (int)out_features, (int)r0, (int)nr, ctx->stream));
        int rc = mcl_cuda_counter_update_dense(ctx, state + r0 * state_row, scale + r0, v + r0, gw,
                                               packed2_out ? packed2_out + r0 * (in_features / 16) : nullptr,
                                               C, in_features, nr, r0, lr, lr_scale, rms_beta, rms_eps, seed);
        if (rc != MCL_CUDA_OK) return rc;
    }
    return MCL_CUDA_OK;
}

int mcl_cuda_matmul_f32(mcl_cuda_ctx* ctx, const float* a, const float* b, float* c, size_t M,
                        size_t K, size_t N, int trans_a, int trans_b) {
    MCL_NEED_CTX(ctx);
    const char* op = "matmul_f32";
    if (M == 0 || N == 0 || K == 0) return fail(ctx, MCL_CUDA_EINVAL, "matmul_f32 requires non-zero dimensions");
    if (M > 0x7fffffffull || N > 0x7fffffffull || K > 0x7fffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, "matmul_f32 dimension exceeds 2^31");
    MCL_TRY(check_ptr(ctx, op, "a", a, 4));
    MCL_TRY(check_ptr(ctx, op, "b", b, 4));
    MCL_TRY(check_ptr(ctx, op, "c", c, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_simt_matmul_f32(a, b, c, (int)M, (int)K, (int)N, trans_a, trans_b, ctx->stream));
    return MCL_CUDA_OK;
}

int mcl_cuda_ternary_gemv(mcl_cuda_ctx* ctx, const float* x, const uint32_t* packed2,
                          const float* scale, float* y, size_t M, size_t in_features,
                          size_t out_features) {
    MCL_NEED_CTX(ctx);
    const char* op = "ternary gemv";
    if (M == 0 || in_features == 0 || out_features == 0) return fail(ctx, MCL_CUDA_EINVAL, "ternary gemv requires non-zero dimensions");
    if (M > 16) return fail(ctx, MCL_CUDA_EINVAL, "ternary gemv serves M <= 16; use counter forward for larger batches");
    if (in_features % 16 != 0) return fail(ctx, MCL_CUDA_EINVAL, "ternary gemv requires in_features % 16 == 0");
    if (in_features > 0x7fffffffull || out_features > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "ternary gemv dimension exceeds 2^31");
    MCL_TRY(check_ptr(ctx, op, "x", x, 16));
    MCL_TRY(check_ptr(ctx, op, "packed2", packed2, 4));
    MCL_TRY(check_ptr(ctx, op, "scale", scale, 4));
    MCL_TRY(check_ptr(ctx, op, "y", y, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_ternary_gemv(x, packed2, scale, y, (int)M, (int)in_features,
                                                 (int)out_features, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}

}  // extern "C"
