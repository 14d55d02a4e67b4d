// mcl_cuda_counter_update_fused_static: the memory-native counter update for callers that
// must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc / cudaFree are off limits -- a host that has
// handed all device memory to its own arena up front and forbids allocations afterwards, a
// plugin called inside a real-time or latency-critical loop where an allocation would
// synchronise the device, or a caller that only owns a stream and a few buffers and no
// library context.  The ordinary entry point (mcl_cuda_counter_update_fused) keeps its
// grad_w row tile in a workspace that the context grows with cudaMalloc on demand; this
// variant keeps that tile in a fixed array that is part of the library image instead.
//
// The scratch: MCL_STATIC_SCRATCH_FLOATS floats (4 MiB) in a file-scope __device__ array.
// Every GPU that loads this library holds those 4 MiB until the process exits.  All calls on
// a device share the one array: two calls that overlap on the GPU (different streams, or
// different host threads) race on it and corrupt each other -- serialise them on one stream.
// The array keeps the previous call's contents; nothing here relies on it starting at zero,
// because every row tile is fully overwritten by the gradient kernel before the update
// kernel reads it.
//
// Limit: one gradient row must fit, in_features <= MCL_STATIC_SCRATCH_FLOATS (1,048,576);
// shapes beyond that are refused with a message.  (The update kernel additionally needs a
// row to fit in shared memory, as in the ordinary entry point.)
//
// Set-up: the first call on each device looks up the device address of the array with
// cudaGetSymbolAddress while that device is current, and caches it.  In host code the
// array's name is only a host-side handle, not a device address, so kernels are always given
// the looked-up pointer.  Make that first call before any stream capture.
#include <cmath>
#include <mutex>
#include <string>

#include "kernels.h"
#include "motifcl_cuda.h"

#define MCL_STATIC_SCRATCH_FLOATS (1u << 20)

namespace {

static __device__ __align__(256) float g_static_scratch[MCL_STATIC_SCRATCH_FLOATS];

struct DeviceSetup {
    bool ready = false;
    float* scratch = nullptr;
    int sm_count = 0;
    size_t max_smem = 0;
};
constexpr int kMaxDevices = 64;
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;
thread_local std::string g_static_error;

int refuse(int code, const std::string& msg) {
    g_static_error = msg;
    return code;
}

// Once per device, with that device current: resolve the array's device address and read the
// two device attributes the launchers need.  No allocation happens here.
int setup_device(int dev, DeviceSetup** out) {
    if (dev < 0 || dev >= kMaxDevices) return refuse(MCL_CUDA_EINVAL, "static update: device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    DeviceSetup& s = g_setup[dev];
    if (!s.ready) {
        float* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return refuse(MCL_CUDA_ECUDA, std::string("static update: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
        int sms = 0, smem = 0, major = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess)
            return refuse(MCL_CUDA_ECUDA, std::string("static update: device query failed: ") + cudaGetErrorString(e));
        if (major != 10) return refuse(MCL_CUDA_EUNSUPPORTED, "static update: this library is built for sm_100a only");
        s.scratch = ptr;
        s.sm_count = sms;
        s.max_smem = (size_t)smem;
        s.ready = true;
    }
    *out = &s;
    return MCL_CUDA_OK;
}

}  // namespace

extern "C" {

const char* mcl_cuda_static_last_error(void) { return g_static_error.c_str(); }

size_t mcl_cuda_static_scratch_floats(void) { return MCL_STATIC_SCRATCH_FLOATS; }

int mcl_cuda_counter_update_fused_static(void* cuda_stream, uint8_t* state, float* scale, float* v,
                                         const float* grad_out, const float* x, uint32_t* packed2_out,
                                         size_t C, size_t in_features, size_t out_features, size_t batch,
                                         float lr, float lr_scale, float rms_beta, float rms_eps,
                                         uint32_t seed) {
    // the refusals of the ordinary entry point, made before anything is launched
    if (C == 0 || in_features == 0 || out_features == 0 || batch == 0)
        return refuse(MCL_CUDA_EINVAL, "static update requires non-zero dimensions");
    if (in_features % 4 != 0) return refuse(MCL_CUDA_EINVAL, "static update requires in_features % 4 == 0");
    if (C > 32 || 3 * (2 * C - 1) > 64) return refuse(MCL_CUDA_EINVAL, "static update: C too large for 6-bit packed state encoding");
    if (in_features > MCL_STATIC_SCRATCH_FLOATS)
        return refuse(MCL_CUDA_EINVAL, "static update: in_features " + std::to_string(in_features) +
                                           " exceeds the built-in scratch of " +
                                           std::to_string(MCL_STATIC_SCRATCH_FLOATS) + " floats (one gradient row must fit)");
    if (out_features > 0x7fffffffull || batch > 0x7fffffffull || in_features * out_features > 0x7fffffffull)
        return refuse(MCL_CUDA_EINVAL, "static update: out_features * in_features exceeds 32-bit element indexing");
    if (!std::isfinite(lr) || !std::isfinite(lr_scale) || !std::isfinite(rms_beta))
        return refuse(MCL_CUDA_EINVAL, "static update requires finite lr, lr_scale and rms_beta");
    if (!std::isfinite(rms_eps) || rms_eps < 0.0f)
        return refuse(MCL_CUDA_EINVAL, "static update requires non-negative finite rms_eps");
    if (!state || !scale || !v || !grad_out || !x) return refuse(MCL_CUDA_EINVAL, "static update: NULL pointer");
    {   // fp32 / uint32 tensors are read with 32-bit accesses: a misaligned one would fault on the device
        const struct { const char* name; const void* p; } al[] = {
            {"grad_out", grad_out}, {"x", x}, {"scale", scale}, {"v", v}, {"packed2_out", packed2_out}};
        for (const auto& a : al)
            if (a.p && reinterpret_cast<uintptr_t>(a.p) % 4 != 0)
                return refuse(MCL_CUDA_EINVAL, std::string("static update: ") + a.name + " must be 4-byte aligned");
    }
    if (packed2_out && in_features % 16 != 0)
        return refuse(MCL_CUDA_EINVAL, "static update: packed2 output requires in_features % 16 == 0");

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return refuse(MCL_CUDA_ECUDA, std::string("static update: ") + cudaGetErrorString(e));
    DeviceSetup* s = nullptr;
    int rc = setup_device(dev, &s);
    if (rc != MCL_CUDA_OK) return rc;

    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    float* gw = s->scratch;                       // device address from cudaGetSymbolAddress
    size_t tile_rows = MCL_STATIC_SCRATCH_FLOATS / in_features;
    if (tile_rows > out_features) tile_rows = out_features;
    const size_t state_row = in_features / 4 * 3;
    for (size_t r0 = 0; r0 < out_features; r0 += tile_rows) {
        const size_t nr = (out_features - r0 < tile_rows) ? out_features - r0 : tile_rows;
        // rows [r0, r0+nr) of grad_out^T x, k ascending with unfused multiply-add: overwrites the tile
        e = mcl::launch_simt_grad_w(grad_out, x, gw, (int)batch, (int)in_features, (int)out_features, (int)r0,
                                    (int)nr, stream);
        if (e != cudaSuccess) return refuse(MCL_CUDA_ECUDA, std::string("static update (grad_w tile): ") + cudaGetErrorString(e));
        e = mcl::launch_counter_update_dense(state + r0 * state_row, scale + r0, v + r0, gw,
                                             packed2_out ? packed2_out + r0 * (in_features / 16) : nullptr, (int)C,
                                             (int)in_features, (int)nr, (int)r0, lr, lr_scale, rms_beta, rms_eps,
                                             seed, nullptr, nullptr, s->sm_count, s->max_smem, stream);
        if (e == cudaErrorInvalidConfiguration)
            return refuse(MCL_CUDA_EUNSUPPORTED, "static update: in_features too large for one row in shared memory");
        if (e != cudaSuccess) return refuse(MCL_CUDA_ECUDA, std::string("static update: ") + cudaGetErrorString(e));
    }
    return MCL_CUDA_OK;
}

}  // extern "C"
