// MotifCL's OpenCL seam served by libmotifcl_cuda.so.
//
// MotifCL's OpenCL backend reaches its device through 28 C entry points of libOpenCL (MotifCL cmake/OpenCL.def; its
// src/runtime/opencl_disabled_stub.cpp stubs the same list when OpenCL is off) and picks kernels by NAME out of .cl
// programs that it compiles at run time (src/runtime/backend.cpp:161-200, src/runtime/program.cpp:11-66).  This file
// defines those entry points on top of the C ABI of include/motifcl_cuda.h and is linked in the place of the disabled
// stub, so Backend::create_opencl() returns a backend whose "OpenCL device" is the B200:
//   * one platform, one GPU device, one context (one mcl_cuda_ctx, one in-order stream), buffers = device memory;
//   * programs are accepted and their text is ignored; clCreateKernel knows the kernels listed in kKernels below
//     (the counter kernels of kernels/compact_counter.cl, the f32 matmuls of kernels/matmul.cl and the generated tiled
//     ones, the mean-squared-error kernels of kernels/loss.cl, the elementwise helpers of kernels/basic.cl that
//     autograd calls) and answers CL_INVALID_KERNEL_NAME for every other name, so a gap fails with its name;
//   * clSetKernelArg stores bytes, clEnqueueNDRangeKernel decodes them by the kernel's signature and calls the ABI.
// The dense and the memory-native counter update are THREE launches in MotifCL (row statistics, tick, copy of the new
// scales: src/nn/compact_counter.cpp:113-231).  The ABI has them as one fused kernel, so the row-statistics launch is
// remembered, the tick launch runs the fused update (state, scale and v in place) and stores the new scales into
// scale_new as well, and the copy launch that follows rewrites the same values.  Nothing reads scale_new, denom or v
// between those launches in MotifCL.
//
// With it MotifCL's tests/test_counter_state.cpp and tests/test_memory_truth_gate.cpp, and through them the dense
// CounterStateLinear::apply_update_seed, run unchanged (Makefile: test_counter_state, test_memory_truth_gate).
#include <CL/cl.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "motifcl_cuda.h"

struct _cl_platform_id { int unused; };
struct _cl_device_id { int index; };
struct _cl_context {
    std::atomic<int> refs{1};
    mcl_cuda_ctx* ctx = nullptr;
    // the row-statistics launch of a counter update, waiting for its tick launch
    struct Pending {
        bool valid = false, fused = false;
        void *state = nullptr, *scale = nullptr, *v = nullptr, *grad = nullptr, *x = nullptr, *scale_new = nullptr;
        int C = 0, in = 0, out = 0, N = 0;
        float lr_scale = 0.f, beta = 0.f, eps = 0.f;
    } pending;
};
struct _cl_command_queue { std::atomic<int> refs{1}; _cl_context* context; };
struct _cl_mem {
    std::atomic<int> refs{1};
    _cl_context* context = nullptr;
    char* dptr = nullptr;
    size_t size = 0;
    _cl_mem* parent = nullptr;      // sub-buffers share the parent's memory
};
struct _cl_program { std::atomic<int> refs{1}; _cl_context* context; };
struct _cl_kernel {
    std::atomic<int> refs{1};
    _cl_context* context = nullptr;
    int id = -1;
    std::string name;
    std::vector<std::vector<unsigned char>> args;
};
struct _cl_event { std::atomic<int> refs{1}; };

namespace {

_cl_platform_id g_platform;
_cl_device_id g_device{0};
mcl_cuda_ctx* g_ctx = nullptr;          // created with the first device query: device names need a context

mcl_cuda_ctx* shared_ctx() {
    if (!g_ctx && mcl_cuda_device_count() > 0) {
        if (mcl_cuda_create(0, &g_ctx) != MCL_CUDA_OK) g_ctx = nullptr;
    }
    return g_ctx;
}

enum KernelId {
    K_DECODE, K_ROW_STATS, K_APPLY, K_ROW_STATS_FUSED, K_APPLY_FUSED, K_BACKWARD_INPUT,
    K_MM_NN, K_MM_TA, K_MM_TB, K_MM_FLAGS,
    K_MSE_PARTIAL, K_MEAN_REDUCE, K_MSE_BACKWARD,
    K_FILL, K_COPY, K_ADD, K_SUB, K_MUL, K_ADD_SCALAR, K_MUL_SCALAR, K_SCALE, K_ADD_INPLACE,
};
struct KernelEntry { const char* name; int id; int nargs; };
const KernelEntry kKernels[] = {
    // kernels/compact_counter.cl
    {"decode_counter_state_weight_f32", K_DECODE, 6},
    {"counter_row_stats_f32", K_ROW_STATS, 12},
    {"counter_apply_update_f32", K_APPLY, 10},
    {"counter_row_stats_fused_f32", K_ROW_STATS_FUSED, 14},
    {"counter_apply_update_fused_f32", K_APPLY_FUSED, 13},
    {"counter_backward_input_f32", K_BACKWARD_INPUT, 8},
    // kernels/matmul.cl and the tiled kernels MotifCL generates (src/runtime/backend.cpp:102-131): all (A, B, C, M, N, K)
    {"matmul_register_block4_f32", K_MM_NN, 6}, {"matmul_register_block4_k512_f32", K_MM_NN, 6},
    {"matmul_tiled_f32_t4", K_MM_NN, 6}, {"matmul_tiled_f32_t8", K_MM_NN, 6}, {"matmul_tiled_f32_t16", K_MM_NN, 6},
    {"matmul_transa_rb4_f32", K_MM_TA, 6}, {"matmul_transa_rb4_k512_f32", K_MM_TA, 6},
    {"matmul_transb_rb4_f32", K_MM_TB, 6}, {"matmul_transb_rb4_k512_f32", K_MM_TB, 6},
    {"matmul_flags_f32", K_MM_FLAGS, 8},
    // kernels/loss.cl
    {"mse_loss_partial_f32", K_MSE_PARTIAL, 4}, {"mean_reduce_f32", K_MEAN_REDUCE, 4}, {"mse_backward_f32", K_MSE_BACKWARD, 5},
    // kernels/basic.cl
    {"fill_f32", K_FILL, 3}, {"copy_f32", K_COPY, 3}, {"add_f32", K_ADD, 4}, {"sub_f32", K_SUB, 4}, {"mul_f32", K_MUL, 4},
    {"add_scalar_f32", K_ADD_SCALAR, 4}, {"mul_scalar_f32", K_MUL_SCALAR, 4}, {"scale_f32", K_SCALE, 3},
    {"add_inplace_f32", K_ADD_INPLACE, 3},
};

cl_int put(const void* src, size_t bytes, size_t avail, void* dst, size_t* ret) {
    if (ret) *ret = bytes;
    if (dst) {
        if (avail < bytes) return CL_INVALID_VALUE;
        std::memcpy(dst, src, bytes);
    }
    return CL_SUCCESS;
}
cl_int put_string(const char* s, size_t avail, void* dst, size_t* ret) { return put(s, std::strlen(s) + 1, avail, dst, ret); }

cl_int failed(_cl_context* c, const char* what) {
    std::fprintf(stderr, "motifcl-cuda OpenCL seam: %s: %s\n", what, mcl_cuda_last_error(c ? c->ctx : nullptr));
    return CL_INVALID_OPERATION;
}

template <class T>
bool scalar(const _cl_kernel* k, int i, T* out) {
    if (i >= (int)k->args.size() || k->args[i].size() != sizeof(T)) return false;
    std::memcpy(out, k->args[i].data(), sizeof(T));
    return true;
}
bool buffer(const _cl_kernel* k, int i, void** out) {
    cl_mem m = nullptr;
    if (!scalar(k, i, &m) || !m) return false;
    *out = m->dptr;
    return true;
}

// out[i] = a[i] * 1: the device-to-device copy the ABI offers
int copy_f32(_cl_context* c, const void* src, void* dst, size_t n) {
    return mcl_cuda_eltwise_f32(c->ctx, MCL_CUDA_ELT_MUL_SCALAR, static_cast<const float*>(src), nullptr,
                                static_cast<float*>(dst), n, 1.0f);
}

cl_int run_kernel(_cl_kernel* k) {
    _cl_context* c = k->context;
    mcl_cuda_ctx* ctx = c->ctx;
    void *b0 = nullptr, *b1 = nullptr, *b2 = nullptr, *b3 = nullptr, *b4 = nullptr, *b5 = nullptr, *b6 = nullptr;
    int i0 = 0, i1 = 0, i2 = 0, i3 = 0, i4 = 0;
    float f0 = 0.f, f1 = 0.f, f2 = 0.f;
    cl_uint u0 = 0;
    bool ok = true;
    int rc = MCL_CUDA_OK;
    switch (k->id) {
    case K_DECODE:          // (state, scale, w, C, in_features, n_groups)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && scalar(k, 3, &i0) && scalar(k, 4, &i1) && scalar(k, 5, &i2);
        if (ok) rc = mcl_cuda_counter_decode_weight(ctx, (const uint8_t*)b0, (const float*)b1, (float*)b2, i1, (size_t)i2 / (i1 / 4), i0);
        break;
    case K_ROW_STATS: {     // (state, scale, v, grad_w, scale_new, denom, C, in, out, lr_scale, rms_beta, rms_eps)
        auto& p = c->pending;
        ok = buffer(k, 0, &p.state) && buffer(k, 1, &p.scale) && buffer(k, 2, &p.v) && buffer(k, 3, &p.grad) &&
             buffer(k, 4, &p.scale_new) && buffer(k, 5, &b5) && scalar(k, 6, &p.C) && scalar(k, 7, &p.in) &&
             scalar(k, 8, &p.out) && scalar(k, 9, &p.lr_scale) && scalar(k, 10, &p.beta) && scalar(k, 11, &p.eps);
        p.valid = ok; p.fused = false; p.x = nullptr; p.N = 0;
        break;
    }
    case K_ROW_STATS_FUSED: {   // (state, scale, v, grad_out, x, scale_new, denom, C, in, out, N, lr_scale, rms_beta, rms_eps)
        auto& p = c->pending;
        ok = buffer(k, 0, &p.state) && buffer(k, 1, &p.scale) && buffer(k, 2, &p.v) && buffer(k, 3, &p.grad) &&
             buffer(k, 4, &p.x) && buffer(k, 5, &p.scale_new) && buffer(k, 6, &b6) && scalar(k, 7, &p.C) &&
             scalar(k, 8, &p.in) && scalar(k, 9, &p.out) && scalar(k, 10, &p.N) && scalar(k, 11, &p.lr_scale) &&
             scalar(k, 12, &p.beta) && scalar(k, 13, &p.eps);
        p.valid = ok; p.fused = true;
        break;
    }
    case K_APPLY: {         // (state, scale, scale_new, denom, grad_w, C, in, n_groups, lr, seed)
        auto& p = c->pending;
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && buffer(k, 4, &b4) && scalar(k, 5, &i0) &&
             scalar(k, 6, &i1) && scalar(k, 7, &i2) && scalar(k, 8, &f0) && scalar(k, 9, &u0);
        if (!ok) break;
        if (!p.valid || p.fused || p.state != b0 || p.scale != b1 || p.scale_new != b2 || p.grad != b4 || p.in != i1 || p.C != i0) {
            std::fprintf(stderr, "motifcl-cuda OpenCL seam: counter_apply_update_f32 without the matching counter_row_stats_f32 launch\n");
            return CL_INVALID_OPERATION;
        }
        p.valid = false;
        rc = mcl_cuda_counter_update_dense(ctx, (uint8_t*)p.state, (float*)p.scale, (float*)p.v, (const float*)p.grad, nullptr,
                                           p.C, p.in, p.out, 0, f0, p.lr_scale, p.beta, p.eps, u0);
        if (rc == MCL_CUDA_OK) rc = copy_f32(c, p.scale, p.scale_new, p.out);
        break;
    }
    case K_APPLY_FUSED: {   // (state, scale, scale_new, denom, grad_out, x, C, in, out, N, n_groups, lr, seed)
        auto& p = c->pending;
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && buffer(k, 4, &b4) && buffer(k, 5, &b5) &&
             scalar(k, 6, &i0) && scalar(k, 7, &i1) && scalar(k, 8, &i2) && scalar(k, 9, &i3) && scalar(k, 11, &f0) && scalar(k, 12, &u0);
        if (!ok) break;
        if (!p.valid || !p.fused || p.state != b0 || p.scale != b1 || p.scale_new != b2 || p.grad != b4 || p.x != b5 ||
            p.in != i1 || p.out != i2 || p.N != i3 || p.C != i0) {
            std::fprintf(stderr, "motifcl-cuda OpenCL seam: counter_apply_update_fused_f32 without the matching counter_row_stats_fused_f32 launch\n");
            return CL_INVALID_OPERATION;
        }
        p.valid = false;
        rc = mcl_cuda_counter_update_fused(ctx, (uint8_t*)p.state, (float*)p.scale, (float*)p.v, (const float*)p.grad,
                                           (const float*)p.x, nullptr, nullptr, nullptr, p.C, p.in, p.out, p.N, f0,
                                           p.lr_scale, p.beta, p.eps, u0);
        if (rc == MCL_CUDA_OK) rc = copy_f32(c, p.scale, p.scale_new, p.out);
        break;
    }
    case K_BACKWARD_INPUT:  // (grad_out, state, scale, grad_x, C, in, out, N)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && buffer(k, 3, &b3) && scalar(k, 4, &i0) &&
             scalar(k, 5, &i1) && scalar(k, 6, &i2) && scalar(k, 7, &i3);
        if (ok) rc = mcl_cuda_counter_backward_input(ctx, (const uint8_t*)b1, (const float*)b2, (const float*)b0, (float*)b3, i3, i1, i2, i0);
        break;
    case K_MM_NN: case K_MM_TA: case K_MM_TB: case K_MM_FLAGS: {   // (A, B, C, M, N, K [, transA, transB])
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && scalar(k, 3, &i0) && scalar(k, 4, &i1) && scalar(k, 5, &i2);
        int ta = k->id == K_MM_TA, tb = k->id == K_MM_TB;
        if (k->id == K_MM_FLAGS) ok = ok && scalar(k, 6, &ta) && scalar(k, 7, &tb);
        if (ok) rc = mcl_cuda_matmul_f32(ctx, (const float*)b0, (const float*)b1, (float*)b2, i0, i2, i1, ta != 0, tb != 0);
        break;
    }
    case K_MSE_PARTIAL:     // (pred, target, partial, n)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && scalar(k, 3, &i0);
        if (ok) rc = mcl_cuda_mse_loss_partial(ctx, (const float*)b0, (const float*)b1, (float*)b2, i0);
        break;
    case K_MEAN_REDUCE:     // (partial, out, partial_count, denominator)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && scalar(k, 2, &i0) && scalar(k, 3, &i1);
        if (ok) rc = mcl_cuda_mean_reduce(ctx, (const float*)b0, (float*)b1, i0, i1 > 0 ? i1 : 0);
        break;
    case K_MSE_BACKWARD:    // (pred, target, grad_out, grad_pred, n)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && buffer(k, 3, &b3) && scalar(k, 4, &i0);
        if (ok) rc = mcl_cuda_mse_backward(ctx, (const float*)b0, (const float*)b1, (const float*)b2, (float*)b3, i0);
        break;
    case K_FILL:            // (x, value, n)
        ok = buffer(k, 0, &b0) && scalar(k, 1, &f0) && scalar(k, 2, &i0);
        if (ok) rc = mcl_cuda_eltwise_f32(ctx, MCL_CUDA_ELT_ZERO, nullptr, nullptr, (float*)b0, i0, 0.0f);
        if (ok && rc == MCL_CUDA_OK && f0 != 0.0f)
            rc = mcl_cuda_eltwise_f32(ctx, MCL_CUDA_ELT_ADD_SCALAR, (const float*)b0, nullptr, (float*)b0, i0, f0);
        break;
    case K_COPY:            // (x, out, n)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && scalar(k, 2, &i0);
        if (ok) rc = copy_f32(c, b0, b1, i0);
        break;
    case K_ADD: case K_SUB: case K_MUL:     // (a, b, out, n)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && buffer(k, 2, &b2) && scalar(k, 3, &i0);
        if (ok) rc = mcl_cuda_eltwise_f32(ctx, k->id == K_ADD ? MCL_CUDA_ELT_ADD : k->id == K_SUB ? MCL_CUDA_ELT_SUB : MCL_CUDA_ELT_MUL,
                                          (const float*)b0, (const float*)b1, (float*)b2, i0, 0.0f);
        break;
    case K_ADD_SCALAR: case K_MUL_SCALAR:   // (x, value, out, n)
        ok = buffer(k, 0, &b0) && scalar(k, 1, &f0) && buffer(k, 2, &b2) && scalar(k, 3, &i0);
        if (ok) rc = mcl_cuda_eltwise_f32(ctx, k->id == K_ADD_SCALAR ? MCL_CUDA_ELT_ADD_SCALAR : MCL_CUDA_ELT_MUL_SCALAR,
                                          (const float*)b0, nullptr, (float*)b2, i0, f0);
        break;
    case K_SCALE:           // (x, alpha, n) in place
        ok = buffer(k, 0, &b0) && scalar(k, 1, &f0) && scalar(k, 2, &i0);
        if (ok) rc = mcl_cuda_eltwise_f32(ctx, MCL_CUDA_ELT_MUL_SCALAR, (const float*)b0, nullptr, (float*)b0, i0, f0);
        break;
    case K_ADD_INPLACE:     // (dst, src, n)
        ok = buffer(k, 0, &b0) && buffer(k, 1, &b1) && scalar(k, 2, &i0);
        if (ok) rc = mcl_cuda_eltwise_f32(ctx, MCL_CUDA_ELT_ADD, (const float*)b0, (const float*)b1, (float*)b0, i0, 0.0f);
        break;
    default:
        return CL_INVALID_KERNEL;
    }
    (void)f1; (void)f2; (void)i4;
    if (!ok) {
        std::fprintf(stderr, "motifcl-cuda OpenCL seam: kernel %s launched with unset or mis-sized arguments\n", k->name.c_str());
        return CL_INVALID_KERNEL_ARGS;
    }
    if (rc != MCL_CUDA_OK) return failed(c, k->name.c_str());
    return CL_SUCCESS;
}

template <class T>
cl_int release(T* obj) {
    if (!obj) return CL_INVALID_VALUE;
    if (--obj->refs == 0) delete obj;
    return CL_SUCCESS;
}
// queues, buffers, programs and kernels keep their context alive (OpenCL's own rule), so the order in which a caller
// lets go of them does not matter
template <class T>
cl_int release_child(T* obj) {
    if (!obj) return CL_INVALID_VALUE;
    if (--obj->refs == 0) {
        _cl_context* c = obj->context;
        delete obj;
        release(c);
    }
    return CL_SUCCESS;
}

}  // namespace

extern "C" {

cl_int clGetPlatformIDs(cl_uint num_entries, cl_platform_id* platforms, cl_uint* num_platforms) {
    const cl_uint n = shared_ctx() ? 1u : 0u;       // no CUDA device: no platform, and MotifCL's device tests skip
    if (num_platforms) *num_platforms = n;
    if (platforms && num_entries >= 1 && n) platforms[0] = &g_platform;
    return CL_SUCCESS;
}

cl_int clGetPlatformInfo(cl_platform_id, cl_platform_info name, size_t size, void* value, size_t* size_ret) {
    switch (name) {
    case CL_PLATFORM_NAME: return put_string("motifcl-cuda", size, value, size_ret);
    case CL_PLATFORM_VENDOR: return put_string("motifcl_b200", size, value, size_ret);
    case CL_PLATFORM_VERSION: return put_string("OpenCL 1.2 motifcl-cuda", size, value, size_ret);
    case CL_PLATFORM_PROFILE: return put_string("FULL_PROFILE", size, value, size_ret);
    case CL_PLATFORM_EXTENSIONS: return put_string("", size, value, size_ret);
    default: return CL_INVALID_VALUE;
    }
}

cl_int clGetDeviceIDs(cl_platform_id, cl_device_type type, cl_uint num_entries, cl_device_id* devices, cl_uint* num_devices) {
    const bool wanted = (type & CL_DEVICE_TYPE_GPU) != 0 || type == CL_DEVICE_TYPE_ALL || (type & CL_DEVICE_TYPE_DEFAULT) != 0;
    if (!wanted || !shared_ctx()) {
        if (num_devices) *num_devices = 0;
        return CL_DEVICE_NOT_FOUND;
    }
    if (num_devices) *num_devices = 1;
    if (devices && num_entries >= 1) devices[0] = &g_device;
    return CL_SUCCESS;
}

cl_int clGetDeviceInfo(cl_device_id, cl_device_info name, size_t size, void* value, size_t* size_ret) {
    mcl_cuda_ctx* ctx = shared_ctx();
    if (!ctx) return CL_INVALID_DEVICE;
    switch (name) {
    case CL_DEVICE_NAME: return put_string(mcl_cuda_device_name(ctx), size, value, size_ret);
    case CL_DEVICE_VENDOR: return put_string("NVIDIA (through libmotifcl_cuda)", size, value, size_ret);
    case CL_DRIVER_VERSION: return put_string("motifcl-cuda", size, value, size_ret);
    case CL_DEVICE_VERSION: return put_string("OpenCL 1.2 motifcl-cuda", size, value, size_ret);
    case CL_DEVICE_PROFILE: return put_string("FULL_PROFILE", size, value, size_ret);
    case CL_DEVICE_EXTENSIONS: return put_string("", size, value, size_ret);
    case CL_DEVICE_TYPE: { cl_device_type t = CL_DEVICE_TYPE_GPU; return put(&t, sizeof(t), size, value, size_ret); }
    case CL_DEVICE_VENDOR_ID: { cl_uint v = 0x10DE; return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_MAX_COMPUTE_UNITS: { cl_uint v = (cl_uint)mcl_cuda_sm_count(ctx); return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_MAX_WORK_ITEM_DIMENSIONS: { cl_uint v = 3; return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_MAX_WORK_GROUP_SIZE: { size_t v = 1024; return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_MAX_CLOCK_FREQUENCY: { cl_uint v = 0; return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_ADDRESS_BITS: { cl_uint v = 64; return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_PREFERRED_VECTOR_WIDTH_FLOAT: { cl_uint v = 1; return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_GLOBAL_MEM_SIZE: case CL_DEVICE_MAX_MEM_ALLOC_SIZE: {
        cl_ulong v = (cl_ulong)mcl_cuda_device_memory_bytes(ctx); return put(&v, sizeof(v), size, value, size_ret); }
    case CL_DEVICE_LOCAL_MEM_SIZE: { cl_ulong v = 48 * 1024; return put(&v, sizeof(v), size, value, size_ret); }
    default: return CL_INVALID_VALUE;
    }
}

cl_context clCreateContext(const cl_context_properties*, cl_uint num_devices, const cl_device_id* devices,
                           void (*)(const char*, const void*, size_t, void*), void*, cl_int* err) {
    mcl_cuda_ctx* ctx = shared_ctx();
    if (!ctx || num_devices != 1 || !devices || devices[0] != &g_device) {
        if (err) *err = CL_INVALID_DEVICE;
        return nullptr;
    }
    auto* c = new _cl_context;
    c->ctx = ctx;           // every context shares the one device context (and its one in-order stream)
    if (err) *err = CL_SUCCESS;
    return c;
}
cl_int clReleaseContext(cl_context c) { return release(c); }

cl_command_queue clCreateCommandQueue(cl_context c, cl_device_id, cl_command_queue_properties, cl_int* err) {
    if (!c) { if (err) *err = CL_INVALID_CONTEXT; return nullptr; }
    auto* q = new _cl_command_queue;
    q->context = c;
    ++c->refs;
    if (err) *err = CL_SUCCESS;
    return q;
}
cl_int clReleaseCommandQueue(cl_command_queue q) { return release_child(q); }

cl_mem clCreateBuffer(cl_context c, cl_mem_flags flags, size_t size, void* host_ptr, cl_int* err) {
    if (!c || size == 0) { if (err) *err = c ? CL_INVALID_VALUE : CL_INVALID_CONTEXT; return nullptr; }
    void* d = nullptr;
    if (mcl_cuda_alloc(c->ctx, size, &d) != MCL_CUDA_OK) { failed(c, "clCreateBuffer"); if (err) *err = CL_INVALID_OPERATION; return nullptr; }
    if ((flags & (CL_MEM_COPY_HOST_PTR | CL_MEM_USE_HOST_PTR)) && host_ptr &&
        mcl_cuda_upload(c->ctx, d, host_ptr, size) != MCL_CUDA_OK) {
        failed(c, "clCreateBuffer (host data)");
        mcl_cuda_free(c->ctx, d);
        if (err) *err = CL_INVALID_OPERATION;
        return nullptr;
    }
    auto* m = new _cl_mem;
    m->context = c; m->dptr = static_cast<char*>(d); m->size = size;
    ++c->refs;
    if (err) *err = CL_SUCCESS;
    return m;
}

cl_mem clCreateSubBuffer(cl_mem parent, cl_mem_flags, cl_buffer_create_type type, const void* info, cl_int* err) {
    const auto* region = static_cast<const cl_buffer_region*>(info);
    if (!parent || type != CL_BUFFER_CREATE_TYPE_REGION || !region || region->origin + region->size > parent->size) {
        if (err) *err = CL_INVALID_VALUE;
        return nullptr;
    }
    auto* m = new _cl_mem;
    m->context = parent->context; m->dptr = parent->dptr + region->origin; m->size = region->size; m->parent = parent;
    ++parent->refs;
    ++m->context->refs;
    if (err) *err = CL_SUCCESS;
    return m;
}
cl_int clRetainMemObject(cl_mem m) { if (!m) return CL_INVALID_MEM_OBJECT; ++m->refs; return CL_SUCCESS; }
cl_int clReleaseMemObject(cl_mem m) {
    if (!m) return CL_INVALID_MEM_OBJECT;
    if (--m->refs == 0) {
        _cl_context* c = m->context;
        if (m->parent) clReleaseMemObject(m->parent);
        else mcl_cuda_free(c->ctx, m->dptr);      // ordered after the work already enqueued
        delete m;
        release(c);
    }
    return CL_SUCCESS;
}

cl_int clEnqueueWriteBuffer(cl_command_queue q, cl_mem m, cl_bool, size_t offset, size_t cb, const void* ptr, cl_uint,
                            const cl_event*, cl_event* event) {
    if (!q || !m || offset + cb > m->size) return CL_INVALID_VALUE;
    if (cb && mcl_cuda_upload(q->context->ctx, m->dptr + offset, ptr, cb) != MCL_CUDA_OK) return failed(q->context, "clEnqueueWriteBuffer");
    if (event) *event = new _cl_event;
    return CL_SUCCESS;
}
cl_int clEnqueueReadBuffer(cl_command_queue q, cl_mem m, cl_bool, size_t offset, size_t cb, void* ptr, cl_uint,
                           const cl_event*, cl_event* event) {
    if (!q || !m || offset + cb > m->size) return CL_INVALID_VALUE;
    if (cb && mcl_cuda_download(q->context->ctx, ptr, m->dptr + offset, cb) != MCL_CUDA_OK) return failed(q->context, "clEnqueueReadBuffer");
    if (event) *event = new _cl_event;
    return CL_SUCCESS;
}

cl_program clCreateProgramWithSource(cl_context c, cl_uint, const char**, const size_t*, cl_int* err) {
    if (!c) { if (err) *err = CL_INVALID_CONTEXT; return nullptr; }
    auto* p = new _cl_program;      // the text is not compiled: kernels are looked up by name in kKernels
    p->context = c;
    ++c->refs;
    if (err) *err = CL_SUCCESS;
    return p;
}
cl_int clBuildProgram(cl_program p, cl_uint, const cl_device_id*, const char*, void (*)(cl_program, void*), void*) {
    return p ? CL_SUCCESS : CL_INVALID_PROGRAM;
}
cl_int clGetProgramBuildInfo(cl_program, cl_device_id, cl_program_build_info name, size_t size, void* value, size_t* size_ret) {
    if (name == CL_PROGRAM_BUILD_LOG || name == CL_PROGRAM_BUILD_OPTIONS) return put_string("", size, value, size_ret);
    return CL_INVALID_VALUE;
}
cl_int clReleaseProgram(cl_program p) { return release_child(p); }

cl_kernel clCreateKernel(cl_program p, const char* name, cl_int* err) {
    if (!p || !name) { if (err) *err = CL_INVALID_PROGRAM; return nullptr; }
    for (const auto& e : kKernels) {
        if (std::strcmp(e.name, name) == 0) {
            auto* k = new _cl_kernel;
            k->context = p->context; k->id = e.id; k->name = name; k->args.resize(e.nargs);
            ++k->context->refs;
            if (err) *err = CL_SUCCESS;
            return k;
        }
    }
    if (err) *err = CL_INVALID_KERNEL_NAME;      // not a kernel of the counter-linear path: the caller reports the name
    return nullptr;
}
cl_int clRetainKernel(cl_kernel k) { if (!k) return CL_INVALID_KERNEL; ++k->refs; return CL_SUCCESS; }
cl_int clReleaseKernel(cl_kernel k) { return release_child(k); }

cl_int clSetKernelArg(cl_kernel k, cl_uint index, size_t size, const void* value) {
    if (!k) return CL_INVALID_KERNEL;
    if (index >= k->args.size()) return CL_INVALID_ARG_INDEX;
    auto& a = k->args[index];
    a.assign(size, 0);                       // value == NULL: local memory of `size` bytes (none of these kernels has any)
    if (value && size) std::memcpy(a.data(), value, size);
    return CL_SUCCESS;
}

cl_int clEnqueueNDRangeKernel(cl_command_queue q, cl_kernel k, cl_uint dim, const size_t*, const size_t* global, const size_t*,
                              cl_uint, const cl_event*, cl_event* event) {
    if (!q || !k) return CL_INVALID_KERNEL;
    if (dim < 1 || dim > 3 || !global) return CL_INVALID_WORK_DIMENSION;
    // the work sizes are MotifCL's tiling of its own kernels; the CUDA kernels behind the ABI choose their own
    const cl_int rc = run_kernel(k);
    if (rc == CL_SUCCESS && event) *event = new _cl_event;
    return rc;
}

cl_int clFinish(cl_command_queue q) {
    if (!q) return CL_INVALID_VALUE;
    return mcl_cuda_finish(q->context->ctx) == MCL_CUDA_OK ? CL_SUCCESS : failed(q->context, "clFinish");
}
cl_int clWaitForEvents(cl_uint n, const cl_event* events) {
    if (!n || !events) return CL_INVALID_VALUE;
    mcl_cuda_ctx* ctx = shared_ctx();       // one in-order stream: waiting for an event is waiting for the stream
    return ctx && mcl_cuda_finish(ctx) == MCL_CUDA_OK ? CL_SUCCESS : CL_INVALID_OPERATION;
}
cl_int clReleaseEvent(cl_event e) { return release(e); }
cl_int clGetEventProfilingInfo(cl_event e, cl_profiling_info, size_t size, void* value, size_t* size_ret) {
    if (!e) return CL_INVALID_VALUE;
    const cl_ulong zero = 0;                // no device timestamps behind this seam
    return put(&zero, sizeof(zero), size, value, size_ret);
}
void* clGetExtensionFunctionAddress(const char*) { return nullptr; }
void* clGetExtensionFunctionAddressForPlatform(cl_platform_id, const char*) { return nullptr; }

}  // extern "C"
