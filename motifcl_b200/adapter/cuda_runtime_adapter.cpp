// MotifCL runtime seam on CUDA: defines the symbols of MotifCL's `motifcl_vulkan_runtime`
// link target (include/motifcl/runtime/vulkan_backend.hpp: VulkanRuntime, VulkanBuffer,
// probe_vulkan_runtime and the run_vulkan_* free functions) on top of the C ABI of
// libmotifcl_cuda.so.  Linked in place of MotifCL's src/runtime/vulkan_backend.cpp it turns
// Backend::create_vulkan() into a CUDA backend, so MotifCL's own sources -- nn::CounterStateLinear,
// its autograd node, its tests -- run unchanged against the B200 kernels.
//
// This file implements the counter-synapse path and the f32 matmuls; every other run_vulkan_*
// entry is a generated stub that reports "not implemented in CUDA runtime" (gen_stubs.py).
// It is compiled against the MotifCL headers where they lie; nothing of MotifCL is copied here.
#include <motifcl/runtime/vulkan_backend.hpp>

#include <cstring>
#include <stdexcept>
#include <utility>

#include "motifcl_cuda.h"

namespace motifcl {

namespace {
// Free functions cannot see the private parts of VulkanBuffer; like MotifCL's own runtime they
// funnel through the public VulkanRuntime::dispatch_cached, which here recognises this tag in
// place of a SPIR-V pointer and reads the operation and its scalar arguments from the
// "word count" and "push constants".
const std::uint32_t kNativeTag[1] = {0x4D434C55u};
enum NativeOp : std::size_t {
    kOpDecode = 1, kOpForward, kOpBackwardInput, kOpUpdateFused, kOpMatmul, kOpEltwise,
    kOpRmsnorm, kOpRmsnormBwdX, kOpRmsnormBwdW, kOpSwiglu, kOpSwigluBwd, kOpCe, kOpCeBwd, kOpGqa, kOpGqaBwd,
    kOpEmbedding, kOpEmbeddingBwd, kOpPositionBwd, kOpRope, kOpAdam
};
struct NativeArgs {
    std::size_t a = 0, b = 0, c = 0, d = 0;          // dimensions (meaning depends on the op)
    std::size_t e = 0, f = 0, g = 0, h = 0, i = 0, j = 0;
    int causal = 0;
    float f0 = 0, f1 = 0, f2 = 0, f3 = 0, f4 = 0, f5 = 0, f6 = 0;
    float lr = 0, lr_scale = 0, rms_beta = 0, rms_eps = 0;
    std::uint32_t seed = 0;
    int trans_a = 0, trans_b = 0;
    int elt_op = 0;
    float alpha = 0;
};

// Owns the C-ABI context; shared by the runtime and every buffer so that buffers may outlive
// the VulkanRuntime object that made them, as MotifCL's Storage assumes.
struct CtxHolder {
    mcl_cuda_ctx* ctx = nullptr;
    ~CtxHolder() { if (ctx) mcl_cuda_destroy(ctx); }
};
}  // namespace

struct VulkanBuffer::Impl {
    std::shared_ptr<CtxHolder> holder;
    void* dptr = nullptr;
    std::size_t nbytes = 0;
    ~Impl() { if (dptr && holder && holder->ctx) mcl_cuda_free(holder->ctx, dptr); }
};

struct VulkanDispatchRecording::Impl {};

struct VulkanRuntime::Impl {
    std::shared_ptr<CtxHolder> holder;
    std::string device_name;
    std::string error;
    VulkanDeviceCaps caps;
    bool batch = false;
    bool capture = false;
};

// ---- VulkanBuffer -------------------------------------------------------------------------
VulkanBuffer::VulkanBuffer() = default;
VulkanBuffer::~VulkanBuffer() = default;
VulkanBuffer::VulkanBuffer(VulkanBuffer&&) noexcept = default;
VulkanBuffer& VulkanBuffer::operator=(VulkanBuffer&&) noexcept = default;
VulkanBuffer::VulkanBuffer(std::shared_ptr<Impl> impl) : impl_(std::move(impl)) {}
bool VulkanBuffer::valid() const { return impl_ && impl_->dptr != nullptr; }
std::size_t VulkanBuffer::nbytes() const { return impl_ ? impl_->nbytes : 0; }

void VulkanBuffer::upload(const void* data, std::size_t bytes, std::size_t offset) {
    if (!valid()) throw std::runtime_error("VulkanBuffer::upload on an invalid buffer");
    if (offset > impl_->nbytes || bytes > impl_->nbytes - offset)
        throw std::runtime_error("VulkanBuffer::upload out of bounds");
    mcl_cuda_ctx* ctx = impl_->holder->ctx;
    if (mcl_cuda_upload(ctx, static_cast<char*>(impl_->dptr) + offset, data, bytes) != MCL_CUDA_OK)
        throw std::runtime_error(std::string("VulkanBuffer::upload failed: ") + mcl_cuda_last_error(ctx));
}
void VulkanBuffer::download(void* data, std::size_t bytes, std::size_t offset) const {
    if (!valid()) throw std::runtime_error("VulkanBuffer::download on an invalid buffer");
    if (offset > impl_->nbytes || bytes > impl_->nbytes - offset)
        throw std::runtime_error("VulkanBuffer::download out of bounds");
    mcl_cuda_ctx* ctx = impl_->holder->ctx;
    if (mcl_cuda_download(ctx, data, static_cast<const char*>(impl_->dptr) + offset, bytes) != MCL_CUDA_OK)
        throw std::runtime_error(std::string("VulkanBuffer::download failed: ") + mcl_cuda_last_error(ctx));
}

// ---- VulkanDispatchRecording (capture / replay is not offered by this runtime) --------------
VulkanDispatchRecording::VulkanDispatchRecording() = default;
VulkanDispatchRecording::~VulkanDispatchRecording() = default;
VulkanDispatchRecording::VulkanDispatchRecording(VulkanDispatchRecording&&) noexcept = default;
VulkanDispatchRecording& VulkanDispatchRecording::operator=(VulkanDispatchRecording&&) noexcept = default;
bool VulkanDispatchRecording::empty() const { return true; }
std::size_t VulkanDispatchRecording::size() const { return 0; }

// ---- VulkanRuntime --------------------------------------------------------------------------
VulkanRuntime::VulkanRuntime() = default;
VulkanRuntime::~VulkanRuntime() = default;
VulkanRuntime::VulkanRuntime(VulkanRuntime&&) noexcept = default;
VulkanRuntime& VulkanRuntime::operator=(VulkanRuntime&&) noexcept = default;
VulkanRuntime::VulkanRuntime(std::shared_ptr<Impl> impl) : impl_(std::move(impl)) {}

VulkanRuntime VulkanRuntime::create() {
    auto impl = std::make_shared<Impl>();
    impl->holder = std::make_shared<CtxHolder>();
    const int rc = mcl_cuda_create(0, &impl->holder->ctx);
    if (rc != MCL_CUDA_OK) {
        impl->error = mcl_cuda_last_error(nullptr);
        impl->holder->ctx = nullptr;
    } else {
        impl->device_name = mcl_cuda_device_name(impl->holder->ctx);
        impl->caps.timestamps = false;
        impl->caps.max_shared_memory_bytes = 232448;
        impl->caps.max_workgroup_invocations = 1024;
        impl->caps.subgroup_arithmetic_compute = true;
        impl->caps.subgroup_size = 32;
        impl->caps.supports_atomic_float = true;
        impl->caps.prefer_rb4_matmul = true;
    }
    return VulkanRuntime(std::move(impl));
}

static const std::string kEmpty;
bool VulkanRuntime::available() const { return impl_ && impl_->holder && impl_->holder->ctx != nullptr; }
const std::string& VulkanRuntime::device_name() const { return impl_ ? impl_->device_name : kEmpty; }
const std::string& VulkanRuntime::error() const { return impl_ ? impl_->error : kEmpty; }
bool VulkanRuntime::supports_storage_buffer_i8() const { return available(); }
const VulkanDeviceCaps& VulkanRuntime::caps() const {
    static const VulkanDeviceCaps none;
    return impl_ ? impl_->caps : none;
}

// The reference defers a step's dispatches into one submit; here calls run eagerly on the
// context's in-order stream, so a batch is only a bracket whose end waits for the stream.
bool VulkanRuntime::batch_begin() {
    if (!available() || impl_->batch) return false;
    impl_->batch = true;
    return true;
}
VulkanOpResult VulkanRuntime::batch_end() {
    VulkanOpResult r;
    r.device_name = device_name();
    if (!available() || !impl_->batch) { r.error = "batch_end without batch_begin"; return r; }
    impl_->batch = false;
    if (mcl_cuda_finish(impl_->holder->ctx) != MCL_CUDA_OK) { r.error = mcl_cuda_last_error(impl_->holder->ctx); return r; }
    r.success = true;
    return r;
}
bool VulkanRuntime::batch_active() const { return impl_ && impl_->batch; }
void VulkanRuntime::set_gpu_timing_enabled(bool) {}
double VulkanRuntime::last_gpu_time_us() const { return -1.0; }
void VulkanRuntime::finish() const {
    if (available()) mcl_cuda_finish(impl_->holder->ctx);
}
bool VulkanRuntime::capture_begin() { return false; }
VulkanDispatchRecording VulkanRuntime::capture_end() { return VulkanDispatchRecording(); }
bool VulkanRuntime::capture_active() const { return false; }
VulkanOpResult VulkanRuntime::replay(const VulkanDispatchRecording&) {
    VulkanOpResult r;
    r.device_name = device_name();
    r.error = "dispatch capture/replay is not implemented in CUDA runtime";
    return r;
}

VulkanBuffer VulkanRuntime::create_buffer(std::size_t nbytes, const void* initial_data) {
    if (!available()) throw std::runtime_error("VulkanRuntime::create_buffer: runtime is not available");
    auto impl = std::make_shared<VulkanBuffer::Impl>();
    impl->holder = impl_->holder;
    impl->nbytes = nbytes;
    if (mcl_cuda_alloc(impl_->holder->ctx, nbytes ? nbytes : 16, &impl->dptr) != MCL_CUDA_OK)
        throw std::runtime_error(std::string("VulkanRuntime::create_buffer failed: ") +
                                 mcl_cuda_last_error(impl_->holder->ctx));
    VulkanBuffer buf(std::move(impl));
    if (initial_data && nbytes) buf.upload(initial_data, nbytes, 0);
    return buf;
}

VulkanOpResult VulkanRuntime::dispatch_cached(const std::uint32_t* spirv, std::size_t op,
                                              const std::vector<const VulkanBuffer*>& bufs, const void* push,
                                              std::uint32_t push_bytes, std::uint32_t, std::uint32_t, std::uint32_t) {
    VulkanOpResult r;
    r.device_name = device_name();
    if (!available()) { r.error = "CUDA runtime is not available"; return r; }
    if (spirv != kNativeTag || push_bytes != sizeof(NativeArgs)) {
        r.error = "SPIR-V dispatch is not implemented in CUDA runtime";
        return r;
    }
    for (const VulkanBuffer* b : bufs)
        if (b == nullptr || !b->valid()) { r.error = "invalid buffer"; return r; }
    mcl_cuda_ctx* ctx = impl_->holder->ctx;
    NativeArgs a;
    std::memcpy(&a, push, sizeof(a));
    auto p = [&](std::size_t i) { return bufs[i]->impl_->dptr; };
    int rc = MCL_CUDA_EINVAL;
    switch (op) {
        case kOpDecode:          // state, scale, weight | in, out, C
            rc = mcl_cuda_counter_decode_weight(ctx, (const uint8_t*)p(0), (const float*)p(1), (float*)p(2), a.a, a.b, a.c);
            break;
        case kOpForward:         // x, state, scale, out | batch, in, out, C
            rc = mcl_cuda_counter_forward(ctx, (const float*)p(0), (const uint8_t*)p(1), (const float*)p(2), (float*)p(3),
                                          a.a, a.b, a.c, a.d);
            break;
        case kOpBackwardInput:   // state, scale, grad_out, grad_x | batch, in, out, C
            rc = mcl_cuda_counter_backward_input(ctx, (const uint8_t*)p(0), (const float*)p(1), (const float*)p(2),
                                                 (float*)p(3), a.a, a.b, a.c, a.d);
            break;
        case kOpUpdateFused:     // state, scale, v, grad_out, x, scratch, scratch | C, in, out, batch
            rc = mcl_cuda_counter_update_fused(ctx, (uint8_t*)p(0), (float*)p(1), (float*)p(2), (const float*)p(3),
                                               (const float*)p(4), (float*)p(5), (float*)p(6), nullptr, a.a, a.b, a.c,
                                               a.d, a.lr, a.lr_scale, a.rms_beta, a.rms_eps, a.seed);
            break;
        case kOpMatmul:          // a, b, c | m, k, n
            rc = mcl_cuda_matmul_f32(ctx, (const float*)p(0), (const float*)p(1), (float*)p(2), a.a, a.b, a.c, a.trans_a,
                                     a.trans_b);
            break;
        case kOpEltwise:         // [a, [b,]] out | elements; the last buffer is the output
            rc = mcl_cuda_eltwise_f32(ctx, a.elt_op, bufs.size() > 1 ? (const float*)p(0) : nullptr,
                                      bufs.size() > 2 ? (const float*)p(1) : nullptr, (float*)p(bufs.size() - 1), a.a,
                                      a.alpha);
            break;
        case kOpRmsnorm:         // x, weight, out | rows, cols, eps
            rc = mcl_cuda_rmsnorm(ctx, (const float*)p(0), (const float*)p(1), (float*)p(2), a.a, a.b, a.alpha);
            break;
        case kOpRmsnormBwdX:     // x, weight, grad_out, grad_x | rows, cols, eps
            rc = mcl_cuda_rmsnorm_backward_x(ctx, (const float*)p(0), (const float*)p(1), (const float*)p(2), (float*)p(3),
                                             a.a, a.b, a.alpha);
            break;
        case kOpRmsnormBwdW:     // x, grad_out, row_inv, grad_weight | rows, cols, eps
            rc = mcl_cuda_rmsnorm_backward_weight(ctx, (const float*)p(0), (const float*)p(1), (float*)p(2), (float*)p(3),
                                                  a.a, a.b, a.alpha);
            break;
        case kOpSwiglu:          // packed, out | rows, hidden
            rc = mcl_cuda_swiglu(ctx, (const float*)p(0), (float*)p(1), a.a, a.b);
            break;
        case kOpSwigluBwd:       // packed, grad_out, grad_packed | rows, hidden
            rc = mcl_cuda_swiglu_backward(ctx, (const float*)p(0), (const float*)p(1), (float*)p(2), a.a, a.b);
            break;
        case kOpCe:              // logits, targets, partial, out | rows, cols
            rc = mcl_cuda_softmax_cross_entropy(ctx, (const float*)p(0), (const int32_t*)p(1), (float*)p(2), (float*)p(3),
                                                a.a, a.b);
            break;
        case kOpCeBwd:           // logits, targets, grad_out, grad_logits | rows, cols
            rc = mcl_cuda_softmax_cross_entropy_backward(ctx, (const float*)p(0), (const int32_t*)p(1), (const float*)p(2),
                                                         (float*)p(3), a.a, a.b);
            break;
        case kOpGqa:             // q, k, v, out | batch, tq, tk, key_stride, heads, kv heads, hd, vhd, offset, window
            rc = mcl_cuda_gqa_forward(ctx, (const float*)p(0), (const float*)p(1), (const float*)p(2), (float*)p(3), a.a, a.b,
                                      a.c, a.d, a.e, a.f, a.g, a.h, a.causal, a.i, a.j, a.alpha);
            break;
        case kOpGqaBwd:          // q, k, v, grad_out, probs, ds, dq, dk, dv | batch, tq, tk, heads, kv heads, hd, offset
            rc = mcl_cuda_gqa_backward(ctx, (const float*)p(0), (const float*)p(1), (const float*)p(2), (const float*)p(3),
                                       (float*)p(4), (float*)p(5), (float*)p(6), (float*)p(7), (float*)p(8), a.a, a.b, a.c,
                                       a.e, a.f, a.g, a.causal, a.i, a.alpha);
            break;
        case kOpEmbedding:       // token_weight, [pos_weight,] ids, out | tokens, vocab, seq_len, dim
            rc = mcl_cuda_token_position_embedding(ctx, (const float*)p(0), bufs.size() > 3 ? (const float*)p(1) : nullptr,
                                                   (const int32_t*)p(bufs.size() - 2), (float*)p(bufs.size() - 1), a.a, a.b,
                                                   a.c, a.d);
            break;
        case kOpEmbeddingBwd:    // ids, grad_out, grad_weight | vocab, dim, tokens, zero_first
            rc = mcl_cuda_embedding_weight_backward(ctx, (const int32_t*)p(0), (const float*)p(1), (float*)p(2), a.a, a.b, a.c,
                                                    a.causal);
            break;
        case kOpPositionBwd:     // grad_out, grad_position | batch, seq_len, dim
            rc = mcl_cuda_position_embedding_backward(ctx, (const float*)p(0), (float*)p(1), a.a, a.b, a.c);
            break;
        case kOpRope:            // x, out | batch, tokens, channels, heads, head_dim, rotary_dim, offset; theta; inverse, split
            rc = mcl_cuda_rope(ctx, (const float*)p(0), (float*)p(1), a.a, a.b, a.c, a.d, a.e, a.f, a.g, a.alpha, a.causal,
                               a.trans_a);
            break;
        case kOpAdam:            // param, grad, m, v | elements; lr, beta1, beta2, eps, weight_decay, c1, c2
            rc = mcl_cuda_adam_update(ctx, (float*)p(0), (const float*)p(1), (float*)p(2), (float*)p(3), a.a, a.f0, a.f1, a.f2,
                                      a.f3, a.f4, a.f5, a.f6);
            break;
        default:
            r.error = "unknown native operation";
            return r;
    }
    if (rc != MCL_CUDA_OK) { r.error = mcl_cuda_last_error(ctx); return r; }
    // Outside a batch the reference submits one command buffer and waits for its fence, so a caller that times
    // a call (benchmarks/bench_vulkan_perf.cpp: "dispatch + wait wall time") times the work, not the enqueue.
    if (!impl_->batch && mcl_cuda_finish(ctx) != MCL_CUDA_OK) { r.error = mcl_cuda_last_error(ctx); return r; }
    r.success = true;
    return r;
}
VulkanStorageBufferDispatchResult VulkanRuntime::dispatch_storage_buffers(
    const std::uint32_t*, std::size_t, const std::vector<VulkanStorageBufferSpec>&, const std::vector<std::size_t>&,
    std::uint32_t, std::uint32_t, std::uint32_t) {
    VulkanStorageBufferDispatchResult r;
    r.error = "SPIR-V dispatch is not implemented in CUDA runtime";
    return r;
}
VulkanStorageBufferDispatchResult VulkanRuntime::dispatch_storage_buffers(
    const std::uint32_t*, std::size_t, const std::vector<const VulkanBuffer*>&, const std::vector<std::size_t>&,
    std::uint32_t, std::uint32_t, std::uint32_t) {
    VulkanStorageBufferDispatchResult r;
    r.error = "SPIR-V dispatch is not implemented in CUDA runtime";
    return r;
}

// ---- probe ------------------------------------------------------------------------------------
VulkanProbeResult probe_vulkan_runtime() {
    VulkanProbeResult r;
    if (mcl_cuda_device_count() <= 0) {
        r.error = "no CUDA device available";
        return r;           // loader_found stays false: device tests skip, as without a Vulkan loader
    }
    mcl_cuda_ctx* ctx = nullptr;
    if (mcl_cuda_create(0, &ctx) != MCL_CUDA_OK) {
        r.error = mcl_cuda_last_error(nullptr);
        return r;
    }
    r.loader_found = true;
    r.instance_created = true;
    r.loader_path = "libmotifcl_cuda.so";
    r.physical_device_count = 1;
    VulkanPhysicalDeviceInfo d;
    d.name = mcl_cuda_device_name(ctx);
    d.vendor_id = 0x10DE;
    d.device_type = 2;      // discrete GPU
    r.devices.push_back(d);
    mcl_cuda_destroy(ctx);
    return r;
}

// ---- counter-synapse path and f32 matmuls ---------------------------------------------------------
namespace {
VulkanOpResult refuse(VulkanRuntime& rt, const std::string& msg) {
    VulkanOpResult r;
    r.device_name = rt.device_name();
    r.error = msg;
    return r;
}
VulkanOpResult native(VulkanRuntime& rt, NativeOp op, const std::vector<const VulkanBuffer*>& bufs, const NativeArgs& a) {
    return rt.dispatch_cached(kNativeTag, op, bufs, &a, sizeof(a), 1, 1, 1);
}
}  // namespace

// Buffer-size checks live here because the C ABI sees raw pointers; dimension and hyper-parameter
// checks are repeated inside the C ABI with the reference's wording.
VulkanOpResult run_vulkan_compact_counter_decode_weight(VulkanRuntime& rt, const VulkanBuffer& state,
                                                        const VulkanBuffer& scale, VulkanBuffer& weight,
                                                        std::size_t in_features, std::size_t out_features,
                                                        std::size_t C) {
    const std::size_t groups = out_features * (in_features / 4);
    if (state.nbytes() < groups * 3 || scale.nbytes() < out_features * 4 ||
        weight.nbytes() < out_features * in_features * 4)
        return refuse(rt, "Vulkan counter decode buffer is too small");
    NativeArgs a; a.a = in_features; a.b = out_features; a.c = C;
    return native(rt, kOpDecode, {&state, &scale, &weight}, a);
}
VulkanOpResult run_vulkan_compact_counter_forward_u8(VulkanRuntime& rt, const VulkanBuffer& x, const VulkanBuffer& state,
                                                     const VulkanBuffer& scale, VulkanBuffer& out, std::size_t batch,
                                                     std::size_t in_features, std::size_t out_features, std::size_t C) {
    if (x.nbytes() < batch * in_features * 4 || out.nbytes() < batch * out_features * 4 ||
        state.nbytes() < out_features * (in_features / 4) * 3 || scale.nbytes() < out_features * 4)
        return refuse(rt, "Vulkan counter forward buffer is too small");
    NativeArgs a; a.a = batch; a.b = in_features; a.c = out_features; a.d = C;
    return native(rt, kOpForward, {&x, &state, &scale, &out}, a);
}
VulkanOpResult run_vulkan_compact_counter_backward_input_u8(VulkanRuntime& rt, const VulkanBuffer& state,
                                                            const VulkanBuffer& scale, const VulkanBuffer& grad_out,
                                                            VulkanBuffer& grad_x, std::size_t batch,
                                                            std::size_t in_features, std::size_t out_features,
                                                            std::size_t C) {
    if (grad_out.nbytes() < batch * out_features * 4 || grad_x.nbytes() < batch * in_features * 4 ||
        state.nbytes() < out_features * (in_features / 4) * 3 || scale.nbytes() < out_features * 4)
        return refuse(rt, "Vulkan counter backward_input buffer is too small");
    NativeArgs a; a.a = batch; a.b = in_features; a.c = out_features; a.d = C;
    return native(rt, kOpBackwardInput, {&state, &scale, &grad_out, &grad_x}, a);
}
VulkanOpResult run_vulkan_compact_counter_apply_update_fused(VulkanRuntime& rt, VulkanBuffer& state, VulkanBuffer& scale,
                                                             VulkanBuffer& v, const VulkanBuffer& grad_out,
                                                             const VulkanBuffer& x, VulkanBuffer& scale_new_scratch,
                                                             VulkanBuffer& denom_scratch, std::size_t C,
                                                             std::size_t in_features, std::size_t out_features,
                                                             std::size_t batch, float lr, float lr_scale, float rms_beta,
                                                             float rms_eps, std::uint32_t seed) {
    if (in_features % 4 == 0 && state.nbytes() < out_features * (in_features / 4) * 3)
        return refuse(rt, "Vulkan counter update state buffer is too small");
    if (scale.nbytes() < out_features * 4 || v.nbytes() < out_features * 4 ||
        scale_new_scratch.nbytes() < out_features * 4 || denom_scratch.nbytes() < out_features * 4)
        return refuse(rt, "Vulkan counter update per-row buffer is too small");
    if (grad_out.nbytes() < batch * out_features * 4 || x.nbytes() < batch * in_features * 4)
        return refuse(rt, "Vulkan counter update activation buffer is too small");
    NativeArgs a; a.a = C; a.b = in_features; a.c = out_features; a.d = batch;
    a.lr = lr; a.lr_scale = lr_scale; a.rms_beta = rms_beta; a.rms_eps = rms_eps; a.seed = seed;
    return native(rt, kOpUpdateFused, {&state, &scale, &v, &grad_out, &x, &scale_new_scratch, &denom_scratch}, a);
}

namespace {
VulkanOpResult matmul(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b, VulkanBuffer& c, std::size_t m,
                      std::size_t k, std::size_t n, int ta, int tb) {
    if (a.nbytes() < m * k * 4 || b.nbytes() < k * n * 4 || c.nbytes() < m * n * 4)
        return refuse(rt, "Vulkan f32 matmul buffer is too small");
    NativeArgs g; g.a = m; g.b = k; g.c = n; g.trans_a = ta; g.trans_b = tb;
    return native(rt, kOpMatmul, {&a, &b, &c}, g);
}
}  // namespace
VulkanOpResult run_vulkan_f32_matmul(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b, VulkanBuffer& c,
                                     std::size_t m, std::size_t k, std::size_t n) { return matmul(rt, a, b, c, m, k, n, 0, 0); }
VulkanOpResult run_vulkan_f32_matmul_transpose_b(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b,
                                                 VulkanBuffer& c, std::size_t m, std::size_t k, std::size_t n) {
    return matmul(rt, a, b, c, m, k, n, 0, 1);
}
VulkanOpResult run_vulkan_f32_matmul_transpose_a(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b,
                                                 VulkanBuffer& c, std::size_t m, std::size_t k, std::size_t n) {
    return matmul(rt, a, b, c, m, k, n, 1, 0);
}
VulkanOpResult run_vulkan_f32_m1_matmul(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b, VulkanBuffer& c,
                                        std::size_t k, std::size_t n) { return matmul(rt, a, b, c, 1, k, n, 0, 0); }

namespace {
VulkanOpResult eltwise(VulkanRuntime& rt, int op, const VulkanBuffer* a, const VulkanBuffer* b, VulkanBuffer& out,
                       std::size_t elements, float alpha) {
    if (out.nbytes() < elements * 4 || (a && a->nbytes() < elements * 4) || (b && b->nbytes() < elements * 4))
        return refuse(rt, "Vulkan elementwise buffer is too small");
    NativeArgs g; g.a = elements; g.elt_op = op; g.alpha = alpha;
    std::vector<const VulkanBuffer*> bufs;
    if (a) bufs.push_back(a);
    if (b) bufs.push_back(b);
    bufs.push_back(&out);
    return native(rt, kOpEltwise, bufs, g);
}
}  // namespace
VulkanOpResult run_vulkan_add(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b, VulkanBuffer& out,
                              std::size_t n) { return eltwise(rt, MCL_CUDA_ELT_ADD, &a, &b, out, n, 0.0f); }
VulkanOpResult run_vulkan_sub(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b, VulkanBuffer& out,
                              std::size_t n) { return eltwise(rt, MCL_CUDA_ELT_SUB, &a, &b, out, n, 0.0f); }
VulkanOpResult run_vulkan_mul(VulkanRuntime& rt, const VulkanBuffer& a, const VulkanBuffer& b, VulkanBuffer& out,
                              std::size_t n) { return eltwise(rt, MCL_CUDA_ELT_MUL, &a, &b, out, n, 0.0f); }
VulkanOpResult run_vulkan_mul_scalar(VulkanRuntime& rt, const VulkanBuffer& x, VulkanBuffer& out, std::size_t n,
                                     float alpha) { return eltwise(rt, MCL_CUDA_ELT_MUL_SCALAR, &x, nullptr, out, n, alpha); }
VulkanOpResult run_vulkan_add_scalar(VulkanRuntime& rt, const VulkanBuffer& x, VulkanBuffer& out, std::size_t n,
                                     float value) { return eltwise(rt, MCL_CUDA_ELT_ADD_SCALAR, &x, nullptr, out, n, value); }
VulkanOpResult run_vulkan_zero_f32(VulkanRuntime& rt, VulkanBuffer& out, std::size_t n) {
    return eltwise(rt, MCL_CUDA_ELT_ZERO, nullptr, nullptr, out, n, 0.0f);
}
VulkanOpResult run_vulkan_sgd_update(VulkanRuntime& rt, const VulkanBuffer& param, const VulkanBuffer& grad,
                                     VulkanBuffer& out, std::size_t n, float lr) {
    return eltwise(rt, MCL_CUDA_ELT_SGD, &param, &grad, out, n, lr);
}

// ---- the fp32 row ops of the ternary15m block stack ------------------------------------------------
VulkanOpResult run_vulkan_rmsnorm(VulkanRuntime& rt, const VulkanBuffer& x, const VulkanBuffer& weight, VulkanBuffer& out,
                                  std::size_t rows, std::size_t cols, float eps) {
    if (x.nbytes() < rows * cols * 4 || out.nbytes() < rows * cols * 4 || weight.nbytes() < cols * 4)
        return refuse(rt, "Vulkan rmsnorm buffer is too small");
    NativeArgs a; a.a = rows; a.b = cols; a.alpha = eps;
    return native(rt, kOpRmsnorm, {&x, &weight, &out}, a);
}
VulkanOpResult run_vulkan_rmsnorm_backward_x(VulkanRuntime& rt, const VulkanBuffer& x, const VulkanBuffer& weight,
                                             const VulkanBuffer& grad_out, VulkanBuffer& grad_x, std::size_t rows,
                                             std::size_t cols, float eps) {
    if (x.nbytes() < rows * cols * 4 || grad_out.nbytes() < rows * cols * 4 || grad_x.nbytes() < rows * cols * 4 ||
        weight.nbytes() < cols * 4)
        return refuse(rt, "Vulkan rmsnorm backward_x buffer is too small");
    NativeArgs a; a.a = rows; a.b = cols; a.alpha = eps;
    return native(rt, kOpRmsnormBwdX, {&x, &weight, &grad_out, &grad_x}, a);
}
VulkanOpResult run_vulkan_rmsnorm_backward_weight(VulkanRuntime& rt, const VulkanBuffer& x, const VulkanBuffer& grad_out,
                                                  VulkanBuffer& row_inv_scratch, VulkanBuffer& grad_weight,
                                                  std::size_t rows, std::size_t cols, float eps) {
    if (x.nbytes() < rows * cols * 4 || grad_out.nbytes() < rows * cols * 4 || row_inv_scratch.nbytes() < rows * 4 ||
        grad_weight.nbytes() < cols * 4)
        return refuse(rt, "Vulkan rmsnorm backward_weight buffer is too small");
    NativeArgs a; a.a = rows; a.b = cols; a.alpha = eps;
    return native(rt, kOpRmsnormBwdW, {&x, &grad_out, &row_inv_scratch, &grad_weight}, a);
}
VulkanOpResult run_vulkan_swiglu(VulkanRuntime& rt, const VulkanBuffer& packed, VulkanBuffer& out, std::size_t rows,
                                 std::size_t hidden) {
    if (packed.nbytes() < rows * hidden * 8 || out.nbytes() < rows * hidden * 4)
        return refuse(rt, "Vulkan swiglu buffer is too small");
    NativeArgs a; a.a = rows; a.b = hidden;
    return native(rt, kOpSwiglu, {&packed, &out}, a);
}
VulkanOpResult run_vulkan_swiglu_backward(VulkanRuntime& rt, const VulkanBuffer& packed, const VulkanBuffer& grad_out,
                                          VulkanBuffer& grad_packed, std::size_t rows, std::size_t hidden) {
    if (packed.nbytes() < rows * hidden * 8 || grad_packed.nbytes() < rows * hidden * 8 ||
        grad_out.nbytes() < rows * hidden * 4)
        return refuse(rt, "Vulkan swiglu backward buffer is too small");
    NativeArgs a; a.a = rows; a.b = hidden;
    return native(rt, kOpSwigluBwd, {&packed, &grad_out, &grad_packed}, a);
}
VulkanOpResult run_vulkan_softmax_cross_entropy(VulkanRuntime& rt, const VulkanBuffer& logits, const VulkanBuffer& targets,
                                                VulkanBuffer& partial, VulkanBuffer& out, std::size_t rows,
                                                std::size_t cols) {
    if (logits.nbytes() < rows * cols * 4 || targets.nbytes() < rows * 4 || partial.nbytes() < rows * 4 || out.nbytes() < 4)
        return refuse(rt, "Vulkan softmax_cross_entropy buffer is too small");
    NativeArgs a; a.a = rows; a.b = cols;
    return native(rt, kOpCe, {&logits, &targets, &partial, &out}, a);
}
VulkanOpResult run_vulkan_softmax_cross_entropy_backward(VulkanRuntime& rt, const VulkanBuffer& logits,
                                                         const VulkanBuffer& targets, const VulkanBuffer& grad_out,
                                                         VulkanBuffer& grad_logits, std::size_t rows, std::size_t cols) {
    if (logits.nbytes() < rows * cols * 4 || grad_logits.nbytes() < rows * cols * 4 || targets.nbytes() < rows * 4 ||
        grad_out.nbytes() < 4)
        return refuse(rt, "Vulkan softmax_cross_entropy backward buffer is too small");
    NativeArgs a; a.a = rows; a.b = cols;
    return native(rt, kOpCeBwd, {&logits, &targets, &grad_out, &grad_logits}, a);
}
VulkanOpResult run_vulkan_grouped_query_attention_general(
    VulkanRuntime& rt, const VulkanBuffer& q, const VulkanBuffer& k, const VulkanBuffer& v, const VulkanBuffer* k_scales,
    const VulkanBuffer* v_scales, const VulkanBuffer* mask, VulkanBuffer& out, std::size_t batch, std::size_t query_tokens,
    std::size_t key_tokens, std::size_t key_stride, std::size_t n_head, std::size_t n_kv_head, std::size_t head_dim,
    std::size_t v_head_dim, bool causal, std::size_t query_offset, std::size_t sliding_window, std::uint32_t,
    std::uint32_t, std::uint32_t mask_dtype, std::uint32_t kv_dtype, float scale) {
    if (kv_dtype != 0 || k_scales != nullptr || v_scales != nullptr)
        return refuse(rt, "quantized keys/values are not implemented in CUDA runtime");
    if (mask != nullptr || mask_dtype != 0) return refuse(rt, "attention masks are not implemented in CUDA runtime");
    if (q.nbytes() < batch * query_tokens * n_head * head_dim * 4 || k.nbytes() < batch * key_stride * n_kv_head * head_dim * 4 ||
        v.nbytes() < batch * key_stride * n_kv_head * v_head_dim * 4 || out.nbytes() < batch * query_tokens * n_head * v_head_dim * 4)
        return refuse(rt, "Vulkan grouped_query_attention buffer is too small");
    NativeArgs a; a.a = batch; a.b = query_tokens; a.c = key_tokens; a.d = key_stride; a.e = n_head; a.f = n_kv_head;
    a.g = head_dim; a.h = v_head_dim; a.causal = causal ? 1 : 0; a.i = query_offset; a.j = sliding_window; a.alpha = scale;
    return native(rt, kOpGqa, {&q, &k, &v, &out}, a);
}
VulkanOpResult run_vulkan_grouped_query_attention(VulkanRuntime& rt, const VulkanBuffer& q, const VulkanBuffer& k,
                                                  const VulkanBuffer& v, VulkanBuffer& out, std::size_t query_tokens,
                                                  std::size_t key_tokens, std::size_t n_head, std::size_t n_kv_head,
                                                  std::size_t head_dim, float scale) {
    return run_vulkan_grouped_query_attention_general(rt, q, k, v, nullptr, nullptr, nullptr, out, 1, query_tokens, key_tokens,
                                                      key_tokens, n_head, n_kv_head, head_dim, head_dim, false, 0, 0, 0, 0,
                                                      0, 0, scale);
}
VulkanOpResult run_vulkan_grouped_query_attention_backward(
    VulkanRuntime& rt, const VulkanBuffer& q, const VulkanBuffer& k, const VulkanBuffer& v, const VulkanBuffer& grad_out,
    VulkanBuffer& probs_scratch, VulkanBuffer& ds_scratch, VulkanBuffer& grad_q, VulkanBuffer& grad_k, VulkanBuffer& grad_v,
    std::size_t batch, std::size_t query_tokens, std::size_t key_tokens, std::size_t n_head, std::size_t n_kv_head,
    std::size_t head_dim, bool causal, std::size_t query_offset, float scale) {
    const std::size_t qn = batch * query_tokens * n_head * head_dim * 4, kn = batch * key_tokens * n_kv_head * head_dim * 4;
    const std::size_t pn = batch * n_head * query_tokens * key_tokens * 4;
    if (q.nbytes() < qn || grad_out.nbytes() < qn || grad_q.nbytes() < qn || k.nbytes() < kn || v.nbytes() < kn ||
        grad_k.nbytes() < kn || grad_v.nbytes() < kn || probs_scratch.nbytes() < pn || ds_scratch.nbytes() < pn)
        return refuse(rt, "Vulkan grouped_query_attention backward buffer is too small");
    NativeArgs a; a.a = batch; a.b = query_tokens; a.c = key_tokens; a.e = n_head; a.f = n_kv_head; a.g = head_dim;
    a.causal = causal ? 1 : 0; a.i = query_offset; a.alpha = scale;
    return native(rt, kOpGqaBwd, {&q, &k, &v, &grad_out, &probs_scratch, &ds_scratch, &grad_q, &grad_k, &grad_v}, a);
}

// ---- embeddings, rope, adam ----------------------------------------------------------------------------
VulkanOpResult run_vulkan_token_position_embedding(VulkanRuntime& rt, const VulkanBuffer& token_weight,
                                                    const VulkanBuffer& pos_weight, const VulkanBuffer& token_ids,
                                                    VulkanBuffer& out, std::size_t vocab_size, std::size_t seq_len,
                                                    std::size_t embed_dim) {
    if (vocab_size == 0 || seq_len == 0 || embed_dim == 0)
        return refuse(rt, "Vulkan token+position embedding requires non-zero shapes");
    // as in the reference, the token count is implied by the output buffer
    const std::size_t tokens = out.nbytes() / (embed_dim * 4);
    if (tokens == 0) return refuse(rt, "Vulkan token+position embedding output buffer too small");
    if (token_ids.nbytes() < tokens * 4 || token_weight.nbytes() < vocab_size * embed_dim * 4 ||
        pos_weight.nbytes() < seq_len * embed_dim * 4)
        return refuse(rt, "Vulkan token+position embedding buffer is too small");
    NativeArgs a; a.a = tokens; a.b = vocab_size; a.c = seq_len; a.d = embed_dim;
    return native(rt, kOpEmbedding, {&token_weight, &pos_weight, &token_ids, &out}, a);
}
VulkanOpResult run_vulkan_embedding_gather(VulkanRuntime& rt, const VulkanBuffer& weight, const VulkanBuffer& indices,
                                           VulkanBuffer& out, std::size_t vocab_size, std::size_t embed_dim,
                                           std::size_t token_count) {
    if (indices.nbytes() < token_count * 4 || weight.nbytes() < vocab_size * embed_dim * 4 ||
        out.nbytes() < token_count * embed_dim * 4)
        return refuse(rt, "Vulkan embedding gather buffer is too small");
    NativeArgs a; a.a = token_count; a.b = vocab_size; a.c = 1; a.d = embed_dim;
    return native(rt, kOpEmbedding, {&weight, &indices, &out}, a);
}
namespace {
VulkanOpResult embedding_backward(VulkanRuntime& rt, const VulkanBuffer& indices, const VulkanBuffer& grad_out,
                                  VulkanBuffer& grad_weight, std::size_t vocab_size, std::size_t embed_dim,
                                  std::size_t token_count, int zero_first) {
    if (indices.nbytes() < token_count * 4 || grad_out.nbytes() < token_count * embed_dim * 4 ||
        grad_weight.nbytes() < vocab_size * embed_dim * 4)
        return refuse(rt, "Vulkan embedding weight backward buffer is too small");
    NativeArgs a; a.a = vocab_size; a.b = embed_dim; a.c = token_count; a.causal = zero_first;
    return native(rt, kOpEmbeddingBwd, {&indices, &grad_out, &grad_weight}, a);
}
}  // namespace
VulkanOpResult run_vulkan_embedding_weight_backward(VulkanRuntime& rt, const VulkanBuffer& indices, const VulkanBuffer& grad_out,
                                                    VulkanBuffer& grad_weight, std::size_t vocab_size, std::size_t embed_dim,
                                                    std::size_t token_count) {
    return embedding_backward(rt, indices, grad_out, grad_weight, vocab_size, embed_dim, token_count, 1);
}
VulkanOpResult run_vulkan_embedding_weight_backward_scatter(VulkanRuntime& rt, const VulkanBuffer& indices,
                                                            const VulkanBuffer& grad_out, VulkanBuffer& grad_weight,
                                                            std::size_t vocab_size, std::size_t embed_dim,
                                                            std::size_t token_count) {
    return embedding_backward(rt, indices, grad_out, grad_weight, vocab_size, embed_dim, token_count, 0);
}
VulkanOpResult run_vulkan_embedding_weight_backward_scatter_cas(VulkanRuntime& rt, const VulkanBuffer& indices,
                                                                const VulkanBuffer& grad_out, VulkanBuffer& grad_weight,
                                                                std::size_t vocab_size, std::size_t embed_dim,
                                                                std::size_t token_count) {
    return embedding_backward(rt, indices, grad_out, grad_weight, vocab_size, embed_dim, token_count, 0);
}
VulkanOpResult run_vulkan_position_embedding_backward(VulkanRuntime& rt, const VulkanBuffer& grad_out,
                                                       VulkanBuffer& grad_position, std::size_t batch, std::size_t seq_len,
                                                       std::size_t embed_dim) {
    if (grad_out.nbytes() < batch * seq_len * embed_dim * 4 || grad_position.nbytes() < seq_len * embed_dim * 4)
        return refuse(rt, "Vulkan position embedding backward buffer is too small");
    NativeArgs a; a.a = batch; a.b = seq_len; a.c = embed_dim;
    return native(rt, kOpPositionBwd, {&grad_out, &grad_position}, a);
}
namespace {
VulkanOpResult rope(VulkanRuntime& rt, const VulkanBuffer& x, VulkanBuffer& out, std::size_t batch, std::size_t tokens,
                    std::size_t channels, std::size_t n_head, std::size_t head_dim, std::size_t rotary_dim,
                    std::size_t token_offset, float theta, bool inverse, int split_half) {
    if (x.nbytes() < batch * tokens * channels * 4 || out.nbytes() < batch * tokens * channels * 4)
        return refuse(rt, "Vulkan rope buffer is too small");
    NativeArgs a; a.a = batch; a.b = tokens; a.c = channels; a.d = n_head; a.e = head_dim; a.f = rotary_dim; a.g = token_offset;
    a.alpha = theta; a.causal = inverse ? 1 : 0; a.trans_a = split_half;
    return native(rt, kOpRope, {&x, &out}, a);
}
}  // namespace
VulkanOpResult run_vulkan_rope(VulkanRuntime& rt, const VulkanBuffer& x, VulkanBuffer& out, std::size_t batch, std::size_t tokens,
                               std::size_t channels, std::size_t n_head, std::size_t head_dim, std::size_t rotary_dim,
                               std::size_t token_offset, float theta, bool inverse) {
    return rope(rt, x, out, batch, tokens, channels, n_head, head_dim, rotary_dim, token_offset, theta, inverse, 0);
}
VulkanOpResult run_vulkan_rope_split_half(VulkanRuntime& rt, const VulkanBuffer& x, VulkanBuffer& out, std::size_t batch,
                                          std::size_t tokens, std::size_t channels, std::size_t n_head, std::size_t head_dim,
                                          std::size_t rotary_dim, std::size_t token_offset, float theta, bool inverse) {
    return rope(rt, x, out, batch, tokens, channels, n_head, head_dim, rotary_dim, token_offset, theta, inverse, 1);
}
VulkanOpResult run_vulkan_adam_update_fast(VulkanRuntime& rt, const VulkanBuffer& param, const VulkanBuffer& grad,
                                           VulkanBuffer& m, VulkanBuffer& v, std::size_t elements, float lr, float beta1,
                                           float beta2, float eps, float weight_decay, float c1, float c2) {
    if (param.nbytes() < elements * 4 || grad.nbytes() < elements * 4 || m.nbytes() < elements * 4 || v.nbytes() < elements * 4)
        return refuse(rt, "Vulkan adam_update buffer is too small");
    NativeArgs a; a.a = elements; a.f0 = lr; a.f1 = beta1; a.f2 = beta2; a.f3 = eps; a.f4 = weight_decay; a.f5 = c1; a.f6 = c2;
    return native(rt, kOpAdam, {&param, &grad, &m, &v}, a);
}
}  // namespace motifcl
