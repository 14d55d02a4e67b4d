// C-ABI layer of libmotifcl_cuda.so: contexts, argument checks, dispatch to the kernels.
// The declarations and the reference interfaces they replace are in include/motifcl_cuda.h.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <set>
#include <string>
#include <vector>

#include "kernels.h"
#include "motifcl_cuda.h"

struct mcl_cuda_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int sm_count = 0;
    size_t max_smem = 0;
    size_t device_mem = 0;
    std::string name;
    std::string error;
    uint64_t launches = 0;
    // grow-only workspace used by entry points that need scratch (row tiles of grad_w, ...)
    void* ws = nullptr;
    size_t ws_bytes = 0;
    // how the contractions run (mcl_cuda_set_gemm_mode)
    int gemm_mode = MCL_CUDA_GEMM_AUTO;
    int act_terms = 3;
    int grad_terms = 6;
    int* err_word = nullptr;     // device word the tensor-core kernels set when a bounded wait gives up
    const uint32_t* seed_offset = nullptr;   // device word added to every update seed (mcl_cuda_set_seed_offset)
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    uint64_t lane_mark = 0;      // launches at the last lane_fork (when this context is a lane)
    bool recording = false;      // between mcl_cuda_batch_begin and mcl_cuda_batch_end
    uint64_t recorded_launches = 0;
    int live_batches = 0;        // recorded batches not yet destroyed: they hold addresses inside the workspace
};

// ticket words of the sliced table look-up GEMV, one per block of 256 output rows
constexpr int kGemvTicketWords = 4096;

struct mcl_cuda_batch {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;        // kernel launches one replay stands for
    mcl_cuda_ctx* ctx = nullptr; // the context it was recorded on (looked up among the live contexts before use)
};

namespace {

thread_local std::string g_error;   // errors raised before a context exists

// live contexts, so that a batch destroyed after its context does not touch freed memory
std::mutex g_ctx_mutex;
std::set<mcl_cuda_ctx*> g_live_ctx;

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
        if (ctx->recording)
            return fail(ctx, MCL_CUDA_EINVAL, "workspace would grow while recording a batch: run the same calls once unrecorded first");
        if (ctx->live_batches > 0)
            return fail(ctx, MCL_CUDA_EINVAL, "workspace would grow (to " + std::to_string(bytes) + " bytes) while " +
                                                  std::to_string(ctx->live_batches) + " recorded batch(es) hold addresses inside it: "
                                                  "run the largest call once before recording, or destroy the batches first");
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
#define MCL_NOT_RECORDING(ctx, what) do { if ((ctx)->recording) return fail(ctx, MCL_CUDA_EINVAL, what " is not allowed while recording a batch"); } while (0)
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
    ctx->device_mem = prop.totalGlobalMem;
    ctx->name = prop.name;
    DeviceGuard guard(device);
    if (own) {
        e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) { delete ctx; return fail_cuda(nullptr, "cudaStreamCreate", e); }
        ctx->own_stream = true;
    } else {
        ctx->stream = stream;
    }
    {   // keep freed blocks in the default pool instead of returning them to the driver at every synchronisation
        cudaMemPool_t pool = nullptr;
        unsigned long long keep = ~0ull;
        if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess)
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        cudaGetLastError();
    }
    // [0] error word, [1] work-item counter, [16 ...) ticket words of the table look-up GEMV (zero between launches)
    e = cudaMalloc(reinterpret_cast<void**>(&ctx->err_word), (16 + kGemvTicketWords) * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->err_word, 0, (16 + kGemvTicketWords) * sizeof(int));
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        return fail_cuda(nullptr, "context setup", e);
    }
    {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        g_live_ctx.insert(ctx);
    }
    *out_ctx = ctx;
    return MCL_CUDA_OK;
}

// Reads (after the stream has drained) whether a tensor-core kernel abandoned a wait.
int check_device_error(mcl_cuda_ctx* ctx) {
    int w = 0;
    cudaError_t e = cudaMemcpy(&w, ctx->err_word, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(ctx, "error-word read", e);
    if (w != 0) {
        cudaMemset(ctx->err_word, 0, sizeof(int));
        const char* who;
        switch (w) {
            case 1: case 11: who = "copy lane (ring slot never released)"; break;
            case 2: case 12: who = "MMA lane (operand tile never arrived)"; break;
            case 13: case 15: who = "epilogue / converter warps (accumulator or tile never completed)"; break;
            case 14: who = "MMA lane (accumulator never drained)"; break;
            case 16: case 17: who = "work-item queue (scheduler lane and its readers lost step)"; break;
            case 21: who = "wide-row counter update (a row slot was never marked ready or released)"; break;
            case 31: who = "peer all-reduce (a rank never announced its partial result)"; break;
            default: who = "epilogue (accumulator never completed)"; break;
        }
        return fail(ctx, MCL_CUDA_ECUDA, std::string("a kernel gave up a bounded wait: ") + who + " [code " +
                                             std::to_string(w) + "]; results of that call are invalid");
    }
    return MCL_CUDA_OK;
}

struct Carver {
    char* base = nullptr;
    size_t off = 0;
    size_t reserve(size_t bytes) { off = (off + 1023) & ~size_t(1023); const size_t at = off; off += bytes; return at; }
};

inline int up8(size_t x) { return (int)((x + 7) & ~size_t(7)); }

bool tc_wanted(const mcl_cuda_ctx* ctx, size_t M, size_t N, size_t K) {
    if (ctx->gemm_mode == MCL_CUDA_GEMM_EXACT) return false;
    if (N % 4 != 0) return false;                       // 128-bit stores of the output tile
    if (M > 0x7fffffffull / 2 || N > 0x7fffffffull / 2 || K > 0x7fffffffull / 2) return false;
    if (ctx->gemm_mode == MCL_CUDA_GEMM_TENSOR) return true;
    return (double)M * (double)N * (double)K >= (double)(1u << 22);
}

// term lists: product of plane pa of A with plane pb of B, smallest contributions first
void act_term_list(int act_terms, int* pa, int* pb, int* n) {
    *n = act_terms;
    for (int t = 0; t < act_terms; ++t) { pa[t] = act_terms - 1 - t; pb[t] = 0; }
}
void grad_term_list(int grad_terms, int* pa, int* pb, int* n, int* planes) {
    if (grad_terms >= 6) {
        const int a[6] = {2, 0, 1, 1, 0, 0}, b[6] = {0, 2, 1, 0, 1, 0};
        for (int t = 0; t < 6; ++t) { pa[t] = a[t]; pb[t] = b[t]; }
        *n = 6; *planes = 3;
    } else {
        const int a[3] = {1, 0, 0}, b[3] = {0, 1, 0};
        for (int t = 0; t < 3; ++t) { pa[t] = a[t]; pb[t] = b[t]; }
        *n = 3; *planes = 2;
    }
}

#define MCL_CU(ctx, what, call) do { cudaError_t _e = (call); if (_e != cudaSuccess) return fail_cuda(ctx, what, _e); } while (0)

// One tensor-core product on prepared planes (adds the split-K workspace to the carve).
int tc_product(mcl_cuda_ctx* ctx, const void* a, int a_planes, int lda, size_t a_stride, const void* b,
               int b_planes, int ldb, size_t b_stride, float* c, int ldc, int M, int N, int K, const int* pa,
               const int* pb, int nterms, const float* col_scale, float* splitk_ws, int splits) {
    int launches = 0;
    cudaError_t e = mcl::launch_tc_gemm(a, a_planes, lda, a_stride, b, b_planes, ldb, b_stride, c, ldc, M, N, K,
                                        pa, pb, nterms, col_scale, splitk_ws, splits, ctx->err_word,
                                        ctx->max_smem, ctx->sm_count, ctx->stream, &launches);
    ctx->launches += launches;
    if (e != cudaSuccess) return fail_cuda(ctx, "tensor-core contraction", e);
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
    {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        g_live_ctx.erase(ctx);
    }
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->err_word) cudaFree(ctx->err_word);
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    if (ctx->ev_join) cudaEventDestroy(ctx->ev_join);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}
const char* mcl_cuda_last_error(mcl_cuda_ctx* ctx) { return ctx ? ctx->error.c_str() : g_error.c_str(); }
const char* mcl_cuda_device_name(mcl_cuda_ctx* ctx) { return ctx ? ctx->name.c_str() : ""; }
int mcl_cuda_sm_count(mcl_cuda_ctx* ctx) { return ctx ? ctx->sm_count : 0; }
size_t mcl_cuda_device_memory_bytes(mcl_cuda_ctx* ctx) { return ctx ? ctx->device_mem : 0; }
uint64_t mcl_cuda_launch_count(mcl_cuda_ctx* ctx) { return ctx ? ctx->launches : 0; }
size_t mcl_cuda_workspace_bytes(mcl_cuda_ctx* ctx) { return ctx ? ctx->ws_bytes : 0; }

int mcl_cuda_batch_begin(mcl_cuda_ctx* ctx) {
    MCL_NEED_CTX(ctx);
    if (ctx->recording) return fail(ctx, MCL_CUDA_EINVAL, "batch_begin: already recording");
    if (ctx->stream == nullptr || ctx->stream == cudaStreamLegacy || ctx->stream == cudaStreamPerThread)
        return fail(ctx, MCL_CUDA_EUNSUPPORTED, "batch_begin: the context runs on a default stream, which cannot be recorded; "
                                              "create the context with its own stream");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return fail_cuda(ctx, "batch_begin", e);
    ctx->recording = true;
    ctx->recorded_launches = ctx->launches;
    return MCL_CUDA_OK;
}
int mcl_cuda_batch_end(mcl_cuda_ctx* ctx, mcl_cuda_batch** out_batch) {
    MCL_NEED_CTX(ctx);
    if (!out_batch) return fail(ctx, MCL_CUDA_EINVAL, "batch_end: out_batch is NULL");
    *out_batch = nullptr;
    if (!ctx->recording) return fail(ctx, MCL_CUDA_EINVAL, "batch_end without batch_begin");
    DeviceGuard guard(ctx->device);
    ctx->recording = false;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess || graph == nullptr) { cudaGetLastError(); return fail_cuda(ctx, "batch_end", e); }
    mcl_cuda_batch* b = new (std::nothrow) mcl_cuda_batch();
    if (!b) { cudaGraphDestroy(graph); return fail(ctx, MCL_CUDA_ENOMEM, "out of host memory"); }
    b->graph = graph;
    b->kernels = ctx->launches - ctx->recorded_launches;
    ctx->launches = ctx->recorded_launches;     // recorded, not run
    e = cudaGraphInstantiate(&b->exec, graph, 0);
    if (e != cudaSuccess) { cudaGraphDestroy(graph); delete b; return fail_cuda(ctx, "batch_end (instantiate)", e); }
    b->ctx = ctx;
    ++ctx->live_batches;
    *out_batch = b;
    return MCL_CUDA_OK;
}
int mcl_cuda_batch_launch(mcl_cuda_ctx* ctx, mcl_cuda_batch* batch) {
    MCL_NEED_CTX(ctx);
    if (!batch || !batch->exec) return fail(ctx, MCL_CUDA_EINVAL, "batch_launch: batch is NULL");
    MCL_NOT_RECORDING(ctx, "batch_launch");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaGraphLaunch(batch->exec, ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "batch_launch", e);
    ctx->launches += batch->kernels;
    return MCL_CUDA_OK;
}
void mcl_cuda_batch_destroy(mcl_cuda_batch* batch) {
    if (!batch) return;
    {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        if (batch->ctx && g_live_ctx.count(batch->ctx) && batch->ctx->live_batches > 0) --batch->ctx->live_batches;
    }
    if (batch->exec) cudaGraphExecDestroy(batch->exec);
    if (batch->graph) cudaGraphDestroy(batch->graph);
    delete batch;
}

int mcl_cuda_lane_fork(mcl_cuda_ctx* ctx, mcl_cuda_ctx* lane) {
    MCL_NEED_CTX(ctx);
    if (!lane || lane == ctx) return fail(ctx, MCL_CUDA_EINVAL, "lane_fork: lane must be another context");
    if (lane->device != ctx->device) return fail(ctx, MCL_CUDA_EINVAL, "lane_fork: lane is on another device");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaEventRecord(lane->ev_fork, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(lane->stream, lane->ev_fork, 0);
    if (e != cudaSuccess) return fail_cuda(ctx, "lane_fork", e);
    lane->recording = ctx->recording;
    lane->lane_mark = lane->launches;
    return MCL_CUDA_OK;
}
int mcl_cuda_lane_join(mcl_cuda_ctx* ctx, mcl_cuda_ctx* lane) {
    MCL_NEED_CTX(ctx);
    if (!lane || lane == ctx) return fail(ctx, MCL_CUDA_EINVAL, "lane_join: lane must be another context");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaEventRecord(lane->ev_join, lane->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, lane->ev_join, 0);
    if (e != cudaSuccess) return fail_cuda(ctx, "lane_join", e);
    lane->recording = false;
    ctx->launches += lane->launches - lane->lane_mark;    // account the lane's kernels to the owner
    lane->launches = lane->lane_mark;
    return MCL_CUDA_OK;
}

int mcl_cuda_finish(mcl_cuda_ctx* ctx) {
    MCL_NEED_CTX(ctx);
    MCL_NOT_RECORDING(ctx, "finish");
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "finish", e);
    return check_device_error(ctx);
}

int mcl_cuda_set_seed_offset(mcl_cuda_ctx* ctx, const uint32_t* device_word) {
    MCL_NEED_CTX(ctx);
    if (device_word && reinterpret_cast<uintptr_t>(device_word) % 4 != 0)
        return fail(ctx, MCL_CUDA_EINVAL, "set_seed_offset: pointer must be 4-byte aligned");
    ctx->seed_offset = device_word;
    return MCL_CUDA_OK;
}

int mcl_cuda_set_gemm_mode(mcl_cuda_ctx* ctx, int mode, int act_terms, int grad_terms) {
    MCL_NEED_CTX(ctx);
    if (mode != MCL_CUDA_GEMM_AUTO && mode != MCL_CUDA_GEMM_EXACT && mode != MCL_CUDA_GEMM_TENSOR)
        return fail(ctx, MCL_CUDA_EINVAL, "set_gemm_mode: unknown mode");
    if (act_terms != 2 && act_terms != 3) return fail(ctx, MCL_CUDA_EINVAL, "set_gemm_mode: act_terms must be 2 or 3");
    if (grad_terms != 3 && grad_terms != 6) return fail(ctx, MCL_CUDA_EINVAL, "set_gemm_mode: grad_terms must be 3 or 6");
    ctx->gemm_mode = mode; ctx->act_terms = act_terms; ctx->grad_terms = grad_terms;
    return MCL_CUDA_OK;
}
int mcl_cuda_alloc(mcl_cuda_ctx* ctx, size_t bytes, void** out_dptr) {
    MCL_NEED_CTX(ctx);
    MCL_NOT_RECORDING(ctx, "alloc");
    if (!out_dptr) return fail(ctx, MCL_CUDA_EINVAL, "alloc: out_dptr is NULL");
    *out_dptr = nullptr;
    if (bytes == 0) return fail(ctx, MCL_CUDA_EINVAL, "alloc: zero-size buffer");
    DeviceGuard guard(ctx->device);
    // Stream-ordered allocation from the device's default pool: a training step allocates and drops
    // hundreds of intermediate tensors, and the pool serves them without a device synchronisation.
    cudaError_t e = cudaMallocAsync(out_dptr, bytes, ctx->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, MCL_CUDA_ENOMEM, "alloc of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e));
    }
    return MCL_CUDA_OK;
}
int mcl_cuda_free(mcl_cuda_ctx* ctx, void* dptr) {
    MCL_NEED_CTX(ctx);
    MCL_NOT_RECORDING(ctx, "free");
    if (!dptr) return MCL_CUDA_OK;
    DeviceGuard guard(ctx->device);
    // Work that still uses the buffer may be queued: the free is ordered after it on the context's
    // stream, which keeps the reference's "free while pending is safe" behaviour without a wait.
    cudaError_t e = cudaFreeAsync(dptr, ctx->stream);
    if (e != cudaSuccess) return fail_cuda(ctx, "free", e);
    return MCL_CUDA_OK;
}
int mcl_cuda_upload(mcl_cuda_ctx* ctx, void* dst, const void* src_host, size_t bytes) {
    MCL_NEED_CTX(ctx);
    MCL_NOT_RECORDING(ctx, "upload");
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
    MCL_NOT_RECORDING(ctx, "download");
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

// defined below, with the grouped step
static bool fused_wanted(const mcl_cuda_ctx* ctx, const float* x, const float* grad_out, const void* ternary,
                         const float* scale, const float* y, const float* grad_x, const float* grad_w, size_t I,
                         size_t O, size_t Nt);
static int fused_products(mcl_cuda_ctx* ctx, const char* op, const float* x, const float* grad_out,
                          const uint8_t* state, const uint32_t* packed2, const float* scale, float* y,
                          float* grad_x, float* grad_w, size_t C, size_t I, size_t O, size_t Nt);

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
    // narrow layers: the tf32 hi/lo kernel reads x in place (no operand-splitting pass)
    if (tc_wanted(ctx, batch, out_features, in_features) &&
        fused_wanted(ctx, x, nullptr, state, scale, y, nullptr, nullptr, in_features, out_features, batch))
        return fused_products(ctx, op, x, nullptr, state, nullptr, scale, y, nullptr, nullptr, C, in_features, out_features, batch);
    if (tc_wanted(ctx, batch, out_features, in_features)) {
        const int ta = ctx->act_terms, ldi = up8(in_features);
        int splits = 1;
        const size_t sk = mcl::tc_splitk_workspace_bytes((int)batch, (int)out_features, (int)in_features,
                                                         ctx->sm_count, 0, &splits);
        Carver cv;
        const size_t o_x = cv.reserve((size_t)ta * batch * ldi * 2), o_t = cv.reserve(out_features * (size_t)ldi * 2),
                     o_k = cv.reserve(sk);
        void* wsp = nullptr;
        MCL_TRY(ws_reserve(ctx, cv.off, &wsp));
        char* w = static_cast<char*>(wsp);
        MCL_LAUNCH(ctx, op, mcl::launch_split_planes(x, (int)batch, (int)in_features, nullptr, w + o_x, ldi, ta,
                                                     nullptr, 0, 0, ctx->stream));
        MCL_LAUNCH(ctx, op, mcl::launch_expand_ternary(state, (int)C, (int)out_features, (int)in_features,
                                                       w + o_t, ldi, nullptr, 0, ctx->stream));
        int pa[6], pb[6], nt;
        act_term_list(ta, pa, pb, &nt);
        return tc_product(ctx, w + o_x, ta, ldi, batch * (size_t)ldi, w + o_t, 1, ldi, out_features * (size_t)ldi, y,
                          (int)out_features, (int)batch, (int)out_features, (int)in_features, pa, pb, nt, scale,
                          reinterpret_cast<float*>(w + o_k), splits);
    }
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
    if (tc_wanted(ctx, batch, in_features, out_features) &&
        fused_wanted(ctx, nullptr, grad_out, state, scale, nullptr, grad_x, nullptr, in_features, out_features, batch))
        return fused_products(ctx, op, nullptr, grad_out, state, nullptr, scale, nullptr, grad_x, nullptr, C, in_features, out_features, batch);
    if (tc_wanted(ctx, batch, in_features, out_features)) {
        const int ta = ctx->act_terms, ldo = up8(out_features);
        int splits = 1;
        const size_t sk = mcl::tc_splitk_workspace_bytes((int)batch, (int)in_features, (int)out_features,
                                                         ctx->sm_count, 0, &splits);
        Carver cv;
        const size_t o_g = cv.reserve((size_t)ta * batch * ldo * 2), o_t = cv.reserve(in_features * (size_t)ldo * 2),
                     o_k = cv.reserve(sk);
        void* wsp = nullptr;
        MCL_TRY(ws_reserve(ctx, cv.off, &wsp));
        char* w = static_cast<char*>(wsp);
        MCL_LAUNCH(ctx, op, mcl::launch_split_planes(grad_out, (int)batch, (int)out_features, scale, w + o_g, ldo, ta,
                                                     nullptr, 0, 0, ctx->stream));
        MCL_LAUNCH(ctx, op, mcl::launch_expand_ternary(state, (int)C, (int)out_features, (int)in_features,
                                                       nullptr, 0, w + o_t, ldo, ctx->stream));
        int pa[6], pb[6], nt;
        act_term_list(ta, pa, pb, &nt);
        return tc_product(ctx, w + o_g, ta, ldo, batch * (size_t)ldo, w + o_t, 1, ldo, in_features * (size_t)ldo,
                          grad_x, (int)in_features, (int)batch, (int)in_features, (int)out_features, pa, pb, nt,
                          nullptr, reinterpret_cast<float*>(w + o_k), splits);
    }
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
                                                     lr_scale, rms_beta, rms_eps, seed, ctx->seed_offset, ctx->err_word,
                                                     ctx->sm_count, ctx->max_smem, ctx->stream);
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
    // Row tile of grad_w: 1/8 of the dense [out,in] gradient, raised to 4 MiB where that is still under 1/5 of the
    // dense gradient (fewer launches for mid-sized layers) and capped at 32 MiB; at least one row; rounded to a multiple
    // of 128 rows when that fits.  The dense gradient is never materialised: the reference's memory-truth gate
    // (tests/test_memory_truth_gate.cpp:30-126) allows the update less than a quarter of a dense weight, and that
    // holds for every layer of more than four rows here.
    const size_t row_b = in_features * sizeof(float);
    const size_t dense = out_features * row_b;
    size_t budget = dense / 8;
    if (budget < (4u << 20)) budget = (4u << 20) < dense / 5 ? (4u << 20) : dense / 5;
    if (budget > (32u << 20)) budget = 32u << 20;
    size_t tile_rows = budget / row_b;
    if (tile_rows < 1) tile_rows = 1;
    if (tile_rows > 128) tile_rows &= ~size_t(127);
    if (tile_rows > out_features) tile_rows = out_features;
    DeviceGuard guard(ctx->device);
    const size_t state_row = in_features / 4 * 3;
    const bool tc = tc_wanted(ctx, tile_rows, in_features, batch) && tile_rows >= 64;
    int pa[6], pb[6], nt = 0, planes = 0, splits = 1;
    const int ldn = up8(batch);
    Carver cv;
    const size_t o_gw = cv.reserve(tile_rows * row_b);
    size_t o_a = 0, o_b = 0, o_k = 0;
    if (tc) {
        grad_term_list(ctx->grad_terms, pa, pb, &nt, &planes);
        const size_t sk = mcl::tc_splitk_workspace_bytes((int)tile_rows, (int)in_features, (int)batch,
                                                         ctx->sm_count, mcl::kGradDepthLimit, &splits);
        o_a = cv.reserve((size_t)planes * out_features * ldn * 2);   // dY^T term planes (activation-sized)
        o_b = cv.reserve((size_t)planes * in_features * ldn * 2);    // X^T term planes
        o_k = cv.reserve(sk);
    }
    void* wsp = nullptr;
    MCL_TRY(ws_reserve(ctx, cv.off, &wsp));
    char* w = static_cast<char*>(wsp);
    float* gw = reinterpret_cast<float*>(w + o_gw);
    if (tc) {
        MCL_LAUNCH(ctx, op, mcl::launch_split_planes(grad_out, (int)batch, (int)out_features, nullptr, nullptr, 0, 0,
                                                     w + o_a, ldn, planes, ctx->stream));
        MCL_LAUNCH(ctx, op, mcl::launch_split_planes(x, (int)batch, (int)in_features, nullptr, nullptr, 0, 0,
                                                     w + o_b, ldn, planes, ctx->stream));
    }
    for (size_t r0 = 0; r0 < out_features; r0 += tile_rows) {
        const size_t nr = (out_features - r0 < tile_rows) ? out_features - r0 : tile_rows;
        if (tc) {
            int sp = splits;
            MCL_TRY(tc_product(ctx, w + o_a + r0 * (size_t)ldn * 2, planes, ldn, out_features * (size_t)ldn,
                               w + o_b, planes, ldn, in_features * (size_t)ldn, gw, (int)in_features, (int)nr,
                               (int)in_features, (int)batch, pa, pb, nt, nullptr,
                               reinterpret_cast<float*>(w + o_k), sp));
        } else {
            MCL_LAUNCH(ctx, "counter update (grad_w tile)",
                       mcl::launch_simt_grad_w(grad_out, x, gw, (int)batch, (int)in_features,
                                               (int)out_features, (int)r0, (int)nr, ctx->stream));
        }
        int rc = mcl_cuda_counter_update_dense(ctx, state + r0 * state_row, scale + r0, v + r0, gw,
                                               packed2_out ? packed2_out + r0 * (in_features / 16) : nullptr,
                                               C, in_features, nr, r0, lr, lr_scale, rms_beta, rms_eps, seed);
        if (rc != MCL_CUDA_OK) return rc;
    }
    return MCL_CUDA_OK;
}

// Y, dX and dW of one linear; the ternary digits come from the packed 6-bit state or, when
// state == NULL, from the 2-bit packed weights.
// Narrow layers take the grouped kernel that splits fp32 operands in shared memory (tc_fused.cu):
// every column tile of a product converts its A slab again, so the form pays while a layer has few
// column tiles; wide layers amortise the pre-split planes of tc_gemm.cu better.
static bool fused_wanted(const mcl_cuda_ctx* ctx, const float* x, const float* grad_out, const void* ternary,
                         const float* scale, const float* y, const float* grad_x, const float* grad_w, size_t I,
                         size_t O, size_t Nt) {
    (void)ternary;
    if (I % 32 != 0 || O % 32 != 0 || Nt % 4 != 0 || I > 1024 || O > 1024) return false;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(grad_out) |
                           reinterpret_cast<uintptr_t>(scale) | reinterpret_cast<uintptr_t>(y) |
                           reinterpret_cast<uintptr_t>(grad_x) | reinterpret_cast<uintptr_t>(grad_w);
    if (bits & 15) return false;
    return 200 * (size_t)1024 <= ctx->max_smem;
}

static int fused_products(mcl_cuda_ctx* ctx, const char* op, const float* x, const float* grad_out,
                          const uint8_t* state, const uint32_t* packed2, const float* scale, float* y,
                          float* grad_x, float* grad_w, size_t C, size_t I, size_t O, size_t Nt) {
    mcl::FusedProblem pr[3];
    mcl::FusedOperand oa[3], ob[3];
    int n = 0, i_dw = -1;
    size_t k_floats = 0;
    // the kernel's split-K slices are 32 deep; the depth limit is stated in k-tiles of 64
    const int depth = mcl::kFusedDwDepth;
    auto add = [&](int mode, int M, int N, int K) {
        mcl::FusedProblem& p = pr[n];
        p = mcl::FusedProblem();
        p.mode = mode; p.M = M; p.N = N; p.K = K;
        return &p;
    };
    auto operand = [](const float* p, size_t rows, size_t cols, int mn, int box_outer) {
        mcl::FusedOperand o = {p, (int)rows, (int)cols, (int)cols, mn, box_outer};
        return o;
    };
    if (grad_w) {      // the long work items (K = tokens) first
        mcl::FusedProblem* p = add(mcl::kFusedDW, (int)O, (int)I, (int)Nt);
        p->C = grad_w; p->ldc = (int)I;
        k_floats = mcl::fused_plan(p, ctx->sm_count, depth);
        oa[n] = operand(grad_out, Nt, O, 1, 4); ob[n] = operand(x, Nt, I, 1, p->BN / 32); i_dw = n++;
    }
    if (y) {
        mcl::FusedProblem* p = add(mcl::kFusedY, (int)Nt, (int)O, (int)I);
        p->col_scale = scale; p->C = y; p->ldc = (int)O;
        mcl::fused_plan(p, 0, 0);
        oa[n] = operand(x, Nt, I, 0, 128); ob[n] = operand(nullptr, O, I, 0, p->BN); ++n;
    }
    if (grad_x) {
        mcl::FusedProblem* p = add(mcl::kFusedDX, (int)Nt, (int)I, (int)O);
        p->a_kscale = scale; p->C = grad_x; p->ldc = (int)I;
        mcl::fused_plan(p, 0, 0);
        oa[n] = operand(grad_out, Nt, O, 0, 128); ob[n] = operand(nullptr, O, I, 1, p->BN / 32); ++n;
    }
    Carver cv;
    const size_t o_t = cv.reserve((y || grad_x) ? O * I * 4 : 0);
    const size_t o_k = cv.reserve(k_floats * 4);
    void* wsp = nullptr;
    MCL_TRY(ws_reserve(ctx, cv.off, &wsp));
    char* w = static_cast<char*>(wsp);
    if (y || grad_x) {   // the ternary digits as fp32: the exact operand of Y and dX
        float* T = reinterpret_cast<float*>(w + o_t);
        MCL_LAUNCH(ctx, op, mcl::launch_ternary_f32(state, packed2, (int)C, (int)O, (int)I, T, ctx->sm_count, ctx->stream));
        for (int i = 0; i < n; ++i)
            if (pr[i].mode != mcl::kFusedDW) ob[i].ptr = T;
    }
    if (i_dw >= 0 && pr[i_dw].splits > 1) pr[i_dw].C = reinterpret_cast<float*>(w + o_k);
    int launches = 0;
    cudaError_t e = mcl::launch_tc_fused(pr, oa, ob, n, ctx->err_word, ctx->max_smem, ctx->sm_count, ctx->stream,
                                         &launches);
    ctx->launches += launches;
    if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    if (i_dw >= 0 && pr[i_dw].splits > 1)
        MCL_LAUNCH(ctx, op, mcl::launch_splitk_reduce(reinterpret_cast<const float*>(w + o_k), grad_w, nullptr, (int)O, (int)I,
                                                      (int)I, pr[i_dw].splits, ctx->stream));
    return MCL_CUDA_OK;
}

static int linear_products(mcl_cuda_ctx* ctx, const char* op, const float* x, const float* grad_out,
                           const uint8_t* state, const uint32_t* packed2, const float* scale, float* y,
                           float* grad_x, float* grad_w, size_t C, size_t I, size_t O, size_t Nt) {
    const bool tc = tc_wanted(ctx, Nt, O, I) && tc_wanted(ctx, Nt, I, O) && tc_wanted(ctx, O, I, Nt);
    if (!tc) {
        if (state) {
            if (y) MCL_TRY(mcl_cuda_counter_forward(ctx, x, state, scale, y, Nt, I, O, C));
            if (grad_x) MCL_TRY(mcl_cuda_counter_backward_input(ctx, state, scale, grad_out, grad_x, Nt, I, O, C));
        } else {
            if (y) MCL_LAUNCH(ctx, op, mcl::launch_simt_ternary_forward(x, packed2, scale, y, (int)Nt, (int)I, (int)O, ctx->stream));
            if (grad_x) MCL_LAUNCH(ctx, op, mcl::launch_simt_ternary_backward_input(packed2, scale, grad_out, grad_x, (int)Nt,
                                                                                 (int)I, (int)O, ctx->stream));
        }
        if (grad_w) MCL_TRY(mcl_cuda_matmul_f32(ctx, grad_out, x, grad_w, O, Nt, I, 1, 0));
        return MCL_CUDA_OK;
    }
    if (fused_wanted(ctx, x, grad_out, state ? static_cast<const void*>(state) : packed2, scale, y, grad_x, grad_w, I, O, Nt))
        return fused_products(ctx, op, x, grad_out, state, packed2, scale, y, grad_x, grad_w, C, I, O, Nt);
    const int ta = ctx->act_terms;
    int pa[6], pb[6], nt, gp;
    grad_term_list(ctx->grad_terms, pa, pb, &nt, &gp);
    const int ldi = up8(I), ldo = up8(O), ldn = up8(Nt);
    int s_y = 1, s_x = 1, s_w = 1;
    const size_t k_y = mcl::tc_splitk_workspace_bytes((int)Nt, (int)O, (int)I, ctx->sm_count, 0, &s_y);
    const size_t k_x = mcl::tc_splitk_workspace_bytes((int)Nt, (int)I, (int)O, ctx->sm_count, 0, &s_x);
    const size_t k_w = mcl::tc_splitk_workspace_bytes((int)O, (int)I, (int)Nt, ctx->sm_count, mcl::kGradDepthLimit, &s_w);
    size_t k_max = k_y > k_x ? k_y : k_x;
    if (k_w > k_max) k_max = k_w;
    Carver cv;
    const size_t o_xp = cv.reserve((size_t)ta * Nt * ldi * 2);    // X terms        [ta][N][I]
    const size_t o_xt = cv.reserve((size_t)gp * I * ldn * 2);     // X^T terms      [gp][I][N]
    const size_t o_gp = cv.reserve((size_t)ta * Nt * ldo * 2);    // (dY.s) terms   [ta][N][O]
    const size_t o_gt = cv.reserve((size_t)gp * O * ldn * 2);     // dY^T terms     [gp][O][N]
    const size_t o_t = cv.reserve(O * (size_t)ldi * 2);           // T   [O][I]
    const size_t o_tt = cv.reserve(I * (size_t)ldo * 2);          // T^T [I][O]
    const size_t o_k = cv.reserve(k_max);
    void* wsp = nullptr;
    MCL_TRY(ws_reserve(ctx, cv.off, &wsp));
    char* w = static_cast<char*>(wsp);
    float* kws = reinterpret_cast<float*>(w + o_k);
    // each fp32 tensor is read once and written as terms in the orientations its products need
    MCL_LAUNCH(ctx, op, mcl::launch_split_planes(x, (int)Nt, (int)I, nullptr, y ? w + o_xp : nullptr, ldi, ta,
                                                 grad_w ? w + o_xt : nullptr, ldn, gp, ctx->stream));
    if (state)
        MCL_LAUNCH(ctx, op, mcl::launch_expand_ternary(state, (int)C, (int)O, (int)I, y ? w + o_t : nullptr, ldi,
                                                       grad_x ? w + o_tt : nullptr, ldo, ctx->stream));
    else
        MCL_LAUNCH(ctx, op, mcl::launch_expand_ternary_p2(packed2, (int)O, (int)I, y ? w + o_t : nullptr, ldi,
                                                          grad_x ? w + o_tt : nullptr, ldo, ctx->stream));
    MCL_LAUNCH(ctx, op, mcl::launch_split_planes(grad_out, (int)Nt, (int)O, scale, grad_x ? w + o_gp : nullptr, ldo, ta,
                                                 grad_w ? w + o_gt : nullptr, ldn, gp, ctx->stream));
    int qa[6], qb[6], qn;
    act_term_list(ta, qa, qb, &qn);
    if (y) MCL_TRY(tc_product(ctx, w + o_xp, ta, ldi, Nt * (size_t)ldi, w + o_t, 1, ldi, O * (size_t)ldi, y, (int)O,
                              (int)Nt, (int)O, (int)I, qa, qb, qn, scale, kws, s_y));
    if (grad_x) MCL_TRY(tc_product(ctx, w + o_gp, ta, ldo, Nt * (size_t)ldo, w + o_tt, 1, ldo, I * (size_t)ldo, grad_x,
                                   (int)I, (int)Nt, (int)I, (int)O, qa, qb, qn, nullptr, kws, s_x));
    if (grad_w) MCL_TRY(tc_product(ctx, w + o_gt, gp, ldn, O * (size_t)ldn, w + o_xt, gp, ldn, I * (size_t)ldn, grad_w,
                                   (int)I, (int)O, (int)I, (int)Nt, pa, pb, nt, nullptr, kws, s_w));
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_linear_step(mcl_cuda_ctx* ctx, const float* x, const float* grad_out,
                                 uint8_t* state, float* scale, float* v, float* y, float* grad_x,
                                 float* grad_w, uint32_t* packed2_out, size_t C, size_t in_features,
                                 size_t out_features, size_t batch, size_t update_rows,
                                 size_t row_offset, float lr, float lr_scale, float rms_beta,
                                 float rms_eps, uint32_t seed) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter linear step";
    MCL_TRY(check_counter_dims(ctx, op, C, in_features, out_features));
    if (batch == 0 || batch > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "counter linear step requires 0 < batch < 2^31");
    MCL_TRY(check_hypers(ctx, op, lr, lr_scale, rms_beta, rms_eps));
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "state", state, 1));
    MCL_TRY(check_ptr(ctx, op, "scale", scale, 4));
    MCL_TRY(check_ptr(ctx, op, "v", v, 4));
    if (grad_w) MCL_TRY(check_ptr(ctx, op, "grad_w", grad_w, 16));
    else if (update_rows != 0) return fail(ctx, MCL_CUDA_EINVAL, "counter linear step: an update needs grad_w");
    if (row_offset + update_rows > out_features)
        return fail(ctx, MCL_CUDA_EINVAL, "counter linear step: update rows exceed out_features");
    const size_t state_row = in_features / 4 * 3;
    const size_t I = in_features;
    DeviceGuard guard(ctx->device);
    MCL_TRY(linear_products(ctx, op, x, grad_out, state, nullptr, scale, y, grad_x, grad_w, C, in_features,
                            out_features, batch));
    if (update_rows > 0)
        return mcl_cuda_counter_update_dense(ctx, state + row_offset * state_row, scale + row_offset, v + row_offset,
                                             grad_w + row_offset * I,
                                             packed2_out ? packed2_out + row_offset * (I / 16) : nullptr, C, I,
                                             update_rows, row_offset, lr, lr_scale, rms_beta, rms_eps, seed);
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_linear_step_many(mcl_cuda_ctx* ctx, const mcl_cuda_linear_desc* layers, size_t n_layers,
                                      size_t C, float lr, float lr_scale, float rms_beta, float rms_eps,
                                      uint32_t seed) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter linear step (many)";
    if (!layers || n_layers == 0) return fail(ctx, MCL_CUDA_EINVAL, "counter linear step (many): no layers");
    MCL_TRY(check_hypers(ctx, op, lr, lr_scale, rms_beta, rms_eps));
    std::vector<size_t> grouped, single;
    for (size_t i = 0; i < n_layers; ++i) {
        const mcl_cuda_linear_desc& L = layers[i];
        MCL_TRY(check_counter_dims(ctx, op, C, L.in_features, L.out_features));
        if (L.batch == 0 || L.batch > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "counter linear step (many) requires 0 < batch < 2^31");
        MCL_TRY(check_ptr(ctx, op, "x", L.x, 4));
        MCL_TRY(check_ptr(ctx, op, "grad_out", L.grad_out, 4));
        MCL_TRY(check_ptr(ctx, op, "scale", L.scale, 4));
        if (L.grad_w) MCL_TRY(check_ptr(ctx, op, "grad_w", L.grad_w, 16));
        else if (L.update_rows != 0) return fail(ctx, MCL_CUDA_EINVAL, "counter linear step (many): an update needs grad_w");
        if (!L.grad_w && !L.y && !L.grad_x) return fail(ctx, MCL_CUDA_EINVAL, "counter linear step (many): a layer asks for no product");
        if (L.state != nullptr) {
            MCL_TRY(check_ptr(ctx, op, "v", L.v, 4));
        } else {
            MCL_TRY(check_ptr(ctx, op, "packed2_in", L.packed2_in, 4));
            if (L.update_rows != 0)
                return fail(ctx, MCL_CUDA_EINVAL, "counter linear step (many): a layer given by its 2-bit words cannot be updated");
            if (L.in_features % 16 != 0)
                return fail(ctx, MCL_CUDA_EINVAL, "counter linear step (many): 2-bit words require in_features % 16 == 0");
        }
        if (L.row_offset + L.update_rows > L.out_features)
            return fail(ctx, MCL_CUDA_EINVAL, "counter linear step (many): update rows exceed out_features");
        const bool tc = tc_wanted(ctx, L.batch, L.out_features, L.in_features);
        const void* tern = L.state ? static_cast<const void*>(L.state) : L.packed2_in;
        if (tc && fused_wanted(ctx, L.x, L.grad_out, tern, L.scale, L.y, L.grad_x, L.grad_w, L.in_features, L.out_features,
                               L.batch))
            grouped.push_back(i);
        else
            single.push_back(i);
    }
    DeviceGuard guard(ctx->device);
    for (size_t i : single) {
        const mcl_cuda_linear_desc& L = layers[i];
        if (L.state == nullptr) {
            MCL_TRY(mcl_cuda_ternary_linear_products(ctx, L.x, L.grad_out, L.packed2_in, L.scale, L.y, L.grad_x, L.grad_w,
                                                     L.in_features, L.out_features, L.batch));
            continue;
        }
        MCL_TRY(mcl_cuda_counter_linear_step(ctx, L.x, L.grad_out, L.state, L.scale, L.v, L.y, L.grad_x, L.grad_w, L.packed2_out,
                                             C, L.in_features, L.out_features, L.batch, L.update_rows, L.row_offset, lr,
                                             lr_scale, rms_beta, rms_eps, seed));
    }
    if (grouped.empty()) return MCL_CUDA_OK;
    const int depth = mcl::kFusedDwDepth;
    const size_t ng = grouped.size();
    // with many layers in flight the K splits of dW only have to respect the accumulation depth
    const int target_items = (int)((2 * (size_t)ctx->sm_count + ng - 1) / ng);
    std::vector<mcl::FusedProblem> pr;
    std::vector<mcl::FusedOperand> oa, ob;
    std::vector<size_t> t_off(ng), k_off(ng);
    std::vector<int> dw_splits(ng, 1);
    Carver cv;
    auto operand = [](const float* p, size_t rows, size_t cols, int mn, int box_outer) {
        mcl::FusedOperand o = {p, (int)rows, (int)cols, (int)cols, mn, box_outer};
        return o;
    };
    for (size_t gi = 0; gi < ng; ++gi) {
        const mcl_cuda_linear_desc& L = layers[grouped[gi]];
        t_off[gi] = cv.reserve((L.y || L.grad_x) ? L.out_features * L.in_features * 4 : 0);
        if (!L.grad_w) { k_off[gi] = cv.reserve(0); continue; }
        mcl::FusedProblem p = mcl::FusedProblem();
        p.mode = mcl::kFusedDW; p.M = (int)L.out_features; p.N = (int)L.in_features; p.K = (int)L.batch;
        k_off[gi] = cv.reserve(mcl::fused_plan(&p, target_items, depth) * 4);
        dw_splits[gi] = p.splits;
    }
    void* wsp = nullptr;
    MCL_TRY(ws_reserve(ctx, cv.off, &wsp));
    char* w = static_cast<char*>(wsp);
    // 1. ternary digits of every layer with a row product, as bf16: T [O][I] in the first half of the layer's block,
    // its transpose after it
    {
        std::vector<const uint8_t*> st;
        std::vector<const uint32_t*> p2;
        std::vector<void*> T, Tt;
        std::vector<int> Os, Is;
        for (size_t gi = 0; gi < ng; ++gi) {
            const mcl_cuda_linear_desc& L = layers[grouped[gi]];
            if (!L.y && !L.grad_x) continue;
            st.push_back(L.state); p2.push_back(L.packed2_in);
            T.push_back(w + t_off[gi]); Tt.push_back(w + t_off[gi] + L.out_features * L.in_features * 2);
            Os.push_back((int)L.out_features); Is.push_back((int)L.in_features);
        }
        int launches = 0;
        cudaError_t e = st.empty() ? cudaSuccess
                                   : mcl::launch_ternary_bf16_group(st.data(), p2.data(), T.data(), Tt.data(), Os.data(), Is.data(), (int)st.size(), (int)C,
                                                                    ctx->sm_count, ctx->stream, &launches);
        ctx->launches += launches;
        if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    }
    // 2. all products.  The weight-gradient products (tf32 terms, K = tokens, long work items) and the row products
    // (bf16 terms against the bf16 digits, 64-deep k-tiles) run in launches of their own: their tiles differ in size,
    // and a launch sizes its rings for the largest tile of its table.
    {
        auto flush = [&]() -> cudaError_t {
            if (pr.empty()) return cudaSuccess;
            int launches = 0;
            cudaError_t e = mcl::launch_tc_fused(pr.data(), oa.data(), ob.data(), (int)pr.size(), ctx->err_word, ctx->max_smem,
                                                 ctx->sm_count, ctx->stream, &launches);
            ctx->launches += launches;
            pr.clear(); oa.clear(); ob.clear();
            return e;
        };
        auto operand_bf16 = [](const void* p, size_t rows, size_t cols, int box_outer) {
            mcl::FusedOperand o = {static_cast<const float*>(p), (int)rows, (int)cols, (int)cols, 0, box_outer, 1};
            return o;
        };
        for (size_t gi = 0; gi < ng; ++gi) {
            const mcl_cuda_linear_desc& L = layers[grouped[gi]];
            const size_t I = L.in_features, O = L.out_features, Nt = L.batch;
            if (!L.grad_w) continue;
            mcl::FusedProblem p = mcl::FusedProblem();
            p.mode = mcl::kFusedDW; p.M = (int)O; p.N = (int)I; p.K = (int)Nt;
            mcl::fused_plan(&p, target_items, depth);
            p.C = p.splits > 1 ? reinterpret_cast<float*>(w + k_off[gi]) : L.grad_w; p.ldc = (int)I;
            pr.push_back(p); oa.push_back(operand(L.grad_out, Nt, O, 1, 4)); ob.push_back(operand(L.x, Nt, I, 1, p.BN / 32));
            if (pr.size() == (size_t)mcl::kFusedMaxProblems) {
                cudaError_t e = flush();
                if (e != cudaSuccess) return fail_cuda(ctx, op, e);
            }
        }
        {
            cudaError_t e = flush();
            if (e != cudaSuccess) return fail_cuda(ctx, op, e);
        }
        // row products: launches of equal size
        size_t n_row = 0;
        for (size_t gi = 0; gi < ng; ++gi) n_row += (layers[grouped[gi]].y ? 1 : 0) + (layers[grouped[gi]].grad_x ? 1 : 0);
        const size_t n_launch = (n_row + mcl::kFusedMaxProblems - 1) / mcl::kFusedMaxProblems;
        const size_t per_launch = n_launch ? (n_row + n_launch - 1) / n_launch : 0;
        for (size_t gi = 0; gi < ng; ++gi) {
            const mcl_cuda_linear_desc& L = layers[grouped[gi]];
            const size_t I = L.in_features, O = L.out_features, Nt = L.batch;
            const char* T = w + t_off[gi];
            const char* Tt = T + O * I * 2;
            mcl::FusedProblem p;
            if (L.y) {
                p = mcl::FusedProblem();
                p.mode = mcl::kFusedYB; p.M = (int)Nt; p.N = (int)O; p.K = (int)I;
                p.col_scale = L.scale; p.C = L.y; p.ldc = (int)O;
                mcl::fused_plan(&p, 0, 0);
                pr.push_back(p); oa.push_back(operand(L.x, Nt, I, 0, 128)); ob.push_back(operand_bf16(T, O, I, p.BN));
            }
            if (L.grad_x) {
                p = mcl::FusedProblem();
                p.mode = mcl::kFusedDXB; p.M = (int)Nt; p.N = (int)I; p.K = (int)O;
                p.a_kscale = L.scale; p.C = L.grad_x; p.ldc = (int)I;
                mcl::fused_plan(&p, 0, 0);
                pr.push_back(p); oa.push_back(operand(L.grad_out, Nt, O, 0, 128)); ob.push_back(operand_bf16(Tt, I, O, p.BN));
            }
            if (pr.size() + 2 > per_launch || pr.size() + 2 > (size_t)mcl::kFusedMaxProblems) {
                cudaError_t e = flush();
                if (e != cudaSuccess) return fail_cuda(ctx, op, e);
            }
        }
        cudaError_t e = flush();
        if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    }
    // 3. split-K reductions of dW
    {
        std::vector<const float*> part;
        std::vector<float*> out;
        std::vector<int> elems, splits;
        for (size_t gi = 0; gi < ng; ++gi) {
            if (dw_splits[gi] <= 1) continue;
            const mcl_cuda_linear_desc& L = layers[grouped[gi]];
            part.push_back(reinterpret_cast<const float*>(w + k_off[gi]));
            out.push_back(L.grad_w);
            elems.push_back((int)(L.out_features * L.in_features));
            splits.push_back(dw_splits[gi]);
        }
        if (!part.empty()) {
            int launches = 0;
            cudaError_t e = mcl::launch_splitk_reduce_group(part.data(), out.data(), elems.data(), splits.data(), (int)part.size(),
                                                            ctx->sm_count, ctx->stream, &launches);
            ctx->launches += launches;
            if (e != cudaSuccess) return fail_cuda(ctx, op, e);
        }
    }
    // 4. updates
    {
        std::vector<mcl::UpdateDesc> ud;
        for (size_t gi = 0; gi < ng; ++gi) {
            const mcl_cuda_linear_desc& L = layers[grouped[gi]];
            if (L.update_rows == 0) continue;
            if ((L.row_offset + L.update_rows) * L.in_features > 0xffffffffull)
                return fail(ctx, MCL_CUDA_EINVAL, "counter update: (row_offset + rows) * in_features exceeds 32-bit element indexing");
            const size_t I = L.in_features, rb = I / 4 * 3;
            mcl::UpdateDesc u;
            u.state = L.state + L.row_offset * rb; u.scale = L.scale + L.row_offset; u.v = L.v + L.row_offset;
            u.grad_w = L.grad_w + L.row_offset * I;
            u.packed2 = L.packed2_out ? L.packed2_out + L.row_offset * (I / 16) : nullptr;
            u.in_features = (int)I; u.rows = (int)L.update_rows; u.row_offset = (int)L.row_offset;
            ud.push_back(u);
        }
        if (!ud.empty()) {
            int launches = 0;
            cudaError_t e = mcl::launch_counter_update_group(ud.data(), (int)ud.size(), (int)C, lr, lr_scale, rms_beta, rms_eps, seed,
                                                             ctx->seed_offset, ctx->err_word, ctx->sm_count, ctx->max_smem, ctx->stream, &launches);
            ctx->launches += launches;
            if (e == cudaErrorNotSupported) {
                for (const mcl::UpdateDesc& u : ud)
                    MCL_TRY(mcl_cuda_counter_update_dense(ctx, u.state, u.scale, u.v, u.grad_w, u.packed2, C, (size_t)u.in_features,
                                                          (size_t)u.rows, (size_t)u.row_offset, lr, lr_scale, rms_beta, rms_eps, seed));
            } else if (e != cudaSuccess) {
                return fail_cuda(ctx, op, e);
            }
        }
    }
    return MCL_CUDA_OK;
}

int mcl_cuda_counter_update_dense_many(mcl_cuda_ctx* ctx, const mcl_cuda_update_desc* layers, size_t n_layers,
                                       size_t C, float lr, float lr_scale, float rms_beta, float rms_eps,
                                       uint32_t seed) {
    MCL_NEED_CTX(ctx);
    const char* op = "counter update (many)";
    if (!layers || n_layers == 0) return fail(ctx, MCL_CUDA_EINVAL, "counter update (many): no layers");
    MCL_TRY(check_hypers(ctx, op, lr, lr_scale, rms_beta, rms_eps));
    std::vector<mcl::UpdateDesc> ud;
    for (size_t i = 0; i < n_layers; ++i) {
        const mcl_cuda_update_desc& L = layers[i];
        if (L.rows == 0) continue;
        MCL_TRY(check_counter_dims(ctx, op, C, L.in_features, L.rows));
        if ((L.row_offset + L.rows) * L.in_features > 0xffffffffull)
            return fail(ctx, MCL_CUDA_EINVAL, "counter update: (row_offset + rows) * in_features exceeds 32-bit element indexing");
        MCL_TRY(check_ptr(ctx, op, "state", L.state, 1));
        MCL_TRY(check_ptr(ctx, op, "scale", L.scale, 4));
        MCL_TRY(check_ptr(ctx, op, "v", L.v, 4));
        MCL_TRY(check_ptr(ctx, op, "grad_w", L.grad_w, 16));
        mcl::UpdateDesc u;
        u.state = L.state; u.scale = L.scale; u.v = L.v; u.grad_w = L.grad_w; u.packed2 = L.packed2_out;
        u.in_features = (int)L.in_features; u.rows = (int)L.rows; u.row_offset = (int)L.row_offset;
        ud.push_back(u);
    }
    if (ud.empty()) return MCL_CUDA_OK;
    DeviceGuard guard(ctx->device);
    int launches = 0;
    cudaError_t e = mcl::launch_counter_update_group(ud.data(), (int)ud.size(), (int)C, lr, lr_scale, rms_beta, rms_eps, seed,
                                                     ctx->seed_offset, ctx->err_word, ctx->sm_count, ctx->max_smem, ctx->stream, &launches);
    ctx->launches += launches;
    if (e == cudaErrorNotSupported) {
        for (const mcl::UpdateDesc& u : ud)
            MCL_TRY(mcl_cuda_counter_update_dense(ctx, u.state, u.scale, u.v, u.grad_w, u.packed2, C, (size_t)u.in_features,
                                                  (size_t)u.rows, (size_t)u.row_offset, lr, lr_scale, rms_beta, rms_eps, seed));
        return MCL_CUDA_OK;
    }
    if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    return MCL_CUDA_OK;
}

int mcl_cuda_ternary_linear_products(mcl_cuda_ctx* ctx, const float* x, const float* grad_out,
                                     const uint32_t* packed2, const float* scale, float* y, float* grad_x,
                                     float* grad_w, size_t in_features, size_t out_features, size_t batch) {
    MCL_NEED_CTX(ctx);
    const char* op = "ternary linear products";
    if (in_features == 0 || out_features == 0 || batch == 0)
        return fail(ctx, MCL_CUDA_EINVAL, "ternary linear products requires non-zero dimensions");
    if (in_features % 16 != 0) return fail(ctx, MCL_CUDA_EINVAL, "ternary linear products requires in_features % 16 == 0");
    if (in_features > 0x7fffffffull || out_features > 0x7fffffffull || batch > 0x7fffffffull ||
        in_features * out_features > 0x7fffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, "ternary linear products: dimension exceeds 32-bit indexing");
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "packed2", packed2, 4));
    MCL_TRY(check_ptr(ctx, op, "scale", scale, 4));
    if (grad_x || grad_w) MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    if (grad_w) MCL_TRY(check_ptr(ctx, op, "grad_w", grad_w, 16));
    DeviceGuard guard(ctx->device);
    return linear_products(ctx, op, x, grad_out, nullptr, packed2, scale, y, grad_x, grad_w, 11, in_features,
                           out_features, batch);
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
    if (tc_wanted(ctx, M, N, K)) {
        int pa[6], pb[6], nt, planes;
        grad_term_list(ctx->grad_terms, pa, pb, &nt, &planes);
        const int ldk = up8(K);
        int splits = 1;
        const size_t sk = mcl::tc_splitk_workspace_bytes((int)M, (int)N, (int)K, ctx->sm_count, mcl::kGradDepthLimit, &splits);
        Carver cv;
        const size_t o_a = cv.reserve((size_t)planes * M * ldk * 2), o_b = cv.reserve((size_t)planes * N * ldk * 2),
                     o_k = cv.reserve(sk);
        void* wsp = nullptr;
        MCL_TRY(ws_reserve(ctx, cv.off, &wsp));
        char* w = static_cast<char*>(wsp);
        // A logical [M,K]: stored [M,K] -> planes as is; stored [K,M] (trans_a) -> transposed planes
        if (!trans_a) MCL_LAUNCH(ctx, op, mcl::launch_split_planes(a, (int)M, (int)K, nullptr, w + o_a, ldk, planes, nullptr, 0, 0, ctx->stream));
        else MCL_LAUNCH(ctx, op, mcl::launch_split_planes(a, (int)K, (int)M, nullptr, nullptr, 0, 0, w + o_a, ldk, planes, ctx->stream));
        // B logical [K,N], needed as [N,K]: stored [N,K] (trans_b) -> as is; stored [K,N] -> transposed planes
        if (trans_b) MCL_LAUNCH(ctx, op, mcl::launch_split_planes(b, (int)N, (int)K, nullptr, w + o_b, ldk, planes, nullptr, 0, 0, ctx->stream));
        else MCL_LAUNCH(ctx, op, mcl::launch_split_planes(b, (int)K, (int)N, nullptr, nullptr, 0, 0, w + o_b, ldk, planes, ctx->stream));
        return tc_product(ctx, w + o_a, planes, ldk, M * (size_t)ldk, w + o_b, planes, ldk, N * (size_t)ldk, c, (int)N,
                          (int)M, (int)N, (int)K, pa, pb, nt, nullptr, reinterpret_cast<float*>(w + o_k), splits);
    }
    MCL_LAUNCH(ctx, op, mcl::launch_simt_matmul_f32(a, b, c, (int)M, (int)K, (int)N, trans_a, trans_b, ctx->stream));
    return MCL_CUDA_OK;
}

int mcl_cuda_eltwise_f32(mcl_cuda_ctx* ctx, int op, const float* a, const float* b, float* out, size_t elements,
                         float alpha) {
    MCL_NEED_CTX(ctx);
    const char* name = "eltwise_f32";
    if (op < 0 || op > MCL_CUDA_ELT_SGD) return fail(ctx, MCL_CUDA_EINVAL, "eltwise_f32: unknown op");
    if (elements == 0) return fail(ctx, MCL_CUDA_EINVAL, "eltwise_f32 requires non-zero elements");
    MCL_TRY(check_ptr(ctx, name, "out", out, 4));
    if (op != MCL_CUDA_ELT_ZERO) MCL_TRY(check_ptr(ctx, name, "a", a, 4));
    if (op <= MCL_CUDA_ELT_MUL || op == MCL_CUDA_ELT_SGD) MCL_TRY(check_ptr(ctx, name, "b", b, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, name, mcl::launch_eltwise_f32(op, a, b, out, elements, alpha, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}

// ---- fp32 row ops of the block stack around the counter layers ----------------------------------------
namespace {
int check_rows(mcl_cuda_ctx* ctx, const char* op, size_t rows, size_t cols) {
    if (rows == 0 || cols == 0) return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + " requires non-zero dimensions");
    if (cols > 0x7fffffffull || rows > 0xffffffffull) return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + " dimension is too large");
    return MCL_CUDA_OK;
}
}  // namespace

int mcl_cuda_rmsnorm(mcl_cuda_ctx* ctx, const float* x, const float* weight, float* out, size_t rows, size_t cols,
                     float eps) {
    MCL_NEED_CTX(ctx);
    const char* op = "rmsnorm";
    MCL_TRY(check_rows(ctx, op, rows, cols));
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "weight", weight, 4));
    MCL_TRY(check_ptr(ctx, op, "out", out, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_rmsnorm(x, weight, out, rows, (int)cols, eps, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_rmsnorm_backward_x(mcl_cuda_ctx* ctx, const float* x, const float* weight, const float* grad_out,
                                float* grad_x, size_t rows, size_t cols, float eps) {
    MCL_NEED_CTX(ctx);
    const char* op = "rmsnorm backward_x";
    MCL_TRY(check_rows(ctx, op, rows, cols));
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "weight", weight, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_x", grad_x, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_rmsnorm_backward_x(x, weight, grad_out, grad_x, rows, (int)cols, eps, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_rmsnorm_backward_weight(mcl_cuda_ctx* ctx, const float* x, const float* grad_out, float* row_inv_scratch,
                                     float* grad_weight, size_t rows, size_t cols, float eps) {
    MCL_NEED_CTX(ctx);
    const char* op = "rmsnorm backward_weight";
    MCL_TRY(check_rows(ctx, op, rows, cols));
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "row_inv_scratch", row_inv_scratch, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_weight", grad_weight, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_rmsnorm_backward_weight(x, grad_out, row_inv_scratch, grad_weight, rows, (int)cols, eps, ctx->sm_count, ctx->stream));
    ctx->launches += 1;     // the row pass and the column pass
    return MCL_CUDA_OK;
}
int mcl_cuda_mse_loss_partial(mcl_cuda_ctx* ctx, const float* pred, const float* target, float* partial, size_t n) {
    MCL_NEED_CTX(ctx);
    const char* op = "mse_loss_partial";
    if (n == 0 || n > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "mse_loss_partial needs 0 < n < 2^31");
    MCL_TRY(check_ptr(ctx, op, "pred", pred, 4));
    MCL_TRY(check_ptr(ctx, op, "target", target, 4));
    MCL_TRY(check_ptr(ctx, op, "partial", partial, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_mse_loss_partial(pred, target, partial, n, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_mean_reduce(mcl_cuda_ctx* ctx, const float* partial, float* out, size_t count, size_t denominator) {
    MCL_NEED_CTX(ctx);
    const char* op = "mean_reduce";
    if (count > 0x7fffffffull || denominator > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "mean_reduce counts exceed 2^31");
    MCL_TRY(check_ptr(ctx, op, "partial", partial, 4));
    MCL_TRY(check_ptr(ctx, op, "out", out, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_mean_reduce(partial, out, (int)count, (int)denominator, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_mse_backward(mcl_cuda_ctx* ctx, const float* pred, const float* target, const float* grad_out,
                          float* grad_pred, size_t n) {
    MCL_NEED_CTX(ctx);
    const char* op = "mse_backward";
    if (n == 0 || n > 0x7fffffffull) return fail(ctx, MCL_CUDA_EINVAL, "mse_backward needs 0 < n < 2^31");
    MCL_TRY(check_ptr(ctx, op, "pred", pred, 4));
    MCL_TRY(check_ptr(ctx, op, "target", target, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_pred", grad_pred, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_mse_backward(pred, target, grad_out, grad_pred, n, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_swiglu(mcl_cuda_ctx* ctx, const float* packed, float* out, size_t rows, size_t hidden) {
    MCL_NEED_CTX(ctx);
    const char* op = "swiglu";
    MCL_TRY(check_rows(ctx, op, rows, hidden));
    MCL_TRY(check_ptr(ctx, op, "packed", packed, 4));
    MCL_TRY(check_ptr(ctx, op, "out", out, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_swiglu(packed, out, rows, (int)hidden, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_swiglu_backward(mcl_cuda_ctx* ctx, const float* packed, const float* grad_out, float* grad_packed,
                             size_t rows, size_t hidden) {
    MCL_NEED_CTX(ctx);
    const char* op = "swiglu backward";
    MCL_TRY(check_rows(ctx, op, rows, hidden));
    MCL_TRY(check_ptr(ctx, op, "packed", packed, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_packed", grad_packed, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_swiglu_backward(packed, grad_out, grad_packed, rows, (int)hidden, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_softmax_cross_entropy(mcl_cuda_ctx* ctx, const float* logits, const int32_t* targets, float* partial,
                                   float* out, size_t rows, size_t cols) {
    MCL_NEED_CTX(ctx);
    const char* op = "softmax_cross_entropy";
    MCL_TRY(check_rows(ctx, op, rows, cols));
    MCL_TRY(check_ptr(ctx, op, "logits", logits, 4));
    MCL_TRY(check_ptr(ctx, op, "targets", targets, 4));
    MCL_TRY(check_ptr(ctx, op, "partial", partial, 4));
    MCL_TRY(check_ptr(ctx, op, "out", out, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_softmax_cross_entropy(logits, targets, partial, out, rows, (int)cols, ctx->sm_count, ctx->stream));
    ctx->launches += 1;     // row losses, then their mean
    return MCL_CUDA_OK;
}
int mcl_cuda_softmax_cross_entropy_backward(mcl_cuda_ctx* ctx, const float* logits, const int32_t* targets,
                                            const float* grad_out, float* grad_logits, size_t rows, size_t cols) {
    MCL_NEED_CTX(ctx);
    const char* op = "softmax_cross_entropy backward";
    MCL_TRY(check_rows(ctx, op, rows, cols));
    MCL_TRY(check_ptr(ctx, op, "logits", logits, 4));
    MCL_TRY(check_ptr(ctx, op, "targets", targets, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_logits", grad_logits, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_softmax_cross_entropy_backward(logits, targets, grad_out, grad_logits, rows, (int)cols, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}

namespace {
int check_gqa(mcl_cuda_ctx* ctx, const char* op, size_t batch, size_t tq, size_t tk, size_t key_stride, size_t n_head,
              size_t n_kv, size_t hd, size_t vhd, size_t q_off, size_t window, bool backward) {
    if (batch == 0 || tq == 0 || tk == 0 || n_head == 0 || n_kv == 0 || hd == 0 || vhd == 0)
        return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + " requires non-zero dimensions");
    if (n_head % n_kv != 0) return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + " requires n_head % n_kv_head == 0");
    if (key_stride < tk) return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + " requires key_stride >= key_tokens");
    if (batch * n_head > 65535 || tq > 0x7fffffffull || tk > 0x7fffffffull || q_off > 0x3fffffffull ||
        window > 0x3fffffffull || hd > 65536 || vhd > 65536)
        return fail(ctx, MCL_CUDA_EINVAL, std::string(op) + " dimension is too large");
    (void)backward;
    return MCL_CUDA_OK;
}
}  // namespace

int mcl_cuda_gqa_forward(mcl_cuda_ctx* ctx, const float* q, const float* k, const float* v, float* out, size_t batch,
                         size_t query_tokens, size_t key_tokens, size_t key_stride, size_t n_head, size_t n_kv_head,
                         size_t head_dim, size_t v_head_dim, int causal, size_t query_offset, size_t sliding_window,
                         float scale) {
    MCL_NEED_CTX(ctx);
    const char* op = "grouped_query_attention";
    MCL_TRY(check_gqa(ctx, op, batch, query_tokens, key_tokens, key_stride, n_head, n_kv_head, head_dim, v_head_dim,
                      query_offset, sliding_window, false));
    MCL_TRY(check_ptr(ctx, op, "q", q, 4));
    MCL_TRY(check_ptr(ctx, op, "k", k, 4));
    MCL_TRY(check_ptr(ctx, op, "v", v, 4));
    MCL_TRY(check_ptr(ctx, op, "out", out, 4));
    DeviceGuard guard(ctx->device);
    // scores of every (batch, head, query) row live in the workspace between the two products; the batch is
    // served in slices that keep it under 4 GiB (one batch element at least)
    const size_t per_batch = n_head * query_tokens * key_tokens * sizeof(float);
    size_t slice = ((size_t)4 << 30) / per_batch;
    if (slice < 1) slice = 1;
    if (slice > batch) slice = batch;
    void* ws = nullptr;
    MCL_TRY(ws_reserve(ctx, slice * per_batch, &ws));
    int launches = 0;
    cudaError_t e = cudaSuccess;
    for (size_t b0 = 0; b0 < batch && e == cudaSuccess; b0 += slice) {
        const size_t nb = batch - b0 < slice ? batch - b0 : slice;
        e = mcl::launch_gqa_forward(q + b0 * query_tokens * n_head * head_dim, k + b0 * key_stride * n_kv_head * head_dim,
                                    v + b0 * key_stride * n_kv_head * v_head_dim, out + b0 * query_tokens * n_head * v_head_dim,
                                    (int)nb, (int)query_tokens, (int)key_tokens, (int)key_stride, (int)n_head, (int)n_kv_head,
                                    (int)head_dim, (int)v_head_dim, causal ? 1 : 0, (int)query_offset, (int)sliding_window,
                                    scale, static_cast<float*>(ws), ctx->stream, &launches);
    }
    if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    ctx->launches += launches;
    return MCL_CUDA_OK;
}
int mcl_cuda_gqa_backward(mcl_cuda_ctx* ctx, const float* q, const float* k, const float* v, const float* grad_out,
                          float* probs_scratch, float* ds_scratch, float* grad_q, float* grad_k, float* grad_v,
                          size_t batch, size_t query_tokens, size_t key_tokens, size_t n_head, size_t n_kv_head,
                          size_t head_dim, int causal, size_t query_offset, float scale) {
    MCL_NEED_CTX(ctx);
    const char* op = "grouped_query_attention backward";
    MCL_TRY(check_gqa(ctx, op, batch, query_tokens, key_tokens, key_tokens, n_head, n_kv_head, head_dim, head_dim,
                      query_offset, 0, true));
    MCL_TRY(check_ptr(ctx, op, "q", q, 4));
    MCL_TRY(check_ptr(ctx, op, "k", k, 4));
    MCL_TRY(check_ptr(ctx, op, "v", v, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "probs_scratch", probs_scratch, 4));
    MCL_TRY(check_ptr(ctx, op, "ds_scratch", ds_scratch, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_q", grad_q, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_k", grad_k, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_v", grad_v, 4));
    DeviceGuard guard(ctx->device);
    int launches = 0;
    cudaError_t e = mcl::launch_gqa_backward(q, k, v, grad_out, probs_scratch, ds_scratch, grad_q, grad_k, grad_v,
                                             (int)batch, (int)query_tokens, (int)key_tokens, (int)n_head, (int)n_kv_head,
                                             (int)head_dim, causal ? 1 : 0, (int)query_offset, scale, ctx->stream, &launches);
    if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    ctx->launches += launches;
    return MCL_CUDA_OK;
}

int mcl_cuda_token_position_embedding(mcl_cuda_ctx* ctx, const float* token_weight, const float* pos_weight,
                                      const int32_t* token_ids, float* out, size_t token_count, size_t vocab_size,
                                      size_t seq_len, size_t embed_dim) {
    MCL_NEED_CTX(ctx);
    const char* op = "token_position_embedding";
    if (token_count == 0 || vocab_size == 0 || embed_dim == 0 || (pos_weight && seq_len == 0))
        return fail(ctx, MCL_CUDA_EINVAL, "token_position_embedding requires non-zero shapes");
    if (vocab_size > 0x7fffffffull || embed_dim > 0x7fffffffull || seq_len > 0x7fffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, "token_position_embedding dimension is too large");
    MCL_TRY(check_ptr(ctx, op, "token_weight", token_weight, 4));
    MCL_TRY(check_ptr(ctx, op, "token_ids", token_ids, 4));
    MCL_TRY(check_ptr(ctx, op, "out", out, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_embedding(token_weight, pos_weight, token_ids, out, token_count, (int)vocab_size,
                                              (int)(seq_len ? seq_len : 1), (int)embed_dim, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_embedding_weight_backward(mcl_cuda_ctx* ctx, const int32_t* indices, const float* grad_out, float* grad_weight,
                                       size_t vocab_size, size_t embed_dim, size_t token_count, int zero_first) {
    MCL_NEED_CTX(ctx);
    const char* op = "embedding weight backward";
    if (vocab_size == 0 || embed_dim == 0) return fail(ctx, MCL_CUDA_EINVAL, "embedding weight backward requires non-zero shapes");
    if (vocab_size > 0x7fffffffull || embed_dim > 0x7fffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, "embedding weight backward dimension is too large");
    MCL_TRY(check_ptr(ctx, op, "grad_weight", grad_weight, 4));
    DeviceGuard guard(ctx->device);
    if (zero_first) {
        cudaError_t e = cudaMemsetAsync(grad_weight, 0, vocab_size * embed_dim * sizeof(float), ctx->stream);
        if (e != cudaSuccess) return fail_cuda(ctx, op, e);
    }
    if (token_count == 0) return MCL_CUDA_OK;
    MCL_TRY(check_ptr(ctx, op, "indices", indices, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_LAUNCH(ctx, op, mcl::launch_embedding_scatter(indices, grad_out, grad_weight, token_count, (int)vocab_size, (int)embed_dim,
                                                      ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_position_embedding_backward(mcl_cuda_ctx* ctx, const float* grad_out, float* grad_position, size_t batch,
                                         size_t seq_len, size_t embed_dim) {
    MCL_NEED_CTX(ctx);
    const char* op = "position embedding backward";
    if (batch == 0 || seq_len == 0 || embed_dim == 0 || batch > 0x7fffffffull || seq_len > 0x7fffffffull || embed_dim > 0x7fffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, "position embedding backward requires non-zero shapes below 2^31");
    MCL_TRY(check_ptr(ctx, op, "grad_out", grad_out, 4));
    MCL_TRY(check_ptr(ctx, op, "grad_position", grad_position, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_position_backward(grad_out, grad_position, (int)batch, (int)seq_len, (int)embed_dim,
                                                      ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_rope(mcl_cuda_ctx* ctx, const float* x, float* out, size_t batch, size_t tokens, size_t channels, size_t n_head,
                  size_t head_dim, size_t rotary_dim, size_t token_offset, float theta, int inverse, int split_half) {
    MCL_NEED_CTX(ctx);
    const char* op = "rope";
    if (batch == 0 || tokens == 0 || channels == 0 || n_head == 0 || head_dim == 0)
        return fail(ctx, MCL_CUDA_EINVAL, "rope requires non-zero shapes");
    if (tokens > 0x7fffffffull || channels > 0x7fffffffull || token_offset > 0x3fffffffull || rotary_dim > head_dim)
        return fail(ctx, MCL_CUDA_EINVAL, "rope dimension is out of range");
    if (n_head * head_dim > channels) return fail(ctx, MCL_CUDA_EINVAL, "rope requires n_head * head_dim <= channels");
    MCL_TRY(check_ptr(ctx, op, "x", x, 4));
    MCL_TRY(check_ptr(ctx, op, "out", out, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_rope(x, out, batch * tokens, (int)tokens, (int)channels, (int)n_head, (int)head_dim,
                                         (int)rotary_dim, (int)token_offset, theta, inverse ? 1 : 0, split_half ? 1 : 0,
                                         ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}
int mcl_cuda_adam_update(mcl_cuda_ctx* ctx, float* param, const float* grad, float* m, float* v, size_t elements, float lr,
                         float beta1, float beta2, float eps, float weight_decay, float c1, float c2) {
    MCL_NEED_CTX(ctx);
    const char* op = "adam_update";
    if (elements == 0) return fail(ctx, MCL_CUDA_EINVAL, "adam_update requires non-zero elements");
    MCL_TRY(check_ptr(ctx, op, "param", param, 4));
    MCL_TRY(check_ptr(ctx, op, "grad", grad, 4));
    MCL_TRY(check_ptr(ctx, op, "m", m, 4));
    MCL_TRY(check_ptr(ctx, op, "v", v, 4));
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_adam(param, grad, m, v, elements, lr, beta1, beta2, eps, weight_decay, c1, c2, ctx->sm_count,
                                         ctx->stream));
    return MCL_CUDA_OK;
}

int mcl_cuda_peer_buffer_create(mcl_cuda_ctx* ctx, size_t bytes, void** out_dptr, unsigned char* handle64) {
    MCL_NEED_CTX(ctx);
    MCL_NOT_RECORDING(ctx, "peer_buffer_create");
    if (!out_dptr || !handle64 || bytes == 0) return fail(ctx, MCL_CUDA_EINVAL, "peer_buffer_create: null argument or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == MCL_CUDA_IPC_HANDLE_BYTES, "IPC handle size");
    DeviceGuard guard(ctx->device);
    void* d = nullptr;
    // plain cudaMalloc: memory of the stream-ordered pool cannot be exported to other processes
    cudaError_t e = cudaMalloc(&d, bytes);
    if (e != cudaSuccess) return fail_cuda(ctx, "peer_buffer_create (cudaMalloc)", e);
    e = cudaMemset(d, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
    if (e != cudaSuccess) { cudaFree(d); return fail_cuda(ctx, "peer_buffer_create (export)", e); }
    std::memcpy(handle64, &h, sizeof(h));
    *out_dptr = d;
    return MCL_CUDA_OK;
}
int mcl_cuda_peer_buffer_open(mcl_cuda_ctx* ctx, const unsigned char* handle64, void** out_dptr) {
    MCL_NEED_CTX(ctx);
    MCL_NOT_RECORDING(ctx, "peer_buffer_open");
    if (!out_dptr || !handle64) return fail(ctx, MCL_CUDA_EINVAL, "peer_buffer_open: null argument");
    DeviceGuard guard(ctx->device);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    void* d = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail_cuda(ctx, "peer_buffer_open", e);
    *out_dptr = d;
    return MCL_CUDA_OK;
}
int mcl_cuda_peer_buffer_close(mcl_cuda_ctx* ctx, void* dptr) {
    MCL_NEED_CTX(ctx);
    if (!dptr) return MCL_CUDA_OK;
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaIpcCloseMemHandle(dptr);
    if (e != cudaSuccess) return fail_cuda(ctx, "peer_buffer_close", e);
    return MCL_CUDA_OK;
}
int mcl_cuda_peer_buffer_destroy(mcl_cuda_ctx* ctx, void* dptr) {
    MCL_NEED_CTX(ctx);
    if (!dptr) return MCL_CUDA_OK;
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaFree(dptr);
    if (e != cudaSuccess) return fail_cuda(ctx, "peer_buffer_destroy", e);
    return MCL_CUDA_OK;
}
int mcl_cuda_peer_allreduce_f32(mcl_cuda_ctx* ctx, const void* const* peer_data, void* const* peer_flags, int rank,
                                int world, size_t n, size_t parity_stride, int parity, float* out) {
    MCL_NEED_CTX(ctx);
    const char* op = "peer allreduce";
    if (world < 1 || world > mcl::kPeerMaxWorld || rank < 0 || rank >= world)
        return fail(ctx, MCL_CUDA_EINVAL, "peer allreduce serves 1 to 8 ranks of one node");
    if (parity != 0 && parity != 1) return fail(ctx, MCL_CUDA_EINVAL, "peer allreduce: parity is 0 or 1");
    if (n == 0 || n % 4 != 0 || parity_stride % 4 != 0 || n > parity_stride || n > 0x7fffffffull)
        return fail(ctx, MCL_CUDA_EINVAL, "peer allreduce needs n and parity_stride in multiples of 4 floats, n <= parity_stride");
    if (!peer_data || !peer_flags) return fail(ctx, MCL_CUDA_EINVAL, "peer allreduce: null pointer tables");
    MCL_TRY(check_ptr(ctx, op, "out", out, 16));
    mcl::PeerTable tab{};
    for (int r = 0; r < world; ++r) {
        if (!peer_data[r] || !peer_flags[r] || reinterpret_cast<uintptr_t>(peer_data[r]) % 16 != 0 ||
            reinterpret_cast<uintptr_t>(peer_flags[r]) % 4 != 0)
            return fail(ctx, MCL_CUDA_EINVAL, "peer allreduce: every rank's data must be 16-byte and its flags 4-byte aligned");
        tab.data[r] = static_cast<const float*>(peer_data[r]);
        tab.flags[r] = static_cast<uint32_t*>(peer_flags[r]);
    }
    tab.parity_stride4 = parity_stride / 4;
    tab.rank = rank; tab.world = world;
    DeviceGuard guard(ctx->device);
    MCL_LAUNCH(ctx, op, mcl::launch_peer_allreduce(tab, n, parity, out, ctx->err_word, ctx->stream));
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
    if (ctx->gemm_mode != MCL_CUDA_GEMM_EXACT && M == 1 &&
        mcl::gemv_lut_supported((int)M, (int)in_features, (int)out_features, packed2, kGemvTicketWords)) {
        // one activation row: one launch that looks pairs of weights up in a table of activation sums
        void* wsp = nullptr;
        const size_t need = mcl::gemv_lut_workspace_bytes((int)in_features, (int)out_features);
        if (need) MCL_TRY(ws_reserve(ctx, need, &wsp));
        MCL_LAUNCH(ctx, op, mcl::launch_ternary_gemv_lut(x, packed2, scale, y, (int)in_features, (int)out_features,
                                                         static_cast<float*>(wsp),
                                                         reinterpret_cast<unsigned int*>(ctx->err_word + 16), ctx->sm_count,
                                                         ctx->max_smem, ctx->stream));
        return MCL_CUDA_OK;
    }
    if (ctx->gemm_mode != MCL_CUDA_GEMM_EXACT && M == 1) {
        // a single activation row whose shape the table kernels do not take: streaming the words through the CUDA
        // cores in one launch still beats the three launches of the tensor-core route
        MCL_LAUNCH(ctx, op, mcl::launch_ternary_gemv_stream(x, packed2, scale, y, (int)M, (int)in_features, (int)out_features,
                                                            ctx->sm_count, ctx->stream));
        return MCL_CUDA_OK;
    }
    if (ctx->gemm_mode != MCL_CUDA_GEMM_EXACT && out_features >= 128 &&
        mcl::gemv_tc_supported((int)M, (int)in_features, (int)out_features) &&
        reinterpret_cast<uintptr_t>(packed2) % 16 == 0) {
        void* wsp = nullptr;
        MCL_TRY(ws_reserve(ctx, mcl::gemv_tc_workspace_bytes((int)M, (int)in_features, (int)out_features), &wsp));
        int launches = 0;
        cudaError_t e = mcl::launch_ternary_gemv_tc(x, packed2, scale, y, (int)M, (int)in_features, (int)out_features,
                                                    wsp, ctx->err_word, ctx->sm_count, ctx->max_smem, ctx->stream,
                                                    &launches);
        ctx->launches += launches;
        if (e != cudaSuccess) return fail_cuda(ctx, op, e);
        return MCL_CUDA_OK;
    }
    MCL_LAUNCH(ctx, op, mcl::launch_ternary_gemv(x, packed2, scale, y, (int)M, (int)in_features,
                                                 (int)out_features, ctx->sm_count, ctx->stream));
    return MCL_CUDA_OK;
}

}  // extern "C"
