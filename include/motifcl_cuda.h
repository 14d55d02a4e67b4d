/* motifcl_cuda.h -- C ABI of the B200 (sm_100a) counter-synapse linear path.
 *
 * This is the boundary a MotifCL maintainer binds to: plain pointers and sizes, no C++ or
 * framework types.  Each entry point names the MotifCL interface it replaces (paths are
 * relative to the MotifCL source tree).  All data pointers are DEVICE pointers on the
 * context's device unless a parameter is called *_host.  Tensors are dense row-major.
 *
 * Conventions
 *   - Every function returns 0 on success or an MCL_CUDA_E* code; the human-readable reason
 *     is kept per context (or per thread when no context exists yet) and read with
 *     mcl_cuda_last_error().  Nothing throws, aborts, exits or traps.
 *   - Work is enqueued on the context's stream in call order and the call returns without
 *     waiting, like the reference's in-order queue; mcl_cuda_finish() and
 *     mcl_cuda_download() wait.  A context is used from one host thread at a time.
 *   - Counter-state layout: uint8 [out, in/4, 3], four 6-bit codes per 3 bytes
 *     (kernels/compact_counter.cl:2-3,25-36).  scale, v: float [out].
 *   - Argument checks mirror the reference's wrappers
 *     (src/runtime/vulkan_backend.cpp:8497-8521,8615-8648,8676-8710,8741-8784): zero sizes,
 *     in % 4 != 0, C == 0 or 3*(2C-1) > 64, non-finite lr / lr_scale / rms_beta, negative or
 *     non-finite rms_eps, out*in beyond 32-bit element indexing are all refused.
 *   - Float inputs must be finite; the update is defined for |counter + tick| < 2^31.
 */
#ifndef MOTIFCL_CUDA_H
#define MOTIFCL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCL_CUDA_OK 0
#define MCL_CUDA_EINVAL 1      /* refused argument (message says which) */
#define MCL_CUDA_ECUDA 2       /* a CUDA runtime call failed */
#define MCL_CUDA_EUNSUPPORTED 3 /* valid request this build cannot serve (message says why) */
#define MCL_CUDA_ENOMEM 4
#define MCL_CUDA_ENODEVICE 5

typedef struct mcl_cuda_ctx mcl_cuda_ctx;

/* ---- context / buffers: replaces VulkanRuntime::create, device_name, finish and
 * VulkanRuntime::create_buffer / VulkanBuffer::upload / download
 * (include/motifcl/runtime/vulkan_backend.hpp:156-243, 80-154). ---- */
int mcl_cuda_device_count(void);   /* 0 when no usable CUDA device: callers skip like probe_vulkan_runtime() */
int mcl_cuda_create(int device, mcl_cuda_ctx** out_ctx);
/* Same, but enqueue on a stream the caller owns (a cudaStream_t passed as void*). */
int mcl_cuda_create_on_stream(int device, void* cuda_stream, mcl_cuda_ctx** out_ctx);
void mcl_cuda_destroy(mcl_cuda_ctx* ctx);
const char* mcl_cuda_last_error(mcl_cuda_ctx* ctx);   /* ctx may be NULL */
const char* mcl_cuda_device_name(mcl_cuda_ctx* ctx);
int mcl_cuda_sm_count(mcl_cuda_ctx* ctx);
size_t mcl_cuda_device_memory_bytes(mcl_cuda_ctx* ctx);   /* total device memory: what an OpenCL seam reports as CL_DEVICE_GLOBAL_MEM_SIZE */
int mcl_cuda_finish(mcl_cuda_ctx* ctx);
int mcl_cuda_alloc(mcl_cuda_ctx* ctx, size_t bytes, void** out_dptr);
int mcl_cuda_free(mcl_cuda_ctx* ctx, void* dptr);
int mcl_cuda_upload(mcl_cuda_ctx* ctx, void* dst, const void* src_host, size_t bytes);
int mcl_cuda_download(mcl_cuda_ctx* ctx, void* dst_host, const void* src, size_t bytes);
/* Number of kernels this library has launched on the context so far. */
uint64_t mcl_cuda_launch_count(mcl_cuda_ctx* ctx);
/* Bytes of device memory the context's internal workspace holds (grow-only scratch of the entry points: the row tile
 * of grad_w of the fused update, operand planes, split-K partial sums).  It is how a caller checks the memory-native
 * property MotifCL gates on (tests/test_memory_truth_gate.cpp:30-126: the fused update may allocate less than a
 * quarter of a dense fp32 weight). */
size_t mcl_cuda_workspace_bytes(mcl_cuda_ctx* ctx);

/* ---- batch recording: replaces VulkanRuntime::batch_begin / batch_end, which wrap a training
 * step into one command-buffer submit (include/motifcl/runtime/vulkan_backend.hpp:174-178;
 * tools/train_ternary15m.cpp:371,381).  Between begin and end, calls on the context are
 * recorded instead of run (CUDA stream capture); batch_end returns a replayable batch that
 * mcl_cuda_batch_launch enqueues as ONE graph launch.  The recorded calls must already have run
 * once unrecorded with the same shapes, so that the context's workspace has its final size;
 * finish, download, upload, alloc and free are refused while recording.
 * A batch holds addresses inside the context's workspace: while any batch of a context is alive,
 * a call that would make the workspace grow is refused (MCL_CUDA_ERR_ARG, "workspace would grow")
 * instead of freeing memory the batch still points into; destroy the batches first, or run the
 * larger call once before recording.
 * Recording captures the calling thread's work on the context's stream only.  Do not enqueue
 * work of other libraries that hands off to streams of their own (an NCCL collective through a
 * framework's process group, for one) between begin and end: such work is not part of the batch
 * and its hand-off events are illegal inside a capture.  Put it between two batches instead. ---- */
typedef struct mcl_cuda_batch mcl_cuda_batch;
/* Optional device word whose value is added to the seed of every counter update enqueued
 * afterwards (NULL = none).  A recorded batch bakes its scalar arguments in; bumping this word
 * between replays gives each step its own seed, as CounterStateLinear::next_seed() does
 * (include/motifcl/nn/compact_counter.hpp:34). */
int mcl_cuda_set_seed_offset(mcl_cuda_ctx* ctx, const uint32_t* device_word);
int mcl_cuda_batch_begin(mcl_cuda_ctx* ctx);
int mcl_cuda_batch_end(mcl_cuda_ctx* ctx, mcl_cuda_batch** out_batch);
int mcl_cuda_batch_launch(mcl_cuda_ctx* ctx, mcl_cuda_batch* batch);
/* Lanes (no reference counterpart: the reference has one queue).  Independent linears can run
 * side by side on further contexts of the same device, each with its own stream and workspace.
 * fork makes everything enqueued on `lane` from now on wait for what `ctx` has enqueued so
 * far; join makes `ctx` wait for what `lane` has enqueued.  Inside a recording on `ctx`, fork
 * pulls the lane's stream into the recording (its calls become parallel branches of the
 * batch) and join must follow before batch_end. */
int mcl_cuda_lane_fork(mcl_cuda_ctx* ctx, mcl_cuda_ctx* lane);
int mcl_cuda_lane_join(mcl_cuda_ctx* ctx, mcl_cuda_ctx* lane);
void mcl_cuda_batch_destroy(mcl_cuda_batch* batch);

/* ---- one-shot sum over the GPUs of a node (no reference counterpart: the reference has no multi-device code).
 * For the [M, out] partial results of a row-sharded decode GEMV.  Every rank holds, in memory that all ranks have
 * mapped, a flag area of 64 uint32 words (zero before the first call; words 0..world-1 are written by the peers, word
 * 32 counts this rank's calls) and two partial buffers `parity_stride` floats apart; peer_data[r] / peer_flags[r]
 * are THIS process's addresses of rank r's buffers and flags.  A call sums the n floats that every rank has written
 * into its buffer `parity` (0 or 1; alternate it from call to call) by earlier work of its stream, in rank order
 * (every rank gets the same bits), into `out`.  All ranks make the same sequence of calls; the call number lives in
 * device memory, so a recorded batch that contains such calls can be replayed.  Ranks meet through the flag words:
 * plain peer stores and loads, a wait of at most 2 s, after which the call's results are invalid and the next
 * mcl_cuda_finish reports it. ---- */
int mcl_cuda_peer_allreduce_f32(mcl_cuda_ctx* ctx, const void* const* peer_data, void* const* peer_flags, int rank,
                                int world, size_t n, size_t parity_stride, int parity, float* out);
/* Memory that the other ranks of the node can map (CUDA IPC; one process per GPU): create makes a zero-filled buffer
 * and the 64-byte handle to send to the peers (by any host channel), open maps a peer's buffer into this process (peer
 * access is enabled on first use), close unmaps it, destroy frees the own buffer.  The owner must outlive the mappings:
 * peers close before the owner destroys (a barrier between the two on the host). */
#define MCL_CUDA_IPC_HANDLE_BYTES 64
int mcl_cuda_peer_buffer_create(mcl_cuda_ctx* ctx, size_t bytes, void** out_dptr, unsigned char* handle64);
int mcl_cuda_peer_buffer_open(mcl_cuda_ctx* ctx, const unsigned char* handle64, void** out_dptr);
int mcl_cuda_peer_buffer_close(mcl_cuda_ctx* ctx, void* dptr);
int mcl_cuda_peer_buffer_destroy(mcl_cuda_ctx* ctx, void* dptr);

/* ---- decode: replaces run_vulkan_compact_counter_decode_weight
 * (include/motifcl/runtime/vulkan_backend.hpp:713-719; kernels/compact_counter.cl:39-55).
 * weight[out,in] = scale[row] * t. ---- */
int mcl_cuda_counter_decode_weight(mcl_cuda_ctx* ctx, const uint8_t* state, const float* scale,
                                   float* weight, size_t in_features, size_t out_features, size_t C);

/* ---- 2-bit pack (no reference counterpart in code; layout of
 * docs/BITNET_TERNARY_VULKAN_PLAN.md:97): packed2 uint32 [out, in/16], weight m of a row in
 * bits [2(m%16)+1 : 2(m%16)] of word m/16, field = t + 1.  Requires in % 16 == 0. ---- */
int mcl_cuda_counter_pack2(mcl_cuda_ctx* ctx, const uint8_t* state, uint32_t* packed2,
                           size_t in_features, size_t out_features, size_t C);

/* ---- forward: replaces run_vulkan_compact_counter_forward_u8
 * (vulkan_backend.hpp:722-730; kernels/vulkan/counter_forward_f32_rb4.comp; OpenCL path
 * src/nn/compact_counter.cpp:287-293).  y[batch,out] = x[batch,in] * (scale . t)^T. ---- */
int mcl_cuda_counter_forward(mcl_cuda_ctx* ctx, const float* x, const uint8_t* state,
                             const float* scale, float* y, size_t batch, size_t in_features,
                             size_t out_features, size_t C);

/* ---- backward to input: replaces run_vulkan_compact_counter_backward_input_u8
 * (vulkan_backend.hpp:752-760; kernels/compact_counter.cl:248-269).
 * grad_x[batch,in] = (grad_out . scale) * t. ---- */
int mcl_cuda_counter_backward_input(mcl_cuda_ctx* ctx, const uint8_t* state, const float* scale,
                                    const float* grad_out, float* grad_x, size_t batch,
                                    size_t in_features, size_t out_features, size_t C);

/* ---- dense fused update: replaces CounterStateLinear::apply_update_seed, i.e. the three
 * launches counter_row_stats_f32 + counter_apply_update_f32 + copy_f32
 * (src/nn/compact_counter.cpp:113-156; kernels/compact_counter.cl:59-139).
 * One kernel: reads state and grad_w[rows,in] once; writes state, scale, v in place and, when
 * packed2_out != NULL (needs in % 16 == 0), the 2-bit weights of the NEW state.
 * `rows` rows are updated; they are rows [row_offset, row_offset+rows) of the full matrix for
 * the purpose of the per-element random stream, so a row shard updates exactly like the same
 * rows of the whole layer.  All pointers address the shard's first row. ---- */
int mcl_cuda_counter_update_dense(mcl_cuda_ctx* ctx, uint8_t* state, float* scale, float* v,
                                  const float* grad_w, uint32_t* packed2_out, size_t C,
                                  size_t in_features, size_t rows, size_t row_offset, float lr,
                                  float lr_scale, float rms_beta, float rms_eps, uint32_t seed);

/* ---- memory-native fused update: replaces run_vulkan_compact_counter_apply_update_fused
 * (vulkan_backend.hpp:731-751; src/nn/compact_counter.cpp:158-231).  grad_w = grad_out^T x is
 * formed in row tiles inside a bounded workspace of the context -- never as a whole
 * [out,in] tensor -- and each tile is consumed by the dense update above.  The two scratch
 * pointers exist for signature parity with the reference and may be NULL (unused).
 * packed2_out may be NULL. ---- */
int mcl_cuda_counter_update_fused(mcl_cuda_ctx* ctx, uint8_t* state, float* scale, float* v,
                                  const float* grad_out, const float* x, float* scale_new_scratch,
                                  float* denom_scratch, uint32_t* packed2_out, size_t C,
                                  size_t in_features, size_t out_features, size_t batch, float lr,
                                  float lr_scale, float rms_beta, float rms_eps, uint32_t seed);

/* ---- how the three contractions are computed (no reference counterpart: the reference has one
 * fp32 path).  mode MCL_CUDA_GEMM_AUTO: tensor cores (tcgen05, bf16 term splitting) for shapes
 * that are large and aligned enough, the exact CUDA-core kernels otherwise;
 * MCL_CUDA_GEMM_EXACT: always the CUDA-core kernels, whose every output equals the reference's
 * k-ascending fp32 sum bit for bit; MCL_CUDA_GEMM_TENSOR: tensor cores whenever the shape
 * allows.  act_terms (2 or 3) = bf16 terms per fp32 activation in Y and dX; grad_terms (3 or 6)
 * = term products in dW = dY^T X.  Defaults: AUTO, 3, 6 (error of every product below 1e-5
 * relative L2 against the fp32 reference sum; 2 / 3 also meet that bound and cost 7/12 of the
 * tensor-core time). ---- */
#define MCL_CUDA_GEMM_AUTO 0
#define MCL_CUDA_GEMM_EXACT 1
#define MCL_CUDA_GEMM_TENSOR 2
int mcl_cuda_set_gemm_mode(mcl_cuda_ctx* ctx, int mode, int act_terms, int grad_terms);

/* ---- the steps of SEVERAL counter linears in one call (the reference records the dispatches of
 * a step into one command buffer, include/motifcl/runtime/vulkan_backend.hpp:138 VulkanDispatchRecording; this is
 * that recording stated as data).  Layer i does exactly what mcl_cuda_counter_linear_step does with
 * the same arguments; layers whose shapes allow it (in and out features multiples of 32 up to 1024,
 * 16-byte aligned tensors) share grouped launches: one expansion of the ternary digits, the
 * products of all layers as one table of tensor-core work items, one split-K reduction, one
 * update.  Layers are independent: no tensor of one may alias a tensor of another. ---- */
typedef struct mcl_cuda_linear_desc {
    const float* x;          /* [batch, in] */
    const float* grad_out;   /* [batch, out] */
    uint8_t* state;          /* [out, in/4*3], updated */
    float* scale;            /* [out], updated */
    float* v;                /* [out], updated */
    float* y;                /* [batch, out] or NULL */
    float* grad_x;           /* [batch, in] or NULL */
    float* grad_w;           /* [out, in], or NULL to skip the weight gradient (then update_rows must be 0): a
                                data-parallel rank forms the weight gradients in one call, starts their
                                reduce-scatter, and forms y / grad_x in a second call that runs under it */
    uint32_t* packed2_out;   /* [out, in/16] or NULL */
    size_t in_features, out_features, batch;
    size_t update_rows, row_offset;   /* as in mcl_cuda_counter_linear_step */
    const uint32_t* packed2_in;  /* used when state is NULL: the layer's 2-bit words; the products come from them as
                                    in mcl_cuda_ternary_linear_products and nothing is updated (update_rows must be 0,
                                    scale is read only, v is ignored) */
} mcl_cuda_linear_desc;
int mcl_cuda_counter_linear_step_many(mcl_cuda_ctx* ctx, const mcl_cuda_linear_desc* layers, size_t n_layers,
                                      size_t C, float lr, float lr_scale, float rms_beta, float rms_eps,
                                      uint32_t seed);

/* ---- the fused updates of several layers (or row shards of layers) in one launch: layer i is exactly
 * mcl_cuda_counter_update_dense with the same arguments.  A data-parallel rank calls this on its
 * shards after the reduce-scatter of the gradients. ---- */
typedef struct mcl_cuda_update_desc {
    uint8_t* state;          /* first updated row */
    float* scale;
    float* v;
    const float* grad_w;     /* [rows, in] */
    uint32_t* packed2_out;   /* [rows, in/16] or NULL */
    size_t in_features, rows, row_offset;
} mcl_cuda_update_desc;
int mcl_cuda_counter_update_dense_many(mcl_cuda_ctx* ctx, const mcl_cuda_update_desc* layers, size_t n_layers,
                                       size_t C, float lr, float lr_scale, float rms_beta, float rms_eps,
                                       uint32_t seed);

/* ---- one whole training step of one counter linear (what MotifCL's autograd does around
 * CounterStateLinear, src/nn/compact_counter.cpp:40-50,266-300, with the dense update of
 * :113-156): y = x W^T; grad_x = (grad_out . scale) T from the PRE-update state; grad_w =
 * grad_out^T x; then the fused update of `rows` rows starting at `row_offset` (pass rows =
 * out_features, row_offset = 0 for the whole layer).  Shares the operand splits between the
 * three products.  y, grad_x and packed2_out may be NULL to skip that output; grad_w holds
 * out*in floats (NULL skips it and needs update_rows == 0).  With update_rows == 0 the update is skipped (the caller reduces grad_w
 * across ranks first and then calls mcl_cuda_counter_update_dense on its shard). ---- */
int mcl_cuda_counter_linear_step(mcl_cuda_ctx* ctx, const float* x, const float* grad_out,
                                 uint8_t* state, float* scale, float* v, float* y, float* grad_x,
                                 float* grad_w, uint32_t* packed2_out, size_t C, size_t in_features,
                                 size_t out_features, size_t batch, size_t update_rows,
                                 size_t row_offset, float lr, float lr_scale, float rms_beta,
                                 float rms_eps, uint32_t seed);

/* ---- the three products of one linear from the 2-bit packed weights (no reference counterpart;
 * same arithmetic as the forward / backward-to-input / weight-gradient entries above with the
 * ternary digit read from packed2).  This is what a data-parallel rank runs for layers whose
 * counter state lives on other ranks: y, grad_x, grad_w (any may be NULL), no update. ---- */
int mcl_cuda_ternary_linear_products(mcl_cuda_ctx* ctx, const float* x, const float* grad_out,
                                     const uint32_t* packed2, const float* scale, float* y, float* grad_x,
                                     float* grad_w, size_t in_features, size_t out_features, size_t batch);

/* ---- generic fp32 matmul: replaces matmul / matmul_transpose_a / matmul_transpose_b
 * (src/ops/matmul.cpp:1131-1233; kernels/matmul.cl:55-129,413-563).
 * c[M,N] = op(a) op(b); trans_a: a stored [K,M]; trans_b: b stored [N,K]. ---- */
int mcl_cuda_matmul_f32(mcl_cuda_ctx* ctx, const float* a, const float* b, float* c, size_t M,
                        size_t K, size_t N, int trans_a, int trans_b);

/* ---- elementwise fp32 helpers: replace run_vulkan_add / _sub / _mul / _mul_scalar / _add_scalar /
 * _zero_f32 (include/motifcl/runtime/vulkan_backend.hpp; src/ops/basic_ops.cpp:67-92,208-211,409,462;
 * kernels/basic.cl), which MotifCL's autograd and its counter tests call between counter layers.
 * out[i] = a[i] (+,-,*) b[i], a[i]*alpha, a[i]+alpha, or 0.  b may be NULL for the scalar ops. ---- */
#define MCL_CUDA_ELT_ADD 0
#define MCL_CUDA_ELT_SUB 1
#define MCL_CUDA_ELT_MUL 2
#define MCL_CUDA_ELT_MUL_SCALAR 3
#define MCL_CUDA_ELT_ADD_SCALAR 4
#define MCL_CUDA_ELT_ZERO 5
#define MCL_CUDA_ELT_SGD 6   /* out = a - alpha*b: run_vulkan_sgd_update (src/ops/optim.cpp:16-29) */
int mcl_cuda_eltwise_f32(mcl_cuda_ctx* ctx, int op, const float* a, const float* b, float* out, size_t elements,
                         float alpha);

/* ---- fp32 row ops of the ternary15m block stack around its counter layers (tests/bench_ternary15m.cpp:145-190).
 * Each replaces the run_vulkan_* free function of the same name in include/motifcl/runtime/vulkan_backend.hpp
 * (:606 rmsnorm, :557 rmsnorm_backward_x, :567 rmsnorm_backward_weight, :613 swiglu, :575 swiglu_backward,
 * :583 softmax_cross_entropy, :590 softmax_cross_entropy_backward, :294 grouped_query_attention_general,
 * :345 grouped_query_attention_backward); callers: src/ops/norm.cpp:74-84,163-175,242-258,
 * src/ops/activation.cpp:314,343, src/ops/loss.cpp:98-160, src/ops/attention.cpp:302-365,2248-2290.
 * Same results as the reference's shaders up to fp32 summation order.
 *   rmsnorm                 out = x * rsqrt(mean(x^2) + eps) * weight              x, out [rows, cols]
 *   rmsnorm_backward_weight row_inv_scratch [rows] receives the inverse RMS; grad_weight [cols] is overwritten
 *   swiglu                  packed [rows, 2*hidden] = gate | up; out = gate * sigmoid(gate) * up
 *   softmax_cross_entropy   partial [rows] = per-row loss (0 for a target outside [0, cols)); out[0] = mean
 *   ..._backward            grad_logits = grad_out[0] / rows * (softmax - onehot)
 *   gqa_forward             q [B*Tq, n_head*hd], k [B*key_stride, n_kv*hd], v [B*key_stride, n_kv*vhd],
 *                           out [B*Tq, n_head*vhd]; causal with query_offset, optional sliding window (0 = none);
 *                           f32 keys/values, no mask
 *   gqa_backward            probs_scratch, ds_scratch [B*n_head*Tq*Tk]; grad_q/k/v shaped like q/k/v ---- */
int mcl_cuda_rmsnorm(mcl_cuda_ctx* ctx, const float* x, const float* weight, float* out, size_t rows, size_t cols,
                     float eps);
int mcl_cuda_rmsnorm_backward_x(mcl_cuda_ctx* ctx, const float* x, const float* weight, const float* grad_out,
                                float* grad_x, size_t rows, size_t cols, float eps);
int mcl_cuda_rmsnorm_backward_weight(mcl_cuda_ctx* ctx, const float* x, const float* grad_out, float* row_inv_scratch,
                                     float* grad_weight, size_t rows, size_t cols, float eps);
int mcl_cuda_swiglu(mcl_cuda_ctx* ctx, const float* packed, float* out, size_t rows, size_t hidden);
/* Mean squared error as MotifCL's OpenCL backend computes it: replaces the kernels mse_loss_partial_f32,
 * mean_reduce_f32 and mse_backward_f32 (kernels/loss.cl:1-43) behind mse_loss / mse_backward_op
 * (src/ops/loss.cpp:21-95).  partial holds ceil(n / 256) floats: the sum of squared differences of each chunk of 256
 * elements, added left to right; mean_reduce adds `count` partial sums (256 strided lanes, then a 128..1 tree) and
 * divides by `denominator` (0 gives 0); mse_backward writes grad_out[0] * 2 * (pred - target) / n.  The orders of
 * summation are the reference's, so the loss is the same float. */
int mcl_cuda_mse_loss_partial(mcl_cuda_ctx* ctx, const float* pred, const float* target, float* partial, size_t n);
int mcl_cuda_mean_reduce(mcl_cuda_ctx* ctx, const float* partial, float* out, size_t count, size_t denominator);
int mcl_cuda_mse_backward(mcl_cuda_ctx* ctx, const float* pred, const float* target, const float* grad_out,
                          float* grad_pred, size_t n);
int mcl_cuda_swiglu_backward(mcl_cuda_ctx* ctx, const float* packed, const float* grad_out, float* grad_packed,
                             size_t rows, size_t hidden);
int mcl_cuda_softmax_cross_entropy(mcl_cuda_ctx* ctx, const float* logits, const int32_t* targets, float* partial,
                                   float* out, size_t rows, size_t cols);
int mcl_cuda_softmax_cross_entropy_backward(mcl_cuda_ctx* ctx, const float* logits, const int32_t* targets,
                                            const float* grad_out, float* grad_logits, size_t rows, size_t cols);
int mcl_cuda_gqa_forward(mcl_cuda_ctx* ctx, const float* q, const float* k, const float* v, float* out, size_t batch,
                         size_t query_tokens, size_t key_tokens, size_t key_stride, size_t n_head, size_t n_kv_head,
                         size_t head_dim, size_t v_head_dim, int causal, size_t query_offset, size_t sliding_window,
                         float scale);
int mcl_cuda_gqa_backward(mcl_cuda_ctx* ctx, const float* q, const float* k, const float* v, const float* grad_out,
                          float* probs_scratch, float* ds_scratch, float* grad_q, float* grad_k, float* grad_v,
                          size_t batch, size_t query_tokens, size_t key_tokens, size_t n_head, size_t n_kv_head,
                          size_t head_dim, int causal, size_t query_offset, float scale);

/* ---- the remaining fp32 ops of the ternary15m trainer step (tools/train_ternary15m.cpp:273-293,377): they replace
 * run_vulkan_token_position_embedding (:821), run_vulkan_embedding_gather (:776), run_vulkan_embedding_weight_backward
 * and its _scatter / _scatter_cas variants (:784-819), run_vulkan_position_embedding_backward (:832), run_vulkan_rope /
 * run_vulkan_rope_split_half (:842,:865) and run_vulkan_adam_update_fast (:704) of
 * include/motifcl/runtime/vulkan_backend.hpp; callers: src/nn/embedding.cpp:18-120,268-300, src/ops/attention.cpp:838-906,
 * src/ops/optim.cpp:47-65.
 *   token_position_embedding  out[t,:] = token_weight[ids[t],:] (0 for an id outside [0,vocab)) + pos_weight[t % seq_len,:];
 *                             pos_weight NULL = plain gather
 *   embedding_weight_backward grad_weight[ids[t],:] += grad_out[t,:]; zero_first != 0 clears grad_weight [vocab,dim] first
 *                             (the reference's scatter variants expect the caller to have cleared it)
 *   position_embedding_backward grad_position[p,:] = sum_b grad_out[b*seq_len+p,:]  (rows p < seq_len only)
 *   rope                      x, out [batch*tokens, channels]; heads of head_dim at the front of each row; rotary_dim 0 =
 *                             head_dim; split_half pairs (i, i+head_dim/2), else (2i, 2i+1); inverse negates the angle
 *   adam_update               m,v,param updated in place; c1, c2 = 1/(1-beta^step) ---- */
int mcl_cuda_token_position_embedding(mcl_cuda_ctx* ctx, const float* token_weight, const float* pos_weight,
                                      const int32_t* token_ids, float* out, size_t token_count, size_t vocab_size,
                                      size_t seq_len, size_t embed_dim);
int mcl_cuda_embedding_weight_backward(mcl_cuda_ctx* ctx, const int32_t* indices, const float* grad_out, float* grad_weight,
                                       size_t vocab_size, size_t embed_dim, size_t token_count, int zero_first);
int mcl_cuda_position_embedding_backward(mcl_cuda_ctx* ctx, const float* grad_out, float* grad_position, size_t batch,
                                         size_t seq_len, size_t embed_dim);
int mcl_cuda_rope(mcl_cuda_ctx* ctx, const float* x, float* out, size_t batch, size_t tokens, size_t channels, size_t n_head,
                  size_t head_dim, size_t rotary_dim, size_t token_offset, float theta, int inverse, int split_half);
int mcl_cuda_adam_update(mcl_cuda_ctx* ctx, float* param, const float* grad, float* m, float* v, size_t elements, float lr,
                         float beta1, float beta2, float eps, float weight_decay, float c1, float c2);

/* ---- ternary decode GEMV, M <= 16 (no reference kernel; semantics of the forward above
 * applied to 2-bit weights).  y[M,out] = x[M,in] * (scale . t)^T.  Requires in % 16 == 0. ---- */
int mcl_cuda_ternary_gemv(mcl_cuda_ctx* ctx, const float* x, const uint32_t* packed2,
                          const float* scale, float* y, size_t M, size_t in_features,
                          size_t out_features);

/* ---- memory-native fused update that allocates nothing (it has no counterpart in the
 * reference).  For callers that may not call cudaMalloc / cudaFree while they run: a host that
 * gave all device memory to its own arena at start-up, a plugin inside a latency-critical loop
 * where an allocation would stall the device, or code that owns only a stream and its buffers
 * and no library context.  Same arithmetic and results as mcl_cuda_counter_update_fused in
 * MCL_CUDA_GEMM_EXACT mode, but the grad_w row tile lives in a 4 MiB array built into the
 * library (every GPU that loads the library holds it until the process exits) instead of a
 * workspace grown on demand.  No context: work is enqueued on `cuda_stream` of the CURRENT
 * device.  Limits and rules:
 *   - in_features <= mcl_cuda_static_scratch_floats() (1,048,576): one gradient row must fit;
 *     larger shapes are refused with a message (mcl_cuda_static_last_error()).
 *   - all calls on a device share the array: calls that overlap on the GPU race; keep them on
 *     one stream.  The array is not cleared between calls and nothing relies on its contents.
 *   - the first call on a device resolves the array's device address (cudaGetSymbolAddress);
 *     make that first call before any stream capture. ---- */
int mcl_cuda_counter_update_fused_static(void* cuda_stream, uint8_t* state, float* scale, float* v,
                                         const float* grad_out, const float* x, uint32_t* packed2_out,
                                         size_t C, size_t in_features, size_t out_features, size_t batch,
                                         float lr, float lr_scale, float rms_beta, float rms_eps,
                                         uint32_t seed);
size_t mcl_cuda_static_scratch_floats(void);
const char* mcl_cuda_static_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MOTIFCL_CUDA_H */
