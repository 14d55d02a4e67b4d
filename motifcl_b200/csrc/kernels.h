// Internal launch interface between the C-ABI layer (abi.cu) and the kernel files.
// Every launcher enqueues on `stream` and returns the launch status; none synchronises.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mcl {

// counter_update.cu
cudaError_t ensure_dynamic_smem(const void* kern, int slot, size_t max_smem);
// err_word (may be null): device word that the wide-row kernel sets when a bounded wait gives up
cudaError_t launch_counter_update_dense(uint8_t* state, float* scale, float* v, const float* grad_w,
                                        uint32_t* packed2, int C, int in_features, int rows,
                                        int row_offset, float lr, float lr_scale, float rms_beta,
                                        float rms_eps, uint32_t seed, const uint32_t* seed_offset, int* err_word,
                                        int sm_count, size_t max_smem, cudaStream_t stream);
struct UpdateDesc {            // rows [row_offset, row_offset + rows) of one layer; pointers at the first row
    uint8_t* state;
    float* scale;
    float* v;
    const float* grad_w;
    uint32_t* packed2;         // may be null
    int in_features, rows, row_offset;
};
cudaError_t launch_counter_update_group(const UpdateDesc* d, int n, int C, float lr, float lr_scale, float rms_beta,
                                        float rms_eps, uint32_t seed, const uint32_t* seed_offset, int* err_word, int sm_count,
                                        size_t max_smem, cudaStream_t stream, int* launches);
cudaError_t launch_decode_weight(const uint8_t* state, const float* scale, float* w, int C,
                                 int in_features, int out_features, int sm_count, cudaStream_t stream);
cudaError_t launch_pack2(const uint8_t* state, uint32_t* packed2, int C, int in_features,
                         int out_features, int sm_count, cudaStream_t stream);

// simt_gemm.cu -- fp32 CUDA-core contractions (any shape; exact fp32 FMA accumulation)
cudaError_t launch_simt_matmul_f32(const float* a, const float* b, float* c, int M, int K, int N,
                                   int transA, int transB, cudaStream_t stream);
cudaError_t launch_simt_counter_forward(const float* x, const uint8_t* state, const float* scale,
                                        float* y, int batch, int in_features, int out_features, int C,
                                        cudaStream_t stream);
cudaError_t launch_simt_counter_backward_input(const uint8_t* state, const float* scale,
                                               const float* grad_out, float* grad_x, int batch,
                                               int in_features, int out_features, int C,
                                               cudaStream_t stream);
cudaError_t launch_simt_ternary_forward(const float* x, const uint32_t* packed2, const float* scale, float* y,
                                        int batch, int in_features, int out_features, cudaStream_t stream);
cudaError_t launch_simt_ternary_backward_input(const uint32_t* packed2, const float* scale, const float* grad_out,
                                               float* grad_x, int batch, int in_features, int out_features,
                                               cudaStream_t stream);
// dW rows [row0, row0+rows) of dY^T X into grad_w[rows, in]
cudaError_t launch_simt_grad_w(const float* grad_out, const float* x, float* grad_w, int batch,
                               int in_features, int out_features, int row0, int rows,
                               cudaStream_t stream);

// tc_gemm.cu -- tcgen05 / TMEM / TMA contractions on bf16 term planes (see the file header)
int tc_pick_bn(int N);
size_t tc_splitk_workspace_bytes(int M, int N, int K, int sm_count, int depth_limit, int* splits_out);
constexpr int kGradDepthLimit = 32;   // k-tiles per accumulator for fp32 x fp32 products (K = 2048)
// C[M,N] (+= over terms) A_pa[M,K] . B_pb[N,K]^T ; planes are bf16 [P][rows][ld], plane stride in elements
cudaError_t launch_tc_gemm(const void* a_planes, int a_nplanes, int lda, size_t a_plane_stride,
                           const void* b_planes, int b_nplanes, int ldb, size_t b_plane_stride, float* c,
                           int ldc, int M, int N, int K, const int* pa, const int* pb, int nterms,
                           const float* col_scale, float* splitk_ws, int splits, int* err_word,
                           size_t max_smem, int sm_count, cudaStream_t stream, int* launches);
// fp32 [R,Cc] -> bf16 term planes [t][R][ld_n] of (src * col_scale) and/or transposed planes
// [t][Cc][ld_t] of src
cudaError_t launch_split_planes(const float* src, int R, int Cc, const float* col_scale, void* planes, int ld_n,
                                int nterms, void* planes_t, int ld_t, int nterms_t, cudaStream_t stream);
// packed 6-bit state -> bf16 ternary digits T [O][ld_i] and/or T^T [I][ld_o]
cudaError_t launch_expand_ternary(const uint8_t* state, int C, int O, int I, void* T, int ld_i, void* Tt, int ld_o,
                                  cudaStream_t stream);

cudaError_t launch_expand_ternary_p2(const uint32_t* packed2, int O, int I, void* T, int ld_i, void* Tt, int ld_o,
                                     cudaStream_t stream);

// tc_fused.cu -- grouped tcgen05 (tf32, two terms) contractions straight from fp32 tensors
// kFusedYB / kFusedDXB are Y and dX with the activation split into two bf16 terms and the ternary digits given
// as a K-major bf16 matrix (T [out,in] for Y, its transpose [in,out] for dX): k-tiles of 64, kind::f16
enum { kFusedY = 0, kFusedDX = 1, kFusedDW = 2, kFusedYB = 3, kFusedDXB = 4 };
constexpr int kFusedMaxProblems = 63;
// dW on tf32 terms: 3 products x 4 instructions per 32-deep k-tile add into one accumulator, each with a truncation error of
// ~2e-8 relative; 16 k-tiles (512 tokens) keep that below 4e-6
#ifndef MCL_FUSED_FLUSH
#define MCL_FUSED_FLUSH 16
#endif
#ifndef MCL_FUSED_DW_DEPTH
#define MCL_FUSED_DW_DEPTH 64
#endif
constexpr int kFusedFlushKtiles = MCL_FUSED_FLUSH;
// k-tiles (of 32 tokens) of one dW work item: longer items mean fewer split-K partials to write and add up
constexpr int kFusedDwDepth = MCL_FUSED_DW_DEPTH;
struct FusedOperand {          // a row-major tensor read through TMA (host side only)
    const float* ptr;          // fp32 elements, or bf16 ones when `bf16` is set
    int rows, cols, ld;
    int mn_major;              // read as a transposed operand (cols % 32 == 0): 32-byte-atom swizzle, 3-D box
    int box_outer;             // rows of the box (K-major) or 32-column chunks per box (MN-major)
    int bf16;                  // K-major bf16 matrix: box of 64 elements x box_outer rows
};
struct FusedProblem {          // C[M,N] = A[M,K] . B[N,K]^T, see the kinds in tc_fused.cu
    const float* a_kscale;     // DX: A is multiplied by a_kscale[k] (rounded to fp32) before the split
    const float* col_scale;    // optional scale of output column n (ignored for split-K partials)
    float* C;                  // [M, ldc], or split-K partials [splits][M][ldc]
    int M, N, K, ldc;
    int mode;
    int BN, tiles_m, tiles_n, splits, ktiles_per_split;   // filled by fused_plan (k-tiles of 32)
    int nprod;                 // products per k-tile
    int flush;                 // k-tiles (of 32) one accumulator takes before the epilogue adds it to the output; 0 = the whole item
    uint32_t prod;             // 4 bits each: A term | B term << 2 (0 = hi, 1 = lo), smallest first
    int a_map, b_map, item_begin;                         // filled by the launcher
};
// chooses the column tile and the K split of a problem; returns the floats of split-K workspace it needs
size_t fused_plan(FusedProblem* p, int target_items, int depth_limit);
// err_word points at two ints: the error word and the work-item counter (zeroed by the launcher)
cudaError_t launch_tc_fused(const FusedProblem* probs, const FusedOperand* a_ops, const FusedOperand* b_ops, int n,
                            int* err_word, size_t max_smem, int sm_count, cudaStream_t stream, int* launches);
// ternary digits of a layer as fp32 [O][I], from the 6-bit state (state != null) or the 2-bit words
cudaError_t launch_ternary_f32(const uint8_t* state, const uint32_t* packed2, int C, int O, int I, float* T,
                               int sm_count, cudaStream_t stream);
// grouped forms: one launch for the layers of a step
cudaError_t launch_ternary_f32_group(const uint8_t* const* state, const uint32_t* const* packed2, float* const* T, const int* O, const int* I, int n, int C,
                                     int sm_count, cudaStream_t stream, int* launches);
cudaError_t launch_splitk_reduce_group(const float* const* partial, float* const* out, const int* elements, const int* splits,
                                       int n, int sm_count, cudaStream_t stream, int* launches);
// ternary digits of the layers as bf16, both orientations: T [O][I] and Tt [I][O]
cudaError_t launch_ternary_bf16_group(const uint8_t* const* state, const uint32_t* const* packed2, void* const* T, void* const* Tt,
                                      const int* O, const int* I, int n, int C, int sm_count, cudaStream_t stream, int* launches);
// tc_gemm.cu: TMA map of a row-major fp32 matrix, 128-byte swizzle, zero fill outside
bool tc_encode_map_f32(void* map, const float* base, int cols, int rows, int ld, int mn_major, int box_outer);
// the same for a K-major bf16 matrix: box of 64 elements x box_outer rows
bool tc_encode_map_bf16(void* map, const void* base, int cols, int rows, int ld, int box_outer);
cudaError_t launch_splitk_reduce(const float* partial, float* c, const float* col_scale, int M, int N, int ldc,
                                 int splits, cudaStream_t stream);

// gemv.cu
// M <= 2: one CUDA-core launch that streams the 2-bit words (in_features % 16 == 0)
cudaError_t launch_ternary_gemv_stream(const float* x, const uint32_t* packed2, const float* scale, float* y, int M,
                                       int in_features, int out_features, int sm_count, cudaStream_t stream);
// table look-up kernels for M = 1 (in_features % 256 == 0, 16-byte aligned words); tickets: zeroed words, one per 256 rows
bool gemv_lut_supported(int M, int in_features, int out_features, const void* packed2, int ticket_words);
size_t gemv_lut_workspace_bytes(int in_features, int out_features);
cudaError_t launch_ternary_gemv_lut(const float* x, const uint32_t* packed2, const float* scale, float* y,
                                    int in_features, int out_features, float* part, unsigned int* tickets, int sm_count,
                                    size_t max_smem, cudaStream_t stream);
cudaError_t launch_ternary_gemv(const float* x, const uint32_t* packed2, const float* scale, float* y,
                                int M, int in_features, int out_features, int sm_count,
                                cudaStream_t stream);


// peer_reduce.cu -- one-shot sum of a small vector over the GPUs of a node (peer loads, bounded flag wait)
constexpr int kPeerMaxWorld = 8;
constexpr int kPeerErrCode = 31;
constexpr int kPeerFlagWords = 64;        // a rank's flag area: one word per rank, then the call counter
constexpr int kPeerCounterWord = 32;
struct PeerTable {
    const float* data[kPeerMaxWorld];     // every rank's partial buffers (two parities, parity_stride4 float4 apart)
    uint32_t* flags[kPeerMaxWorld];       // every rank's flag words: flags[r][s] = last partial number rank s announced to rank r
    size_t parity_stride4;
    int rank, world;
};
cudaError_t launch_peer_allreduce(const PeerTable& tab, size_t n, int parity, float* out, int* err_word, cudaStream_t stream);

// gemv_tc.cu -- the same GEMV as integer tensor-core MMA on digit-split activations
bool gemv_tc_supported(int M, int in_features, int out_features);
size_t gemv_tc_workspace_bytes(int M, int in_features, int out_features);
cudaError_t launch_ternary_gemv_tc(const float* x, const uint32_t* packed2, const float* scale, float* y, int M,
                                   int in_features, int out_features, void* workspace, int* err_word, int sm_count,
                                   size_t max_smem, cudaStream_t stream, int* launches);

// eltwise.cu: op 0 add, 1 sub, 2 mul, 3 mul_scalar, 4 add_scalar, 5 zero, 6 a - alpha*b
cudaError_t launch_eltwise_f32(int op, const float* a, const float* b, float* out, size_t n, float alpha,
                               int sm_count, cudaStream_t stream);

// trainer_ops.cu -- the fp32 row ops of the ternary15m block stack around its counter layers
cudaError_t launch_rmsnorm(const float* x, const float* w, float* out, size_t rows, int cols, float eps, int sm_count,
                           cudaStream_t stream);
cudaError_t launch_rmsnorm_backward_x(const float* x, const float* w, const float* dy, float* dx, size_t rows, int cols,
                                      float eps, int sm_count, cudaStream_t stream);
cudaError_t launch_rmsnorm_backward_weight(const float* x, const float* dy, float* row_inv, float* dw, size_t rows,
                                           int cols, float eps, int sm_count, cudaStream_t stream);
cudaError_t launch_mse_loss_partial(const float* pred, const float* target, float* partial, size_t n, cudaStream_t stream);
cudaError_t launch_mean_reduce(const float* partial, float* out, int count, int denominator, cudaStream_t stream);
cudaError_t launch_mse_backward(const float* pred, const float* target, const float* grad_out, float* grad_pred, size_t n,
                                cudaStream_t stream);
cudaError_t launch_swiglu(const float* packed, float* out, size_t rows, int hidden, int sm_count, cudaStream_t stream);
cudaError_t launch_swiglu_backward(const float* packed, const float* dy, float* dpacked, size_t rows, int hidden,
                                   int sm_count, cudaStream_t stream);
cudaError_t launch_softmax_cross_entropy(const float* logits, const int* targets, float* partial, float* out, size_t rows,
                                         int cols, int sm_count, cudaStream_t stream);
cudaError_t launch_softmax_cross_entropy_backward(const float* logits, const int* targets, const float* grad_out,
                                                  float* grad_logits, size_t rows, int cols, int sm_count,
                                                  cudaStream_t stream);
cudaError_t launch_embedding(const float* token_weight, const float* pos_weight, const int* ids, float* out, size_t tokens,
                             int vocab, int seq_len, int dim, int sm_count, cudaStream_t stream);
cudaError_t launch_embedding_scatter(const int* ids, const float* grad_out, float* grad_weight, size_t tokens, int vocab, int dim,
                                     int sm_count, cudaStream_t stream);
cudaError_t launch_position_backward(const float* grad_out, float* grad_position, int batch, int seq_len, int dim, int sm_count,
                                     cudaStream_t stream);
cudaError_t launch_rope(const float* x, float* out, size_t rows, int tokens, int channels, int n_head, int head_dim,
                        int rotary_dim, int token_offset, float theta, int inverse, int split_half, int sm_count,
                        cudaStream_t stream);
cudaError_t launch_adam(float* param, const float* grad, float* m, float* v, size_t n, float lr, float beta1, float beta2,
                        float eps, float weight_decay, float c1, float c2, int sm_count, cudaStream_t stream);
cudaError_t launch_gqa_forward(const float* q, const float* k, const float* v, float* out, int batch, int tq, int tk,
                               int key_stride, int n_head, int n_kv, int hd, int vhd, int causal, int q_off, int window,
                               float scale, float* scores_ws, cudaStream_t stream, int* launches);
cudaError_t launch_gqa_backward(const float* q, const float* k, const float* v, const float* dout, float* probs, float* ds,
                                float* dq, float* dk, float* dv, int batch, int tq, int tk, int n_head, int n_kv, int hd,
                                int causal, int q_off, float scale, cudaStream_t stream, int* launches);

}  // namespace mcl
