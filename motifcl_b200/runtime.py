"""Python face of the C ABI: a `Context` owns one mcl_cuda_ctx and forwards calls.

Device buffers are torch CUDA tensors (or raw integer device pointers); torch is used only
for device memory and streams.  Every method enqueues on the context's stream and raises
MotifclCudaError when the C call refuses or fails.
"""
from __future__ import annotations

import ctypes
import ctypes as C

from ._lib import MotifclCudaError, lib


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


class LinearDesc(ctypes.Structure):
    """mcl_cuda_linear_desc: one layer of mcl_cuda_counter_linear_step_many."""
    _fields_ = [("x", ctypes.c_void_p), ("grad_out", ctypes.c_void_p), ("state", ctypes.c_void_p),
                ("scale", ctypes.c_void_p), ("v", ctypes.c_void_p), ("y", ctypes.c_void_p),
                ("grad_x", ctypes.c_void_p), ("grad_w", ctypes.c_void_p), ("packed2_out", ctypes.c_void_p),
                ("in_features", ctypes.c_size_t), ("out_features", ctypes.c_size_t), ("batch", ctypes.c_size_t),
                ("update_rows", ctypes.c_size_t), ("row_offset", ctypes.c_size_t), ("packed2_in", ctypes.c_void_p)]


class UpdateDesc(ctypes.Structure):
    """mcl_cuda_update_desc: one layer (or row shard) of mcl_cuda_counter_update_dense_many."""
    _fields_ = [("state", ctypes.c_void_p), ("scale", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("grad_w", ctypes.c_void_p), ("packed2_out", ctypes.c_void_p),
                ("in_features", ctypes.c_size_t), ("rows", ctypes.c_size_t), ("row_offset", ctypes.c_size_t)]


def _fill(struct_type, entries):
    arr = (struct_type * len(entries))()
    for d, e in zip(arr, entries):
        for name, ctype in struct_type._fields_:
            val = e.get(name)
            setattr(d, name, _ptr(val) if ctype is ctypes.c_void_p else int(val or 0))
    return arr


def linear_descs(entries):
    """entries: dicts with the fields of LinearDesc (tensors or None for pointers) -> ctypes array."""
    return _fill(LinearDesc, entries)


def update_descs(entries):
    """entries: dicts with the fields of UpdateDesc -> ctypes array."""
    return _fill(UpdateDesc, entries)


class Context:
    """One device + one in-order stream, like the reference's Backend
    (MotifCL include/motifcl/runtime/backend.hpp:43-81)."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self._lib = lib()
        self._ctx = C.c_void_p()
        if stream is None:
            rc = self._lib.mcl_cuda_create(device, C.byref(self._ctx))
        else:
            rc = self._lib.mcl_cuda_create_on_stream(device, C.c_void_p(stream), C.byref(self._ctx))
        if rc != 0:
            raise MotifclCudaError(rc, self._lib.mcl_cuda_last_error(None).decode())
        self.device = device
        self.stream_handle = stream      # the cudaStream_t the context enqueues on (None: a stream of its own)

    @classmethod
    def on_torch_stream(cls, device: int = 0) -> "Context":
        import torch
        return cls(device, torch.cuda.current_stream(device).cuda_stream)

    def close(self):
        if self._ctx:
            self._lib.mcl_cuda_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise MotifclCudaError(rc, self._lib.mcl_cuda_last_error(self._ctx).decode())

    # -- context -------------------------------------------------------------------------
    @property
    def device_name(self) -> str:
        return self._lib.mcl_cuda_device_name(self._ctx).decode()

    @property
    def sm_count(self) -> int:
        return self._lib.mcl_cuda_sm_count(self._ctx)

    @property
    def launch_count(self) -> int:
        return int(self._lib.mcl_cuda_launch_count(self._ctx))

    @property
    def workspace_bytes(self) -> int:
        """Device bytes held by the context's internal grow-only workspace."""
        return int(self._lib.mcl_cuda_workspace_bytes(self._ctx))

    def finish(self):
        self._check(self._lib.mcl_cuda_finish(self._ctx))

    def alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self._check(self._lib.mcl_cuda_alloc(self._ctx, nbytes, C.byref(p)))
        return p.value

    def free(self, dptr: int):
        self._check(self._lib.mcl_cuda_free(self._ctx, dptr))

    def upload(self, dst, src_host_ptr: int, nbytes: int):
        self._check(self._lib.mcl_cuda_upload(self._ctx, _ptr(dst), src_host_ptr, nbytes))

    def download(self, dst_host_ptr: int, src, nbytes: int):
        self._check(self._lib.mcl_cuda_download(self._ctx, dst_host_ptr, _ptr(src), nbytes))

    # -- batch recording (one graph launch per recorded step) -------------------------------
    def batch_begin(self):
        self._check(self._lib.mcl_cuda_batch_begin(self._ctx))

    def batch_end(self) -> "Batch":
        b = C.c_void_p()
        self._check(self._lib.mcl_cuda_batch_end(self._ctx, C.byref(b)))
        return Batch(self, b)

    def lane_fork(self, lane: "Context"):
        self._check(self._lib.mcl_cuda_lane_fork(self._ctx, lane._ctx))

    def lane_join(self, lane: "Context"):
        self._check(self._lib.mcl_cuda_lane_join(self._ctx, lane._ctx))

    def set_seed_offset(self, device_word):
        self._check(self._lib.mcl_cuda_set_seed_offset(self._ctx, _ptr(device_word)))

    # -- counter path --------------------------------------------------------------------
    def counter_decode_weight(self, state, scale, weight, in_features, out_features, C_):
        self._check(self._lib.mcl_cuda_counter_decode_weight(
            self._ctx, _ptr(state), _ptr(scale), _ptr(weight), in_features, out_features, C_))

    def counter_pack2(self, state, packed2, in_features, out_features, C_):
        self._check(self._lib.mcl_cuda_counter_pack2(
            self._ctx, _ptr(state), _ptr(packed2), in_features, out_features, C_))

    def counter_forward(self, x, state, scale, y, batch, in_features, out_features, C_):
        self._check(self._lib.mcl_cuda_counter_forward(
            self._ctx, _ptr(x), _ptr(state), _ptr(scale), _ptr(y), batch, in_features, out_features, C_))

    def counter_backward_input(self, state, scale, grad_out, grad_x, batch, in_features, out_features, C_):
        self._check(self._lib.mcl_cuda_counter_backward_input(
            self._ctx, _ptr(state), _ptr(scale), _ptr(grad_out), _ptr(grad_x), batch, in_features,
            out_features, C_))

    def counter_update_dense(self, state, scale, v, grad_w, packed2_out, C_, in_features, rows,
                             row_offset, lr, lr_scale, rms_beta, rms_eps, seed):
        self._check(self._lib.mcl_cuda_counter_update_dense(
            self._ctx, _ptr(state), _ptr(scale), _ptr(v), _ptr(grad_w), _ptr(packed2_out), C_,
            in_features, rows, row_offset, lr, lr_scale, rms_beta, rms_eps, seed & 0xFFFFFFFF))

    def counter_update_fused(self, state, scale, v, grad_out, x, packed2_out, C_, in_features,
                             out_features, batch, lr, lr_scale, rms_beta, rms_eps, seed):
        self._check(self._lib.mcl_cuda_counter_update_fused(
            self._ctx, _ptr(state), _ptr(scale), _ptr(v), _ptr(grad_out), _ptr(x), None, None,
            _ptr(packed2_out), C_, in_features, out_features, batch, lr, lr_scale, rms_beta, rms_eps,
            seed & 0xFFFFFFFF))

    GEMM_MODES = {"auto": 0, "exact": 1, "tensor": 2}

    def set_gemm_mode(self, mode: str = "auto", act_terms: int = 3, grad_terms: int = 6):
        """auto | exact (CUDA cores, bit-equal to the reference sums) | tensor (tcgen05)."""
        self._check(self._lib.mcl_cuda_set_gemm_mode(self._ctx, self.GEMM_MODES[mode], act_terms, grad_terms))

    def counter_linear_step(self, x, grad_out, state, scale, v, y, grad_x, grad_w, packed2_out, C_,
                            in_features, out_features, batch, update_rows, row_offset, lr, lr_scale,
                            rms_beta, rms_eps, seed):
        self._check(self._lib.mcl_cuda_counter_linear_step(
            self._ctx, _ptr(x), _ptr(grad_out), _ptr(state), _ptr(scale), _ptr(v), _ptr(y), _ptr(grad_x),
            _ptr(grad_w), _ptr(packed2_out), C_, in_features, out_features, batch, update_rows, row_offset,
            lr, lr_scale, rms_beta, rms_eps, seed & 0xFFFFFFFF))

    def counter_linear_step_many(self, descs, C_, lr, lr_scale, rms_beta, rms_eps, seed):
        """descs: array from linear_descs(); the steps of all its layers with grouped launches."""
        self._check(self._lib.mcl_cuda_counter_linear_step_many(
            self._ctx, ctypes.cast(descs, ctypes.c_void_p), len(descs), C_, lr, lr_scale, rms_beta, rms_eps,
            seed & 0xFFFFFFFF))

    def counter_update_dense_many(self, descs, C_, lr, lr_scale, rms_beta, rms_eps, seed):
        """descs: array from update_descs(); the fused updates of all its layers in one launch."""
        self._check(self._lib.mcl_cuda_counter_update_dense_many(
            self._ctx, ctypes.cast(descs, ctypes.c_void_p), len(descs), C_, lr, lr_scale, rms_beta, rms_eps,
            seed & 0xFFFFFFFF))

    def ternary_linear_products(self, x, grad_out, packed2, scale, y, grad_x, grad_w, in_features,
                                out_features, batch):
        self._check(self._lib.mcl_cuda_ternary_linear_products(
            self._ctx, _ptr(x), _ptr(grad_out), _ptr(packed2), _ptr(scale), _ptr(y), _ptr(grad_x), _ptr(grad_w),
            in_features, out_features, batch))

    def matmul_f32(self, a, b, c, M, K, N, trans_a=False, trans_b=False):
        self._check(self._lib.mcl_cuda_matmul_f32(self._ctx, _ptr(a), _ptr(b), _ptr(c), M, K, N,
                                                  int(trans_a), int(trans_b)))

    # ---- fp32 row ops of the ternary15m block stack (MotifCL src/ops/norm.cpp, activation.cpp, loss.cpp,
    # attention.cpp on its Vulkan seam) -------------------------------------------------------------
    def eltwise(self, op: int, a, b, out, elements, alpha=0.0):
        self._check(self._lib.mcl_cuda_eltwise_f32(self._ctx, op, _ptr(a) if a is not None else None,
                                                   _ptr(b) if b is not None else None, _ptr(out), elements, alpha))

    def rmsnorm(self, x, weight, out, rows, cols, eps):
        self._check(self._lib.mcl_cuda_rmsnorm(self._ctx, _ptr(x), _ptr(weight), _ptr(out), rows, cols, eps))

    def rmsnorm_backward_x(self, x, weight, grad_out, grad_x, rows, cols, eps):
        self._check(self._lib.mcl_cuda_rmsnorm_backward_x(self._ctx, _ptr(x), _ptr(weight), _ptr(grad_out),
                                                          _ptr(grad_x), rows, cols, eps))

    def rmsnorm_backward_weight(self, x, grad_out, row_inv, grad_weight, rows, cols, eps):
        self._check(self._lib.mcl_cuda_rmsnorm_backward_weight(self._ctx, _ptr(x), _ptr(grad_out), _ptr(row_inv),
                                                               _ptr(grad_weight), rows, cols, eps))

    def mse_loss(self, pred, target, partial, out, n):
        """mean((pred - target)^2) with MotifCL's OpenCL summation order; partial: ceil(n / 256) floats."""
        self._check(self._lib.mcl_cuda_mse_loss_partial(self._ctx, _ptr(pred), _ptr(target), _ptr(partial), n))
        self._check(self._lib.mcl_cuda_mean_reduce(self._ctx, _ptr(partial), _ptr(out), (n + 255) // 256, n))

    def mse_backward(self, pred, target, grad_out, grad_pred, n):
        self._check(self._lib.mcl_cuda_mse_backward(self._ctx, _ptr(pred), _ptr(target), _ptr(grad_out), _ptr(grad_pred), n))

    def swiglu(self, packed, out, rows, hidden):
        self._check(self._lib.mcl_cuda_swiglu(self._ctx, _ptr(packed), _ptr(out), rows, hidden))

    def swiglu_backward(self, packed, grad_out, grad_packed, rows, hidden):
        self._check(self._lib.mcl_cuda_swiglu_backward(self._ctx, _ptr(packed), _ptr(grad_out), _ptr(grad_packed),
                                                       rows, hidden))

    def softmax_cross_entropy(self, logits, targets, partial, out, rows, cols):
        self._check(self._lib.mcl_cuda_softmax_cross_entropy(self._ctx, _ptr(logits), _ptr(targets), _ptr(partial),
                                                             _ptr(out), rows, cols))

    def softmax_cross_entropy_backward(self, logits, targets, grad_out, grad_logits, rows, cols):
        self._check(self._lib.mcl_cuda_softmax_cross_entropy_backward(self._ctx, _ptr(logits), _ptr(targets),
                                                                      _ptr(grad_out), _ptr(grad_logits), rows, cols))

    def token_position_embedding(self, token_weight, pos_weight, token_ids, out, token_count, vocab, seq_len, dim):
        self._check(self._lib.mcl_cuda_token_position_embedding(
            self._ctx, _ptr(token_weight), _ptr(pos_weight) if pos_weight is not None else None, _ptr(token_ids),
            _ptr(out), token_count, vocab, seq_len, dim))

    def embedding_weight_backward(self, indices, grad_out, grad_weight, vocab, dim, token_count, zero_first=True):
        self._check(self._lib.mcl_cuda_embedding_weight_backward(self._ctx, _ptr(indices), _ptr(grad_out),
                                                                 _ptr(grad_weight), vocab, dim, token_count,
                                                                 int(zero_first)))

    def position_embedding_backward(self, grad_out, grad_position, batch, seq_len, dim):
        self._check(self._lib.mcl_cuda_position_embedding_backward(self._ctx, _ptr(grad_out), _ptr(grad_position),
                                                                   batch, seq_len, dim))

    def rope(self, x, out, batch, tokens, channels, n_head, head_dim, rotary_dim=0, token_offset=0, theta=10000.0,
             inverse=False, split_half=False):
        self._check(self._lib.mcl_cuda_rope(self._ctx, _ptr(x), _ptr(out), batch, tokens, channels, n_head, head_dim,
                                            rotary_dim, token_offset, theta, int(inverse), int(split_half)))

    def adam_update(self, param, grad, m, v, elements, lr, beta1, beta2, eps, weight_decay, c1, c2):
        self._check(self._lib.mcl_cuda_adam_update(self._ctx, _ptr(param), _ptr(grad), _ptr(m), _ptr(v), elements, lr,
                                                   beta1, beta2, eps, weight_decay, c1, c2))

    def gqa_forward(self, q, k, v, out, batch, tq, tk, key_stride, n_head, n_kv_head, head_dim, v_head_dim,
                    causal, query_offset, sliding_window, scale):
        self._check(self._lib.mcl_cuda_gqa_forward(self._ctx, _ptr(q), _ptr(k), _ptr(v), _ptr(out), batch, tq, tk,
                                                   key_stride, n_head, n_kv_head, head_dim, v_head_dim, int(causal),
                                                   query_offset, sliding_window, scale))

    def gqa_backward(self, q, k, v, grad_out, probs, ds, grad_q, grad_k, grad_v, batch, tq, tk, n_head, n_kv_head,
                     head_dim, causal, query_offset, scale):
        self._check(self._lib.mcl_cuda_gqa_backward(self._ctx, _ptr(q), _ptr(k), _ptr(v), _ptr(grad_out), _ptr(probs),
                                                    _ptr(ds), _ptr(grad_q), _ptr(grad_k), _ptr(grad_v), batch, tq, tk,
                                                    n_head, n_kv_head, head_dim, int(causal), query_offset, scale))

    def ternary_gemv(self, x, packed2, scale, y, M, in_features, out_features):
        self._check(self._lib.mcl_cuda_ternary_gemv(self._ctx, _ptr(x), _ptr(packed2), _ptr(scale),
                                                    _ptr(y), M, in_features, out_features))


class Batch:
    """A recorded sequence of calls (Context.batch_begin ... batch_end), replayed with launch()."""

    def __init__(self, ctx: Context, handle):
        self._ctx, self._h = ctx, handle

    def launch(self):
        self._ctx._check(self._ctx._lib.mcl_cuda_batch_launch(self._ctx._ctx, self._h))

    def close(self):
        if self._h:
            self._ctx._lib.mcl_cuda_batch_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
