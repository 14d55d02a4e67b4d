"""Loader for libmotifcl_cuda.so (the C ABI declared in include/motifcl_cuda.h).

There is no CPU or PyTorch fallback: if the library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import re
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
# MOTIFCL_CUDA_LIBRARY names another build of the library (same C ABI) to load instead of the in-tree one
LIB_PATH = os.environ.get("MOTIFCL_CUDA_LIBRARY") or os.path.join(_PKG, "lib", "libmotifcl_cuda.so")
HEADER_PATH = os.path.join(os.path.dirname(_PKG), "include", "motifcl_cuda.h")


class MotifclCudaError(RuntimeError):
    """A C-ABI call returned a non-zero status; `.code` holds it."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[mcl_cuda status {code}] {message}")
        self.code = code
        self.message = message


def build_library(verbose: bool = False) -> str:
    """Compile the CUDA sources for sm_100a into lib/libmotifcl_cuda.so (nvcc, no GPU needed)."""
    cmd = ["make", "-C", os.path.join(_PKG, "csrc"), "-j8"]
    if not verbose:
        cmd.insert(1, "-s")
    subprocess.check_call(cmd)
    return LIB_PATH


def declared_symbols() -> list[str]:
    """Entry points declared in include/motifcl_cuda.h."""
    text = open(HEADER_PATH).read()
    return sorted(set(re.findall(r"\b(mcl_cuda_[a-z0-9_]+)\s*\(", text)))


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} not found: build it with motifcl_b200.build_library() "
                "(there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        vp, sz, i, f, u32 = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_uint32
        L.mcl_cuda_device_count.restype = i
        L.mcl_cuda_create.argtypes = [i, C.POINTER(vp)]
        L.mcl_cuda_create_on_stream.argtypes = [i, vp, C.POINTER(vp)]
        L.mcl_cuda_destroy.argtypes = [vp]
        L.mcl_cuda_destroy.restype = None
        L.mcl_cuda_last_error.argtypes = [vp]
        L.mcl_cuda_last_error.restype = C.c_char_p
        L.mcl_cuda_device_name.argtypes = [vp]
        L.mcl_cuda_device_name.restype = C.c_char_p
        L.mcl_cuda_sm_count.argtypes = [vp]
        L.mcl_cuda_device_memory_bytes.argtypes = [vp]
        L.mcl_cuda_device_memory_bytes.restype = C.c_size_t
        L.mcl_cuda_launch_count.argtypes = [vp]
        L.mcl_cuda_launch_count.restype = C.c_uint64
        L.mcl_cuda_workspace_bytes.argtypes = [vp]
        L.mcl_cuda_workspace_bytes.restype = C.c_size_t
        L.mcl_cuda_finish.argtypes = [vp]
        L.mcl_cuda_alloc.argtypes = [vp, sz, C.POINTER(vp)]
        L.mcl_cuda_free.argtypes = [vp, vp]
        L.mcl_cuda_upload.argtypes = [vp, vp, vp, sz]
        L.mcl_cuda_download.argtypes = [vp, vp, vp, sz]
        L.mcl_cuda_counter_decode_weight.argtypes = [vp, vp, vp, vp, sz, sz, sz]
        L.mcl_cuda_counter_pack2.argtypes = [vp, vp, vp, sz, sz, sz]
        L.mcl_cuda_counter_forward.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, sz]
        L.mcl_cuda_counter_backward_input.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, sz]
        L.mcl_cuda_counter_update_dense.argtypes = [vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f, f, f, f, u32]
        L.mcl_cuda_counter_update_fused.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz,
                                                    f, f, f, f, u32]
        L.mcl_cuda_batch_begin.argtypes = [vp]
        L.mcl_cuda_batch_end.argtypes = [vp, C.POINTER(vp)]
        L.mcl_cuda_batch_launch.argtypes = [vp, vp]
        L.mcl_cuda_batch_destroy.argtypes = [vp]
        L.mcl_cuda_batch_destroy.restype = None
        L.mcl_cuda_lane_fork.argtypes = [vp, vp]
        L.mcl_cuda_lane_join.argtypes = [vp, vp]
        L.mcl_cuda_set_seed_offset.argtypes = [vp, vp]
        L.mcl_cuda_set_gemm_mode.argtypes = [vp, i, i, i]
        L.mcl_cuda_counter_linear_step.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, sz,
                                                   f, f, f, f, u32]
        L.mcl_cuda_counter_linear_step_many.argtypes = [vp, vp, sz, sz, f, f, f, f, u32]
        L.mcl_cuda_counter_update_dense_many.argtypes = [vp, vp, sz, sz, f, f, f, f, u32]
        L.mcl_cuda_ternary_linear_products.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, sz, sz]
        L.mcl_cuda_eltwise_f32.argtypes = [vp, i, vp, vp, vp, sz, f]
        L.mcl_cuda_matmul_f32.argtypes = [vp, vp, vp, vp, sz, sz, sz, i, i]
        L.mcl_cuda_rmsnorm.argtypes = [vp, vp, vp, vp, sz, sz, f]
        L.mcl_cuda_rmsnorm_backward_x.argtypes = [vp, vp, vp, vp, vp, sz, sz, f]
        L.mcl_cuda_rmsnorm_backward_weight.argtypes = [vp, vp, vp, vp, vp, sz, sz, f]
        L.mcl_cuda_swiglu.argtypes = [vp, vp, vp, sz, sz]
        L.mcl_cuda_mse_loss_partial.argtypes = [vp, vp, vp, vp, sz]
        L.mcl_cuda_peer_allreduce_f32.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.c_int, C.c_int, sz, sz, C.c_int, vp]
        L.mcl_cuda_peer_buffer_create.argtypes = [vp, sz, C.POINTER(vp), C.c_char_p]
        L.mcl_cuda_peer_buffer_open.argtypes = [vp, C.c_char_p, C.POINTER(vp)]
        L.mcl_cuda_peer_buffer_close.argtypes = [vp, vp]
        L.mcl_cuda_peer_buffer_destroy.argtypes = [vp, vp]
        L.mcl_cuda_mean_reduce.argtypes = [vp, vp, vp, sz, sz]
        L.mcl_cuda_mse_backward.argtypes = [vp, vp, vp, vp, vp, sz]
        L.mcl_cuda_swiglu_backward.argtypes = [vp, vp, vp, vp, sz, sz]
        L.mcl_cuda_softmax_cross_entropy.argtypes = [vp, vp, vp, vp, vp, sz, sz]
        L.mcl_cuda_softmax_cross_entropy_backward.argtypes = [vp, vp, vp, vp, vp, sz, sz]
        L.mcl_cuda_token_position_embedding.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, sz]
        L.mcl_cuda_embedding_weight_backward.argtypes = [vp, vp, vp, vp, sz, sz, sz, i]
        L.mcl_cuda_position_embedding_backward.argtypes = [vp, vp, vp, sz, sz, sz]
        L.mcl_cuda_rope.argtypes = [vp, vp, vp, sz, sz, sz, sz, sz, sz, sz, f, i, i]
        L.mcl_cuda_adam_update.argtypes = [vp, vp, vp, vp, vp, sz, f, f, f, f, f, f, f]
        L.mcl_cuda_gqa_forward.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, sz, sz, sz, i, sz, sz, f]
        L.mcl_cuda_gqa_backward.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, sz, i, sz, f]
        L.mcl_cuda_ternary_gemv.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz]
        L.mcl_cuda_counter_update_fused_static.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f, f, f, f, u32]
        L.mcl_cuda_static_scratch_floats.restype = C.c_size_t
        L.mcl_cuda_static_last_error.restype = C.c_char_p
        _lib = L
    return _lib
