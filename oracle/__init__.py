"""ctypes bindings for the CPU checker (TEST INFRASTRUCTURE ONLY).

`oracle.port` wraps liboracle.so (oracle/counter_oracle.cpp, the restatement of the
reference's counter-linear arithmetic) and `oracle.ref` wraps _ref/libmotifcl_ref.so (the
reference's own kernels/compact_counter.cl and src/runtime/native_matmul.cpp compiled by
oracle/Makefile; None when it was not built).  Only tests, the smoke check and the
benchmark's CPU-baseline leg may import this package; the product never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")


def build(ref_tree: str | None = None) -> None:
    """Compile liboracle.so, and the compiled-reference library when `ref_tree` exists."""
    if ref_tree is None:      # MOTIFCL_REF, else a `reference` directory beside this repository
        ref_tree = os.environ.get("MOTIFCL_REF", os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"))
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])
    if os.path.isfile(os.path.join(ref_tree, "kernels", "compact_counter.cl")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={ref_tree}"])


def _load(path):
    return C.CDLL(path) if os.path.isfile(path) else None


class _Port:
    def __init__(self, lib):
        self.lib = lib
        L = lib
        i, f, u = C.c_int, C.c_float, C.c_uint32
        L.orc_set_threads.argtypes = [i]
        L.orc_get_threads.restype = i
        L.orc_pack_codes.argtypes = [_u8p, _u8p, C.c_int64]
        L.orc_unpack_codes.argtypes = [_u8p, _u8p, C.c_int64]
        L.orc_decode_weight.argtypes = [_u8p, _f32p, _f32p, i, i, i]
        L.orc_pack2.argtypes = [_u8p, _u32p, i, i, i]
        L.orc_row_stats.argtypes = [_u8p, _f32p, _f32p, _f32p, _f32p, _f32p, i, i, i, f, f, f]
        L.orc_update_dense.argtypes = [_u8p, _f32p, _f32p, _f32p, C.c_void_p, i, i, i, i, f, f, f, f, u]
        L.orc_grad_w.argtypes = [_f32p, _f32p, _f32p, i, i, i]
        L.orc_update_fused.argtypes = [_u8p, _f32p, _f32p, _f32p, _f32p, C.c_void_p, i, i, i, i, f, f, f, f, u]
        L.orc_forward.argtypes = [_f32p, _u8p, _f32p, _f32p, i, i, i, i]
        L.orc_backward_input.argtypes = [_f32p, _u8p, _f32p, _f32p, i, i, i, i]
        L.orc_matmul_f32.argtypes = [_f32p, _f32p, _f32p, i, i, i, i, i]
        L.orc_matmul_f64acc.argtypes = [_f32p, _f32p, _f64p, i, i, i, i, i]
        L.orc_matmul_f32_m1.argtypes = [_f32p, _f32p, _f32p, C.c_int64, C.c_int64]
        L.orc_ternary_gemv.argtypes = [_f32p, _u32p, _f32p, _f32p, i, i, i]
        L.orc_ternary_gemv_f64.argtypes = [_f32p, _u32p, _f32p, _f64p, i, i, i]

    def set_threads(self, n):
        self.lib.orc_set_threads(int(n))

    def pack_codes(self, codes):
        codes = np.ascontiguousarray(codes, np.uint8)
        st = np.empty(codes.size // 4 * 3, np.uint8)
        self.lib.orc_pack_codes(codes.reshape(-1), st, codes.size)
        return st

    def unpack_codes(self, state, n_weights):
        out = np.empty(n_weights, np.uint8)
        self.lib.orc_unpack_codes(np.ascontiguousarray(state), out, n_weights)
        return out

    def decode_weight(self, state, scale, Cc, I, O):
        w = np.empty((O, I), np.float32)
        self.lib.orc_decode_weight(state, scale, w, Cc, I, O)
        return w

    def pack2(self, state, Cc, I, O):
        p = np.empty((O, I // 16), np.uint32)
        self.lib.orc_pack2(state, p, Cc, I, O)
        return p

    def update_dense(self, state, scale, v, grad_w, Cc, I, rows, row_offset, lr, lr_scale, beta,
                     eps, seed, want_packed2=True):
        """Returns new (state, scale, v, packed2|None); inputs are not modified."""
        st, sc, vv = state.copy(), scale.copy(), v.copy()
        p2 = np.zeros((rows, I // 16), np.uint32) if (want_packed2 and I % 16 == 0) else None
        self.lib.orc_update_dense(st, sc, vv, np.ascontiguousarray(grad_w, np.float32),
                                  p2.ctypes.data if p2 is not None else None, Cc, I, rows,
                                  row_offset, lr, lr_scale, beta, eps, seed)
        return st, sc, vv, p2

    def grad_w(self, grad_out, x):
        N, O = grad_out.shape
        I = x.shape[1]
        gw = np.empty((O, I), np.float32)
        self.lib.orc_grad_w(grad_out, x, gw, N, I, O)
        return gw

    def update_fused(self, state, scale, v, grad_out, x, Cc, lr, lr_scale, beta, eps, seed):
        N, O = grad_out.shape
        I = x.shape[1]
        st, sc, vv = state.copy(), scale.copy(), v.copy()
        p2 = np.zeros((O, I // 16), np.uint32) if I % 16 == 0 else None
        self.lib.orc_update_fused(st, sc, vv, grad_out, x,
                                  p2.ctypes.data if p2 is not None else None, Cc, I, O, N, lr,
                                  lr_scale, beta, eps, seed)
        return st, sc, vv, p2

    def forward(self, x, state, scale, Cc, O):
        N, I = x.shape
        y = np.empty((N, O), np.float32)
        self.lib.orc_forward(x, state, scale, y, N, I, O, Cc)
        return y

    def backward_input(self, grad_out, state, scale, Cc, I):
        N, O = grad_out.shape
        gx = np.empty((N, I), np.float32)
        self.lib.orc_backward_input(grad_out, state, scale, gx, N, I, O, Cc)
        return gx

    def matmul(self, A, B, M, K, N, transA=False, transB=False, f64=False):
        out = np.empty((M, N), np.float64 if f64 else np.float32)
        fn = self.lib.orc_matmul_f64acc if f64 else self.lib.orc_matmul_f32
        fn(np.ascontiguousarray(A, np.float32), np.ascontiguousarray(B, np.float32), out, M, K, N,
           int(transA), int(transB))
        return out

    def matmul_m1(self, a, b):
        k, n = b.shape
        out = np.empty(n, np.float32)
        self.lib.orc_matmul_f32_m1(a, b, out, k, n)
        return out

    def ternary_gemv(self, x, packed2, scale, f64=False):
        M, I = x.shape
        O = packed2.shape[0]
        y = np.empty((M, O), np.float64 if f64 else np.float32)
        fn = self.lib.orc_ternary_gemv_f64 if f64 else self.lib.orc_ternary_gemv
        fn(x, packed2, scale, y, M, I, O)
        return y


class _Ref:
    def __init__(self, lib):
        self.lib = lib
        L = lib
        i, f, u = C.c_int, C.c_float, C.c_uint32
        L.ref_decode_weight.argtypes = [_u8p, _f32p, _f32p, i, i, i]
        L.ref_update_dense.argtypes = [_u8p, _f32p, _f32p, _f32p, i, i, i, f, f, f, f, u]
        L.ref_update_fused.argtypes = [_u8p, _f32p, _f32p, _f32p, _f32p, i, i, i, i, f, f, f, f, u]
        L.ref_backward_input.argtypes = [_f32p, _u8p, _f32p, _f32p, i, i, i, i]
        L.ref_matmul_f32_m1.argtypes = [_f32p, _f32p, _f32p, C.c_longlong, C.c_longlong]

    def decode_weight(self, state, scale, Cc, I, O):
        w = np.empty((O, I), np.float32)
        self.lib.ref_decode_weight(state, scale, w, Cc, I, O)
        return w

    def update_dense(self, state, scale, v, grad_w, Cc, I, O, lr, lr_scale, beta, eps, seed):
        st, sc, vv = state.copy(), scale.copy(), v.copy()
        self.lib.ref_update_dense(st, sc, vv, np.ascontiguousarray(grad_w, np.float32), Cc, I, O,
                                  lr, lr_scale, beta, eps, seed)
        return st, sc, vv

    def update_fused(self, state, scale, v, grad_out, x, Cc, lr, lr_scale, beta, eps, seed):
        N, O = grad_out.shape
        I = x.shape[1]
        st, sc, vv = state.copy(), scale.copy(), v.copy()
        self.lib.ref_update_fused(st, sc, vv, grad_out, x, Cc, I, O, N, lr, lr_scale, beta, eps, seed)
        return st, sc, vv

    def backward_input(self, grad_out, state, scale, Cc, I):
        N, O = grad_out.shape
        gx = np.empty((N, I), np.float32)
        self.lib.ref_backward_input(grad_out, state, scale, gx, Cc, I, O, N)
        return gx

    def matmul_m1(self, a, b):
        k, n = b.shape
        out = np.empty(n, np.float32)
        self.lib.ref_matmul_f32_m1(a, b, out, k, n)
        return out


def _get_port():
    path = os.path.join(_HERE, "liboracle.so")
    if not os.path.isfile(path):
        build(ref_tree="")
    return _Port(C.CDLL(path))


port = _get_port()
_reflib = _load(os.path.join(_HERE, "_ref", "libmotifcl_ref.so"))
ref = _Ref(_reflib) if _reflib is not None else None
