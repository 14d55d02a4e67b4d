"""Host-side mirror of MotifCL's nn::CounterStateLinear for the CUDA path.

Same constructor arguments, member names and call order as the reference class
(MotifCL include/motifcl/nn/compact_counter.hpp:16-60, src/nn/compact_counter.cpp:55-300),
so tests written against it read like the reference's own.  All arithmetic happens in the
CUDA library behind the C ABI; this class only holds the three persistent tensors and the
hyper-parameters, and sequences calls.
"""
from __future__ import annotations

import numpy as np
import torch

from . import codec
from .runtime import Context


def initial_ternary(seed: int, n: int) -> np.ndarray:
    """The digits std::uniform_int_distribution<int>(-1, 1) draws from std::mt19937(seed) in
    the reference constructor (src/nn/compact_counter.cpp:67-72, libstdc++): each 32-bit
    draw r gives floor(3 r / 2^32) - 1, and a draw of exactly 0 is rejected and redrawn."""
    rs = np.random.RandomState(seed & 0xFFFFFFFF)
    out = np.empty(n, np.int8)
    filled = 0
    while filled < n:
        raw = rs.randint(0, 2 ** 32, size=n - filled, dtype=np.uint64)
        raw = raw[raw != 0]
        out[filled:filled + raw.size] = ((raw * np.uint64(3)) >> np.uint64(32)).astype(np.int8) - 1
        filled += raw.size
    return out


class CounterStateLinear:
    """Ternary finite-state counter linear layer: y = x @ (scale . t)^T, self-updating."""

    def __init__(self, ctx: Context, in_features: int, out_features: int, C: int = 11,
                 lr: float = 3e-3, lr_scale: float = 0.0, init_gain: float = 1.0,
                 rms_beta: float = 0.9, rms_eps: float = 1e-3, seed: int = 12345):
        if in_features <= 0 or out_features <= 0:
            raise ValueError("CounterStateLinear requires positive dimensions")
        if 3 * (2 * C - 1) > 64:
            raise ValueError("C too large for 6-bit packed state encoding")
        if in_features % 4 != 0:
            raise ValueError("CounterStateLinear requires in_features divisible by 4 (6-bit packing)")
        self.ctx = ctx
        self.in_features, self.out_features, self.C = in_features, out_features, C
        self.lr, self.lr_scale = float(lr), float(lr_scale)
        self.rms_beta, self.rms_eps = float(rms_beta), float(rms_eps)
        self._seed = seed & 0xFFFFFFFF
        self.training = True
        dev = torch.device("cuda", ctx.device)
        t = initial_ternary(seed, out_features * in_features).reshape(out_features, in_features)
        st = codec.pack_codes(codec.encode(t, np.zeros_like(t), C))
        self.state = torch.from_numpy(st.reshape(-1)).to(dev)                      # U8 [out*in/4*3]
        s0 = np.float32(init_gain) * np.sqrt(np.float32(3.0) / (np.float32(2.0) * np.float32(in_features)))
        self.scale = torch.full((out_features,), float(s0), dtype=torch.float32, device=dev)
        self.v = torch.zeros(out_features, dtype=torch.float32, device=dev)

    # -- reference API -------------------------------------------------------------------
    def next_seed(self) -> int:
        s = self._seed
        self._seed = (self._seed + 1) & 0xFFFFFFFF
        return s

    def set_training(self, t: bool):
        self.training = bool(t)

    def set_lr(self, lr: float):
        self.lr = float(lr)

    def decode_weight(self) -> torch.Tensor:
        w = torch.empty(self.out_features, self.in_features, dtype=torch.float32, device=self.state.device)
        self.ctx.counter_decode_weight(self.state, self.scale, w, self.in_features, self.out_features, self.C)
        return w

    def pack2(self) -> torch.Tensor:
        p = torch.empty(self.out_features, self.in_features // 16, dtype=torch.int32, device=self.state.device)
        self.ctx.counter_pack2(self.state, p, self.in_features, self.out_features, self.C)
        return p

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype != torch.float32 or x.dim() != 2:
            raise ValueError("CounterStateLinear expects rank-2 f32 input")
        if x.shape[1] != self.in_features:
            raise ValueError("CounterStateLinear input feature mismatch")
        x = x.contiguous()
        y = torch.empty(x.shape[0], self.out_features, dtype=torch.float32, device=x.device)
        self.ctx.counter_forward(x, self.state, self.scale, y, x.shape[0], self.in_features,
                                 self.out_features, self.C)
        return y

    def backward_input_from_state(self, grad_out: torch.Tensor) -> torch.Tensor:
        grad_out = grad_out.contiguous()
        gx = torch.empty(grad_out.shape[0], self.in_features, dtype=torch.float32, device=grad_out.device)
        self.ctx.counter_backward_input(self.state, self.scale, grad_out, gx, grad_out.shape[0],
                                        self.in_features, self.out_features, self.C)
        return gx

    def apply_update_seed(self, grad_w: torch.Tensor, seed: int, packed2_out: torch.Tensor | None = None):
        self.ctx.counter_update_dense(self.state, self.scale, self.v, grad_w.contiguous(), packed2_out,
                                      self.C, self.in_features, self.out_features, 0, self.lr,
                                      self.lr_scale, self.rms_beta, self.rms_eps, seed)

    def apply_update_backward(self, grad_out: torch.Tensor, x: torch.Tensor, seed: int,
                              packed2_out: torch.Tensor | None = None):
        self.ctx.counter_update_fused(self.state, self.scale, self.v, grad_out.contiguous(),
                                      x.contiguous(), packed2_out, self.C, self.in_features,
                                      self.out_features, x.shape[0], self.lr, self.lr_scale,
                                      self.rms_beta, self.rms_eps, seed)

    # -- several micro-batches per counter update -------------------------------------------
    # MotifCL updates the counters after every backward pass and names the small effective batch as the main
    # quality gap of its pretraining run (docs/TERNARY15M_PRETRAIN_RESULTS.md:90-97).  Here the weight gradient
    # of several micro-batches can be summed (fp32, in the order of the calls) before ONE update; the update
    # itself is the reference's dense one (apply_update_seed), so given the summed gradient its result is
    # bit-identical to the reference's.
    def accumulate_backward(self, x: torch.Tensor, grad_out: torch.Tensor, need_grad_x: bool = True):
        """grad_x from the current state; dW = grad_out^T x is added to the layer's gradient buffer."""
        gx = self.backward_input_from_state(grad_out) if need_grad_x else None
        x, grad_out = x.contiguous(), grad_out.contiguous()
        n = self.out_features * self.in_features
        first = getattr(self, "_acc", None) is None
        if first:
            self._acc = torch.empty(self.out_features, self.in_features, dtype=torch.float32, device=x.device)
            self._acc_tmp = torch.empty_like(self._acc)
            self._acc_count = 0
        dst = self._acc if self._acc_count == 0 else self._acc_tmp
        self.ctx.matmul_f32(grad_out, x, dst, self.out_features, x.shape[0], self.in_features, trans_a=True)
        if self._acc_count > 0:
            self.ctx.eltwise(0, self._acc, self._acc_tmp, self._acc, n)     # MCL_CUDA_ELT_ADD
        self._acc_count += 1
        return gx

    def apply_accumulated(self, seed: int, packed2_out: torch.Tensor | None = None) -> int:
        """One counter update with the summed gradient; returns how many micro-batches it covered."""
        count = getattr(self, "_acc_count", 0)
        if count == 0:
            raise RuntimeError("apply_accumulated: no gradient has been accumulated")
        self.apply_update_seed(self._acc, seed, packed2_out)
        self._acc_count = 0
        return count

    def backward(self, x: torch.Tensor, grad_out: torch.Tensor, seed: int, need_grad_x: bool = True):
        """What CounterBackwardNode::backward does (src/nn/compact_counter.cpp:40-50): grad_x
        from the PRE-update state, then the fused update."""
        gx = self.backward_input_from_state(grad_out) if need_grad_x else None
        self.apply_update_backward(grad_out, x, seed)
        return gx
