"""Step driver for a stack of counter linears: forward, backward-to-input, weight gradient and
the fused counter update for every linear of a configuration, optionally data-parallel.

One training step of a counter linear is what MotifCL's autograd does around
nn::CounterStateLinear (src/nn/compact_counter.cpp:40-50,266-300): Y = X W^T at forward
time; at backward time dX from the PRE-update state, then the update.  Here the update is
the dense form (dW = dY^T X materialised once, then one fused kernel) because that is the
form whose gradient can be summed across data-parallel ranks.

Data parallelism (not present in the reference; defined here): every rank holds the packed
state, scale and v of its contiguous block of weight rows plus replicated 2-bit weights and
scales.  Per linear: local dW = dY^T X -> reduce-scatter (sum) along rows -> fused update of
the local row shard with row_offset (so the random stream matches the unsharded layer) ->
all-gather of the shard's 2-bit words and scales.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .runtime import Context
from .synth import LinearShape


@dataclass
class Hyper:
    C: int = 11
    lr: float = 3e-3
    lr_scale: float = 0.0
    rms_beta: float = 0.9
    rms_eps: float = 1e-3


def shard_rows(out_features: int, rank: int, world: int) -> tuple[int, int]:
    """(row_offset, rows) of `rank`'s contiguous block; the first (out % world) ranks get one
    extra row so any out_features shards."""
    base, extra = divmod(out_features, world)
    rows = base + (1 if rank < extra else 0)
    off = rank * base + min(rank, extra)
    return off, rows


class CounterLinearState:
    """Device tensors of one counter linear on one rank."""

    def __init__(self, shape: LinearShape, state: np.ndarray, scale: np.ndarray, v: np.ndarray,
                 device, rank: int = 0, world: int = 1):
        self.shape = shape
        O, I = shape.out_features, shape.in_features
        self.row_bytes = I // 4 * 3
        self.off, self.rows = shard_rows(O, rank, world)
        # replicated: full packed state (forward/backward read it), full scale
        self.state = torch.from_numpy(np.ascontiguousarray(state).reshape(-1)).to(device)
        self.scale = torch.from_numpy(np.ascontiguousarray(scale)).to(device)
        self.v = torch.from_numpy(np.ascontiguousarray(v)).to(device)
        self.packed2 = torch.zeros(O, I // 16, dtype=torch.int32, device=device)
        self.grad_w = torch.empty(O, I, dtype=torch.float32, device=device)
        self.y = None
        self.dx = None


class CounterStack:
    def __init__(self, ctx: Context, linears: list[CounterLinearState], hyper: Hyper, tokens: int,
                 group=None, lanes: int = 1):
        """lanes > 1: the linears of a step are independent, so they are spread round-robin over
        `lanes` contexts (own stream, own workspace) that run side by side between a fork and a
        join on `ctx`."""
        self.ctx, self.linears, self.h, self.tokens = ctx, linears, hyper, tokens
        self.lanes = [ctx] + [Context(ctx.device) for _ in range(max(0, lanes - 1))]
        self.group = group
        self.world = 1 if group is None else torch.distributed.get_world_size(group)
        self.rank = 0 if group is None else torch.distributed.get_rank(group)
        dev = linears[0].state.device
        for l in linears:
            l.y = torch.empty(tokens, l.shape.out_features, dtype=torch.float32, device=dev)
            l.dx = torch.empty(tokens, l.shape.in_features, dtype=torch.float32, device=dev)
            if self.world > 1:
                l.gw_shard = torch.empty(max(l.rows, 1), l.shape.in_features, dtype=torch.float32, device=dev)
        self.step_index = 0
        self._batch = None
        self._batch_key = None
        self._step_word = torch.zeros(1, dtype=torch.int32, device=dev)

    def step(self, xs, dys, base_seed: int = 12345, recorded: bool = False):
        """xs[i]: [tokens, in_i], dys[i]: [tokens, out_i] device tensors.  One full step.

        recorded=True (single GPU): the first call runs eagerly (sizing the workspace), the
        second records the same calls into one batch, later ones replay it -- one graph launch
        per step, as the reference submits one command buffer per step.  The per-step seed then
        comes from a device word that is bumped after every replay."""
        if recorded and self.world == 1:
            return self._step_recorded(xs, dys, base_seed)
        self._step_eager(xs, dys, (base_seed + self.step_index) & 0xFFFFFFFF)
        self.step_index += 1

    def _step_recorded(self, xs, dys, base_seed):
        key = (tuple(t.data_ptr() for t in xs), tuple(t.data_ptr() for t in dys), base_seed)
        if self._batch is None or self._batch_key != key:
            if self._batch is not None:
                self._batch.close()
                self._batch = None
            self._step_word.fill_(self.step_index)
            for lane in self.lanes:
                lane.set_seed_offset(self._step_word)
            try:
                self._step_eager(xs, dys, base_seed)          # this call's step; also sizes the workspace
                self._step_word.add_(1)
                self.step_index += 1
                self.ctx.finish()
                self.ctx.batch_begin()
                try:
                    self._step_eager(xs, dys, base_seed)      # recorded, not run
                finally:
                    self._batch = self.ctx.batch_end()
            finally:
                for lane in self.lanes:
                    lane.set_seed_offset(None)
            self._batch_key = key
            return
        self._batch.launch()
        self._step_word.add_(1)
        self.step_index += 1

    def _step_eager(self, xs, dys, seed):
        ctx, h = self.ctx, self.h
        nl = len(self.lanes) if self.world == 1 else 1      # collectives stay on the main stream
        for lane in self.lanes[1:nl]:
            ctx.lane_fork(lane)
        for i, (l, x, dy) in enumerate(zip(self.linears, xs, dys)):
            O, I = l.shape.out_features, l.shape.in_features
            upd = O if self.world == 1 else 0     # data parallel: reduce grad_w first, then update the shard
            self.lanes[i % nl].counter_linear_step(x, dy, l.state, l.scale, l.v, l.y, l.dx, l.grad_w, l.packed2,
                                                   h.C, I, O, self.tokens, upd, 0, h.lr, h.lr_scale, h.rms_beta,
                                                   h.rms_eps, seed)
            if self.world > 1:
                self._dp_update(l, seed)
        for lane in self.lanes[1:nl]:
            ctx.lane_join(lane)

    def _dp_update(self, l: CounterLinearState, seed: int):
        import torch.distributed as dist
        ctx, h = self.ctx, self.h
        O, I = l.shape.out_features, l.shape.in_features
        if O % self.world == 0:
            dist.reduce_scatter_tensor(l.gw_shard, l.grad_w, op=dist.ReduceOp.SUM, group=self.group)
        else:   # ragged shards: all-reduce then slice (rare; none of the benchmark shapes)
            dist.all_reduce(l.grad_w, op=dist.ReduceOp.SUM, group=self.group)
            l.gw_shard.copy_(l.grad_w[l.off:l.off + l.rows])
        st = l.state[l.off * l.row_bytes:(l.off + l.rows) * l.row_bytes]
        p2 = l.packed2[l.off:l.off + l.rows]
        ctx.counter_update_dense(st, l.scale[l.off:l.off + l.rows], l.v[l.off:l.off + l.rows],
                                 l.gw_shard, p2, h.C, I, l.rows, l.off, h.lr, h.lr_scale, h.rms_beta,
                                 h.rms_eps, seed)
        if O % self.world == 0:
            dist.all_gather_into_tensor(l.packed2, p2.contiguous(), group=self.group)
            dist.all_gather_into_tensor(l.scale, l.scale[l.off:l.off + l.rows].contiguous(), group=self.group)
            dist.all_gather_into_tensor(l.state.view(O, l.row_bytes), st.view(l.rows, l.row_bytes).contiguous(),
                                        group=self.group)
        else:
            raise NotImplementedError("all-gather of ragged shards")
