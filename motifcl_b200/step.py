"""Step driver for a stack of counter linears: forward, backward-to-input, weight gradient and
the fused counter update for every linear of a configuration, optionally data-parallel.

One training step of a counter linear is what MotifCL's autograd does around
nn::CounterStateLinear (src/nn/compact_counter.cpp:40-50,266-300): Y = X W^T at forward
time; at backward time dX from the PRE-update state, then the update.  Here the update is
the dense form (dW = dY^T X materialised once, then one fused kernel) because that is the
form whose gradient can be summed across data-parallel ranks.

Single GPU: one mcl_cuda_counter_linear_step per linear, spread over parallel lanes and
recorded into one batch.  Data parallel (see dp.py): the three products come from the
replicated 2-bit weights, the update runs on the local row shard after a reduce-scatter, and
the new 2-bit words and scales are all-gathered.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import dp
from .dp import shard_rows  # noqa: F401  (re-exported)
from .runtime import Context
from .synth import LinearShape


@dataclass
class Hyper:
    C: int = 11
    lr: float = 3e-3
    lr_scale: float = 0.0
    rms_beta: float = 0.9
    rms_eps: float = 1e-3


class CounterLinearState:
    """Device tensors of one counter linear on one rank (whole layer when world == 1)."""

    def __init__(self, shape: LinearShape, state: np.ndarray, scale: np.ndarray, v: np.ndarray,
                 device, rank: int = 0, world: int = 1):
        self.shape = shape
        O, I = shape.out_features, shape.in_features
        self.row_bytes = I // 4 * 3
        self.off, self.rows = shard_rows(O, rank, world)
        self.world = world
        self.state = torch.from_numpy(np.ascontiguousarray(state).reshape(-1)).to(device)
        self.scale = torch.from_numpy(np.ascontiguousarray(scale)).to(device)
        self.v = torch.from_numpy(np.ascontiguousarray(v)).to(device)
        self.packed2 = torch.zeros(O, I // 16, dtype=torch.int32, device=device)
        self.grad_w = torch.empty(O, I, dtype=torch.float32, device=device)
        self.y = None
        self.dx = None
        self.sharded = None     # dp.ShardedLinear once the stack knows its process group


class CounterStack:
    def __init__(self, ctx: Context, linears: list[CounterLinearState], hyper: Hyper, tokens: int,
                 group=None, lanes: int = 1, grouped: bool = False):
        """lanes > 1: the linears of a step are independent, so they are spread round-robin over
        `lanes` contexts (own stream, own workspace) that run side by side between a fork and a
        join on `ctx`."""
        self.ctx, self.linears, self.h, self.tokens = ctx, linears, hyper, tokens
        self.grouped = grouped      # single GPU: all linears through mcl_cuda_counter_linear_step_many
        self.lanes = [ctx] + [Context(ctx.device) for _ in range(max(0, lanes - 1))]
        self.group = group
        self.world = 1 if group is None else torch.distributed.get_world_size(group)
        self.rank = 0 if group is None else torch.distributed.get_rank(group)
        dev = linears[0].state.device
        for l in linears:
            O, I = l.shape.out_features, l.shape.in_features
            l.y = torch.empty(tokens, O, dtype=torch.float32, device=dev)
            l.dx = torch.empty(tokens, I, dtype=torch.float32, device=dev)
            if self.world > 1:
                # the 2-bit weights of the initial state are replicated; state and v keep only the shard
                ctx.counter_pack2(l.state, l.packed2, I, O, hyper.C)
                ctx.finish()
                l.sharded = dp.ShardedLinear(O, I, l.state.cpu(), l.scale.cpu(), l.v.cpu(), l.packed2.cpu(),
                                             self.rank, self.world, dev)
                l.sharded.grad_w = l.grad_w
                l.state, l.v, l.scale, l.packed2 = (l.sharded.state, l.sharded.v, l.sharded.scale,
                                                    l.sharded.packed2)
        self.step_index = 0
        self._batch = None
        self._batch_key = None
        self._step_word = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.world > 1:
            # The collectives are ordered against torch's CURRENT stream, the library's kernels against the
            # context's stream: they must be one and the same stream.
            cur = torch.cuda.current_stream(dev)
            if ctx.stream_handle != cur.cuda_stream:
                raise RuntimeError("data-parallel CounterStack: make the Context with Context.on_torch_stream() and keep "
                                   "that stream current (collectives and kernels must share one stream)")
            self._main = cur
            self._comm = torch.cuda.Stream(device=dev)         # reduce-scatter, shard update, all-gather
            self._comm_ctx = Context(ctx.device, self._comm.cuda_stream)
            self._ev_dw, self._ev_rows, self._ev_rs, self._ev_done = (torch.cuda.Event() for _ in range(4))
            self._rows_batch = self._upd_batch = None
            self._pending = False

    def set_gemm_mode(self, mode: str = "auto", act_terms: int = 3, grad_terms: int = 6):
        """Applies to every lane; recorded batches are dropped because they bake the old setting in."""
        for lane in self.lanes:
            lane.set_gemm_mode(mode, act_terms, grad_terms)
        for name in ("_batch", "_upd_batch"):
            b = getattr(self, name, None)
            if b is not None:
                b.close()
            setattr(self, name, None)
        self._batch_key = None

    def step(self, xs, dys, base_seed: int = 12345, recorded: bool = False):
        """xs[i]: [tokens, in_i], dys[i]: [tokens, out_i] device tensors.  One full step.

        recorded=True (single GPU): the first call runs eagerly (sizing the workspace) and
        records the same calls into one batch; later calls replay it -- one graph launch per
        step, as the reference submits one command buffer per step.  The per-step seed then
        comes from a device word that is bumped after every replay."""
        if self.world > 1:
            self._step_dp(xs, dys, (base_seed + self.step_index) & 0xFFFFFFFF)
            self.step_index += 1
            return
        if recorded:
            return self._step_recorded(xs, dys, base_seed)
        self._step_eager(xs, dys, (base_seed + self.step_index) & 0xFFFFFFFF)
        self.step_index += 1

    # -- single GPU --------------------------------------------------------------------------
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

    def _fork(self):
        for lane in self.lanes[1:]:
            self.ctx.lane_fork(lane)

    def _join(self):
        for lane in self.lanes[1:]:
            self.ctx.lane_join(lane)

    def _descs(self, xs, dys, update: bool, part: str = "all"):
        """part: "all" products, "dw" the weight gradients only, "rows" Y and dX only."""
        key = (tuple(t.data_ptr() for t in xs), tuple(t.data_ptr() for t in dys), update, part)
        cache = self.__dict__.setdefault("_desc_cache", {})
        if key not in cache:
            from .runtime import linear_descs
            cache[key] = linear_descs([
                dict(x=x, grad_out=dy, state=None if self.world > 1 else l.state, scale=l.scale, v=l.v,
                     y=l.y if part != "dw" else None, grad_x=l.dx if part != "dw" else None,
                     grad_w=l.grad_w if part != "rows" else None, packed2_out=l.packed2 if update else None,
                     packed2_in=l.packed2 if self.world > 1 else None,      # ranks compute from the replicated 2-bit words
                     in_features=l.shape.in_features, out_features=l.shape.out_features, batch=self.tokens,
                     update_rows=l.shape.out_features if update else 0, row_offset=0)
                for l, x, dy in zip(self.linears, xs, dys)])
        return cache[key]

    def _step_eager(self, xs, dys, seed):
        h, nl = self.h, len(self.lanes)
        if self.grouped:
            self.ctx.counter_linear_step_many(self._descs(xs, dys, True), h.C, h.lr, h.lr_scale, h.rms_beta, h.rms_eps,
                                              seed)
            return
        self._fork()
        for i, (l, x, dy) in enumerate(zip(self.linears, xs, dys)):
            O, I = l.shape.out_features, l.shape.in_features
            self.lanes[i % nl].counter_linear_step(x, dy, l.state, l.scale, l.v, l.y, l.dx, l.grad_w, l.packed2,
                                                   h.C, I, O, self.tokens, O, 0, h.lr, h.lr_scale, h.rms_beta,
                                                   h.rms_eps, seed)
        self._join()

    # -- data parallel -------------------------------------------------------------------------
    def _record(self, fn):
        """Run fn once eagerly (sizes workspaces), then record the same calls into a batch."""
        fn()
        self.ctx.finish()
        self.ctx.batch_begin()
        try:
            fn()
        finally:
            batch = self.ctx.batch_end()
        return batch

    def _step_dp(self, xs, dys, seed):
        """One data-parallel step with the reduce-scatter under the row products.

        main stream   A: weight gradients of all linears + split-K reduction (recorded batch)
                      B: digits from the replicated 2-bit words + Y and dX of all linears (recorded batch)
        comm stream   coalesced reduce-scatter of the gradients (starts when A is done, runs under B),
                      then -- once B has read the pre-update weights -- the fused update of the local row
                      shards (recorded batch, seeded through the device word) and the coalesced in-place
                      all-gather of the new 2-bit words and scales.
        The next step's A overlaps this step's update + all-gather; its B waits for them."""
        key = (tuple(t.data_ptr() for t in xs), tuple(t.data_ptr() for t in dys))
        main, comm = self._main, self._comm
        if self._batch is None or self._batch_key != key:
            # first step on these inputs: each part runs once eagerly (sizing the workspace; these are the
            # step's own products) and is recorded; nothing overlaps yet
            self.sync_streams()
            for name in ("_batch", "_rows_batch"):
                b = getattr(self, name)
                if b is not None:
                    b.close()
            if not getattr(self, "_ws_sized", False):
                # The context's workspace only grows, and a recorded batch holds addresses inside it: make the call with the
                # largest footprint (all three products at once) before anything is recorded.
                self.products_only(xs, dys)
                self.ctx.finish()
                self._ws_sized = True
            self._batch = self._record(lambda: self._products_part(xs, dys, "dw"))
            self._rows_batch = self._record(lambda: self._products_part(xs, dys, "rows"))
            self._batch_key = key
            self._ev_dw.record(main)
        else:
            if self._pending:
                main.wait_event(self._ev_rs)           # the previous reduce-scatter has read grad_w
            self._batch.launch()
            self._ev_dw.record(main)
            if self._pending:
                main.wait_event(self._ev_done)         # the previous step's 2-bit words and scales have landed
            self._rows_batch.launch()
        self._ev_rows.record(main)
        lins = [l.sharded for l in self.linears]
        with torch.cuda.stream(comm):
            comm.wait_event(self._ev_dw)
            dp.reduce_scatter_many(lins, self.group)
            self._ev_rs.record(comm)
            comm.wait_event(self._ev_rows)
            self._step_word.fill_(seed - (1 << 32) if seed >= (1 << 31) else seed)     # uint32 bits in an int32 word
            cctx = self._comm_ctx
            if self._upd_batch is None:
                cctx.set_seed_offset(self._step_word)
                try:
                    cctx.finish()
                    self.update_only(seed=0, ctx=cctx)          # this step's update (seed = 0 + word)
                    cctx.finish()
                    cctx.batch_begin()
                    try:
                        self.update_only(seed=0, ctx=cctx)
                    finally:
                        self._upd_batch = cctx.batch_end()
                finally:
                    cctx.set_seed_offset(None)
            else:
                self._upd_batch.launch()
            dp.all_gather_many(lins, self.group)
            self._ev_done.record(comm)
        self._pending = True

    def sync_streams(self):
        """Make the main stream wait for the communication stream's queued work (the tail of the last
        data-parallel step); callers that time or read results call this first."""
        if self.world > 1 and self._pending:
            self._main.wait_event(self._ev_done)
            self._pending = False

    def comm_launches(self) -> int:
        """Kernels this library launched on the communication stream's context so far (shard updates)."""
        return self._comm_ctx.launch_count if self.world > 1 else 0

    def _products_part(self, xs, dys, part):
        h = self.h
        self.ctx.counter_linear_step_many(self._descs(xs, dys, False, part), h.C, h.lr, h.lr_scale, h.rms_beta, h.rms_eps, 0)

    def step_linear(self, i: int, x, dy, seed: int):
        """The step of linear `i` alone on the main context (single GPU), for callers that
        pipeline host-to-device copies against compute linear by linear."""
        h, l = self.h, self.linears[i]
        O, I = l.shape.out_features, l.shape.in_features
        self.ctx.counter_linear_step(x, dy, l.state, l.scale, l.v, l.y, l.dx, l.grad_w, l.packed2, h.C, I, O,
                                     self.tokens, O, 0, h.lr, h.lr_scale, h.rms_beta, h.rms_eps, seed)

    # -- parts of a step, for per-kernel timing ---------------------------------------------------
    def products_only(self, xs, dys):
        """Y, dX and dW of every linear, no update (and no collectives)."""
        h, nl = self.h, len(self.lanes)
        if self.grouped:
            self.ctx.counter_linear_step_many(self._descs(xs, dys, False), h.C, h.lr, h.lr_scale, h.rms_beta, h.rms_eps, 0)
            return
        self._fork()
        for i, (l, x, dy) in enumerate(zip(self.linears, xs, dys)):
            O, I = l.shape.out_features, l.shape.in_features
            if self.world > 1:
                self.lanes[i % nl].ternary_linear_products(x, dy, l.packed2, l.scale, l.y, l.dx, l.grad_w, I, O,
                                                           self.tokens)
            else:
                self.lanes[i % nl].counter_linear_step(x, dy, l.state, l.scale, l.v, l.y, l.dx, l.grad_w, None,
                                                       h.C, I, O, self.tokens, 0, 0, h.lr, h.lr_scale, h.rms_beta,
                                                       h.rms_eps, 0)
        self._join()

    def update_only(self, seed: int = 777, ctx=None):
        """The fused update of every linear's local rows from the gradient already in place."""
        h = self.h
        ctx = ctx or self.ctx
        if self.grouped:
            if getattr(self, "_upd_descs", None) is None:
                from .runtime import update_descs
                ents = []
                for l in self.linears:
                    if self.world > 1:
                        sh = l.sharded
                        if sh.rows == 0:
                            continue
                        sl = slice(sh.off, sh.off + sh.rows)
                        ents.append(dict(state=sh.state, scale=sh.scale[sl], v=sh.v, grad_w=sh.gw_shard[:sh.rows],
                                         packed2_out=sh.packed2[sl], in_features=l.shape.in_features, rows=sh.rows,
                                         row_offset=sh.off))
                    else:
                        ents.append(dict(state=l.state, scale=l.scale, v=l.v, grad_w=l.grad_w, packed2_out=l.packed2,
                                         in_features=l.shape.in_features, rows=l.shape.out_features, row_offset=0))
                self._upd_descs = update_descs(ents)
                self._upd_keep = ents        # the sliced views must outlive the descriptor array
            if len(self._upd_descs):
                ctx.counter_update_dense_many(self._upd_descs, h.C, h.lr, h.lr_scale, h.rms_beta, h.rms_eps, seed)
            return
        for l in self.linears:
            I = l.shape.in_features
            if self.world > 1:
                sh = l.sharded
                sl = slice(sh.off, sh.off + sh.rows)
                ctx.counter_update_dense(sh.state, sh.scale[sl], sh.v, sh.gw_shard[:sh.rows], sh.packed2[sl], h.C,
                                              I, sh.rows, sh.off, h.lr, h.lr_scale, h.rms_beta, h.rms_eps, seed)
            else:
                ctx.counter_update_dense(l.state, l.scale, l.v, l.grad_w, l.packed2, h.C, I,
                                              l.shape.out_features, 0, h.lr, h.lr_scale, h.rms_beta, h.rms_eps, seed)


class WideStack:
    """Layer-by-layer step driver for stacks of WIDE counter linears (1B / 8B-scale shapes), where one
    linear is seconds of tensor-core work and activations of all layers would not fit beside each other:
    X, dY, Y, dX and the gradient live once per distinct SHAPE and are reused by every layer of that shape
    (synthetic activations, drawn on the device), state / scale / v / 2-bit words once per layer.

    Single GPU: mcl_cuda_counter_linear_step per layer.  Data parallel: per layer, the three products from
    the replicated 2-bit words on the main stream; on the communication stream the reduce-scatter of that
    layer's gradient along rows, the fused update of the local row shard and the in-place all-gather of
    its new 2-bit words and scales -- all under the NEXT layers' products (two gradient buffers per shape).
    """

    def __init__(self, ctx: Context, shapes: list[LinearShape], tokens: int, hyper: Hyper, device, sigma: float,
                 group=None, seed: int = 1):
        self.ctx, self.shapes, self.tokens, self.h = ctx, shapes, tokens, hyper
        self.group = group
        self.world = 1 if group is None else torch.distributed.get_world_size(group)
        self.rank = 0 if group is None else torch.distributed.get_rank(group)
        dev = self.dev = torch.device(device)
        g = torch.Generator(device=dev).manual_seed(seed)             # the same layers on every rank
        gx = torch.Generator(device=dev).manual_seed(seed + 1000 * (self.rank + 1))   # each rank its own tokens
        self.buf = {}
        nbuf = 2 if self.world > 1 else 1
        for sh in shapes:
            key = (sh.out_features, sh.in_features)
            if key in self.buf:
                continue
            O, I = key
            b = dict(x=torch.randn(tokens, I, device=dev, generator=gx),
                     dy=torch.randn(tokens, O, device=dev, generator=gx) * sigma,
                     y=torch.empty(tokens, O, device=dev), dx=torch.empty(tokens, I, device=dev),
                     gw=[torch.empty(O, I, device=dev) for _ in range(nbuf)], turn=0)
            if self.world > 1:
                if O % self.world:
                    raise ValueError("WideStack shards rows evenly: out_features must divide by the world size")
                b["gw_shard"] = [torch.empty(O // self.world, I, device=dev) for _ in range(nbuf)]
                b["free"] = [torch.cuda.Event() for _ in range(nbuf)]     # the buffer's reduce-scatter / update is done
                b["used"] = [False] * nbuf
            self.buf[key] = b
        self.layers = []
        for sh in shapes:
            O, I = sh.out_features, sh.in_features
            codes = torch.randint(0, 64, (O, I // 4, 4), device=dev, generator=g, dtype=torch.int32)
            w = codes[..., 0] | (codes[..., 1] << 6) | (codes[..., 2] << 12) | (codes[..., 3] << 18)
            st = torch.stack([w & 255, (w >> 8) & 255, (w >> 16) & 255], -1).to(torch.uint8).reshape(-1).contiguous()
            del codes, w
            scale = torch.full((O,), float(np.sqrt(np.float32(3.0) / np.float32(2.0 * I))), device=dev)
            p2 = torch.zeros(O, I // 16, dtype=torch.int32, device=dev)
            off, rows = shard_rows(O, self.rank, self.world)
            L = dict(O=O, I=I, scale=scale, packed2=p2, off=off, rows=rows, v=torch.zeros(rows, device=dev))
            if self.world > 1:
                ctx.counter_pack2(st, p2, I, O, hyper.C)
                ctx.finish()
                rb = I // 4 * 3
                L["state"] = st[off * rb:(off + rows) * rb].clone()
                L["views"] = (p2[off:off + rows], scale[off:off + rows])
                L["ready"] = torch.cuda.Event()       # this layer's new 2-bit words and scales have landed
                L["stepped"] = False
            else:
                L["state"] = st
            del st
            self.layers.append(L)
        self.step_index = 0
        if self.world > 1:
            cur = torch.cuda.current_stream(dev)
            if ctx.stream_handle != cur.cuda_stream:
                raise RuntimeError("data-parallel WideStack: make the Context with Context.on_torch_stream()")
            self._main = cur
            self._comm = torch.cuda.Stream(device=dev)
            self._comm_ctx = Context(ctx.device, self._comm.cuda_stream)
            self._ev_prod = [torch.cuda.Event() for _ in self.layers]
            self._ev_done = torch.cuda.Event()
            self._pending = False

    @property
    def weights(self) -> int:
        return sum(L["O"] * L["I"] for L in self.layers)

    def step(self, base_seed: int = 12345):
        h, T = self.h, self.tokens
        seed = (base_seed + self.step_index) & 0xFFFFFFFF
        self.step_index += 1
        if self.world == 1:
            for L in self.layers:
                b = self.buf[(L["O"], L["I"])]
                self.ctx.counter_linear_step(b["x"], b["dy"], L["state"], L["scale"], L["v"], b["y"], b["dx"], b["gw"][0],
                                             L["packed2"], h.C, L["I"], L["O"], T, L["O"], 0, h.lr, h.lr_scale, h.rms_beta,
                                             h.rms_eps, seed)
            return
        import torch.distributed as dist
        main, comm, cctx = self._main, self._comm, self._comm_ctx
        for li, L in enumerate(self.layers):
            b = self.buf[(L["O"], L["I"])]
            t = b["turn"]
            b["turn"] = (t + 1) % len(b["gw"])
            if b["used"][t]:
                main.wait_event(b["free"][t])       # the last reduce-scatter out of this gradient buffer is done
            if L["stepped"]:
                main.wait_event(L["ready"])         # the previous step's weights of this layer have landed
            self.ctx.ternary_linear_products(b["x"], b["dy"], L["packed2"], L["scale"], b["y"], b["dx"], b["gw"][t],
                                             L["I"], L["O"], T)
            self._ev_prod[li].record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(self._ev_prod[li])
                dist.reduce_scatter_tensor(b["gw_shard"][t], b["gw"][t], op=dist.ReduceOp.SUM, group=self.group)
                p2s, scs = L["views"]
                cctx.counter_update_dense(L["state"], scs, L["v"], b["gw_shard"][t], p2s, h.C, L["I"], L["rows"], L["off"],
                                          h.lr, h.lr_scale, h.rms_beta, h.rms_eps, seed)
                b["free"][t].record(comm)
                dist.all_gather_into_tensor(L["packed2"], p2s, group=self.group)
                dist.all_gather_into_tensor(L["scale"], scs, group=self.group)
                L["ready"].record(comm)
            b["used"][t] = True
            L["stepped"] = True
        self._ev_done.record(comm)
        self._pending = True

    def sync_streams(self):
        if self.world > 1 and self._pending:
            self._main.wait_event(self._ev_done)
            self._pending = False
