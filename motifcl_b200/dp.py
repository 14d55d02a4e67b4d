"""Row-sharded data parallelism for counter linears: host-side plumbing only.

The reference has no multi-device code; this defines it.  A counter update has no coupling
between weight rows (MotifCL kernels/compact_counter.cl:67-99,113-137) and its random stream
depends only on the global element index and the seed (:127), so a layer shards by
contiguous row blocks:

    replicated on every rank   2-bit packed weights, per-row scale  (what Y and dX need)
    sharded by rows            6-bit counter state, v, and the reduced weight gradient

Per linear and step: local dW = dY^T X  ->  reduce-scatter (sum) along rows  ->  fused
update of the local shard, told its row_offset so that it hashes like the unsharded layer
->  all-gather of the shard's 2-bit words and scales.  Summing (not averaging) makes dW equal
to what one device would see for all ranks' tokens.

Everything here works on torch tensors of any device and any torch.distributed backend, so
the logic is tested with gloo ranks on CPU; the arithmetic is injected as `update_fn`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(out_features: int, rank: int, world: int) -> tuple[int, int]:
    """(row_offset, rows) of `rank`'s contiguous block; the first (out % world) ranks get one
    extra row, so any out_features shards."""
    base, extra = divmod(out_features, world)
    rows = base + (1 if rank < extra else 0)
    off = rank * base + min(rank, extra)
    return off, rows


def max_shard_rows(out_features: int, world: int) -> int:
    return (out_features + world - 1) // world


def reduce_scatter_rows(grad_w: torch.Tensor, out: torch.Tensor, rank: int, world: int, group=None):
    """out[:rows] = rows [off, off+rows) of sum over ranks of grad_w ([O, I])."""
    O = grad_w.shape[0]
    off, rows = shard_rows(O, rank, world)
    if O % world == 0:
        dist.reduce_scatter_tensor(out[:rows], grad_w, op=dist.ReduceOp.SUM, group=group)
    else:   # ragged blocks: sum everywhere, keep the local block
        dist.all_reduce(grad_w, op=dist.ReduceOp.SUM, group=group)
        out[:rows].copy_(grad_w[off:off + rows])
    return out[:rows]


def all_gather_rows(full: torch.Tensor, rank: int, world: int, group=None, scratch=None):
    """Every rank owns rows [off, off+rows) of `full` ([O, ...]); afterwards all ranks hold all
    rows.  Even blocks are gathered straight into `full` from a copy of the rank's own block (the
    per-layer helper; the coalesced step gathers in place without that copy); ragged blocks go through
    a padded scratch."""
    O = full.shape[0]
    off, rows = shard_rows(O, rank, world)
    if O % world == 0:
        dist.all_gather_into_tensor(full, full[off:off + rows].clone(), group=group)
        return
    m = max_shard_rows(O, world)
    pad = torch.zeros((m,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
    pad[:rows].copy_(full[off:off + rows])
    if scratch is None:
        scratch = torch.empty((world * m,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
    dist.all_gather_into_tensor(scratch, pad, group=group)
    for r in range(world):
        o, n = shard_rows(O, r, world)
        full[o:o + n].copy_(scratch[r * m:r * m + n])


class ShardedLinear:
    """Tensors of one counter linear on one data-parallel rank."""

    def __init__(self, out_features: int, in_features: int, state_full, scale_full, v_full, packed2_full,
                 rank: int, world: int, device):
        self.O, self.I = out_features, in_features
        self.rank, self.world = rank, world
        self.off, self.rows = shard_rows(out_features, rank, world)
        rb = in_features // 4 * 3
        st = torch.as_tensor(state_full).reshape(out_features, rb)
        self.state = st[self.off:self.off + self.rows].contiguous().reshape(-1).to(device)   # shard
        self.v = torch.as_tensor(v_full)[self.off:self.off + self.rows].contiguous().to(device)  # shard
        self.scale = torch.as_tensor(scale_full).clone().to(device)                              # replicated
        self.packed2 = torch.as_tensor(packed2_full).clone().to(device)                          # replicated
        self.grad_w = torch.zeros(out_features, in_features, dtype=torch.float32, device=device)
        self.gw_shard = torch.zeros(max_shard_rows(out_features, world), in_features, dtype=torch.float32,
                                    device=device)


def exchange_and_update(lin: ShardedLinear, update_fn, seed: int, group=None):
    """The collective half of a data-parallel step for one linear whose local grad_w is ready.

    update_fn(state_shard, scale_shard, v_shard, grad_shard, packed2_shard, rows, row_offset, seed)
    updates its arguments in place (the fused counter update on `rows` rows)."""
    gw = reduce_scatter_rows(lin.grad_w, lin.gw_shard, lin.rank, lin.world, group)
    sl = slice(lin.off, lin.off + lin.rows)
    if lin.rows > 0:
        update_fn(lin.state, lin.scale[sl], lin.v, gw, lin.packed2[sl], lin.rows, lin.off, seed)
    all_gather_rows(lin.packed2, lin.rank, lin.world, group)
    all_gather_rows(lin.scale, lin.rank, lin.world, group)


def _coalescable(lins, group) -> bool:
    return dist.get_backend(group) == "nccl" and all(l.O % l.world == 0 for l in lins)


def reduce_scatter_many(lins, group=None):
    """gw_shard[:rows] of every linear = its rows of the rank-summed grad_w; one coalesced NCCL
    collective when all layers divide evenly."""
    if not _coalescable(lins, group):
        for l in lins:
            reduce_scatter_rows(l.grad_w, l.gw_shard, l.rank, l.world, group)
        return
    for l in lins:
        if getattr(l, "_scatter_view", None) is None:
            l._scatter_view = l.gw_shard[:l.rows]
    with dist._coalescing_manager(group=group, device=lins[0].grad_w.device, async_ops=False):
        for l in lins:
            dist.reduce_scatter_tensor(l._scatter_view, l.grad_w, op=dist.ReduceOp.SUM, group=group)


def all_gather_many(lins, group=None):
    """Replicate every linear's freshly updated 2-bit words and scales."""
    if not _coalescable(lins, group):
        for l in lins:
            all_gather_rows(l.packed2, l.rank, l.world, group)
            all_gather_rows(l.scale, l.rank, l.world, group)
        return
    # In place: with equal shards a rank's rows already sit at rank * rows of the full tensor, which is where
    # NCCL's all-gather expects the send buffer of an in-place call; no copies, and the views are made once.
    for l in lins:
        if getattr(l, "_gather_views", None) is None:
            l._gather_views = (l.packed2[l.off:l.off + l.rows], l.scale[l.off:l.off + l.rows])
    with dist._coalescing_manager(group=group, device=lins[0].grad_w.device, async_ops=False):
        for l in lins:
            p2s, scs = l._gather_views
            dist.all_gather_into_tensor(l.packed2, p2s, group=group)
            dist.all_gather_into_tensor(l.scale, scs, group=group)


def exchange_and_update_many(lins, update_fn, seed: int, group=None):
    """exchange_and_update for a whole stack: reduce-scatter all, update all shards, gather all."""
    reduce_scatter_many(lins, group)
    for l in lins:
        if l.rows > 0:
            sl = slice(l.off, l.off + l.rows)
            update_fn(l.state, l.scale[sl], l.v, l.gw_shard[:l.rows], l.packed2[sl], l.rows, l.off, seed)
    all_gather_many(lins, group)
