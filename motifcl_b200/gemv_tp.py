"""Weight-sharded decode GEMV over several ranks: host-side plumbing only.

The reference has no multi-device code; this defines it for the M <= 16 ternary GEMV.  A layer
y[M, O] = scale[O] * (x[M, I] . T[O, I]^T) shards in the two classic ways:

    column parallel (split O)   rank r holds rows [off, off+rows) of the 2-bit words and of scale;
                                it computes its slice of y from the whole x: no communication
                                (w1, w3 and q of a transformer block; the result feeds a
                                row-parallel layer slice by slice)
    row parallel (split I)      rank r holds columns [c0, c1) of every row and the whole scale; it
                                computes scale * (x[:, c0:c1] . T[:, c0:c1]^T), a partial sum of the
                                full y; one all-reduce (sum) of [M, O] fp32 finishes it (w2, o)

The scale factors out of the sum, so scaled partials add up to the scaled result.  Column slices
are whole 64-weight blocks, the granularity of the tensor-core GEMV's k-tiles.

Everything here works on torch tensors of any device and any torch.distributed backend; the
arithmetic is injected as `gemv_fn(x, packed2, scale, y, M, in_features, out_features)`, so the
sharding logic is tested with gloo ranks on CPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .dp import shard_rows


def _sum_over_ranks(y: torch.Tensor, group=None):
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)


def shard_cols(in_features: int, rank: int, world: int, block: int = 64) -> tuple[int, int]:
    """(first column, columns) of `rank`'s slice of the input features, in whole blocks."""
    assert in_features % block == 0, "in_features must be a multiple of the column block"
    b0, nb = shard_rows(in_features // block, rank, world)
    return b0 * block, nb * block


class ColumnParallelGemv:
    """Rank-local slice [off, off+rows) of the output features."""

    def __init__(self, packed2_full: torch.Tensor, scale_full: torch.Tensor, in_features: int, rank: int, world: int):
        self.I, self.O = in_features, packed2_full.shape[0]
        self.off, self.rows = shard_rows(self.O, rank, world)
        self.packed2 = packed2_full[self.off:self.off + self.rows].contiguous()
        self.scale = scale_full[self.off:self.off + self.rows].contiguous()

    def __call__(self, gemv_fn, x: torch.Tensor, y_shard: torch.Tensor):
        """y_shard[M, rows] = this rank's output features."""
        if self.rows > 0:
            gemv_fn(x, self.packed2, self.scale, y_shard, x.shape[0], self.I, self.rows)
        return y_shard


class RowParallelGemv:
    """Rank-local slice [c0, c0+cols) of the input features; the result needs one all-reduce."""

    def __init__(self, packed2_full: torch.Tensor, scale_full: torch.Tensor, in_features: int, rank: int, world: int):
        self.I, self.O = in_features, packed2_full.shape[0]
        self.c0, self.cols = shard_cols(in_features, rank, world)
        self.packed2 = packed2_full[:, self.c0 // 16:(self.c0 + self.cols) // 16].contiguous()
        self.scale = scale_full.clone()

    def __call__(self, gemv_fn, x_shard: torch.Tensor, y: torch.Tensor, group=None, reducer=None):
        """x_shard[M, cols] = this rank's input features (what a column-parallel layer before it
        produced); y[M, O] = the full result on every rank.  With a `reducer` (peer.PeerReducer) the
        partial result is written into its shared buffer and summed by one kernel per rank instead of a
        collective call."""
        M = x_shard.shape[0]
        part = reducer.partial(M * self.O).view(M, self.O) if reducer is not None else y
        if self.cols > 0:
            gemv_fn(x_shard, self.packed2, self.scale, part, M, self.cols, self.O)
        else:
            part.zero_()
        if reducer is not None:
            reducer.allreduce(y, M * self.O)
        else:
            _sum_over_ranks(y, group)
        return y


class TensorParallelMlp:
    """w1, w3 column parallel -> elementwise gate on the local slice -> w2 row parallel (one all-reduce),
    the FFN of a Llama-style block at decode time."""

    def __init__(self, w1, s1, w3, s3, w2, s2, dim: int, ffn: int, rank: int, world: int):
        # the slice of the hidden features that w1/w3 produce must be the slice w2 consumes
        self.c0, self.cols = shard_cols(ffn, rank, world)
        sl = slice(self.c0, self.c0 + self.cols)
        self.dim, self.ffn = dim, ffn
        self.w1, self.s1 = w1[sl].contiguous(), s1[sl].contiguous()
        self.w3, self.s3 = w3[sl].contiguous(), s3[sl].contiguous()
        self.w2 = w2[:, self.c0 // 16:(self.c0 + self.cols) // 16].contiguous()
        self.s2 = s2.clone()

    def __call__(self, gemv_fn, x, h1, h3, y, group=None, reducer=None, gate=True):
        """x[M, dim] -> y[M, dim]; h1, h3: scratch [M, cols].  gate=False leaves the elementwise gate out (a sweep
        that times the matrix products alone).  reducer: see RowParallelGemv."""
        M = x.shape[0]
        part = reducer.partial(M * self.dim).view(M, self.dim) if reducer is not None else y
        if self.cols > 0:
            gemv_fn(x, self.w1, self.s1, h1, M, self.dim, self.cols)
            gemv_fn(x, self.w3, self.s3, h3, M, self.dim, self.cols)
            if gate:
                h1.copy_(torch.nn.functional.silu(h1) * h3)
            gemv_fn(h1, self.w2, self.s2, part, M, self.cols, self.dim)
        else:
            part.zero_()
        if reducer is not None:
            reducer.allreduce(y, M * self.dim)
        else:
            _sum_over_ranks(y, group)
        return y
