"""Tensor-parallel decode GEMV on CPU ranks (gloo, world size 2 and 3): column-parallel slices,
row-parallel partial sums with their all-reduce, and the FFN composition.  The per-rank arithmetic
is the CPU checker standing in for the CUDA GEMV, so the test pins the sharding logic alone."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from motifcl_b200 import gemv_tp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _weights(O, I, seed):
    rng = np.random.default_rng(seed)
    p2 = rng.integers(0, 2 ** 32, size=(O, I // 16), dtype=np.uint64).astype(np.uint32)
    # fields 0..2 only (t in {-1, 0, 1}); clear field value 3
    both = (p2 >> 1) & p2 & np.uint32(0x55555555)
    p2 = p2 & ~(both | (both << 1))
    return p2.view(np.int32), rng.uniform(0.02, 0.2, O).astype(np.float32)


def _oracle_gemv():
    import oracle

    def fn(x, p2, sc, y, M, I, O):
        out = oracle.port.ternary_gemv(np.ascontiguousarray(x.numpy()), np.ascontiguousarray(p2.numpy()).view(np.uint32), sc.numpy())
        y.copy_(torch.from_numpy(np.asarray(out, dtype=np.float32).reshape(M, O)))
    return fn


def _worker(rank, world, port, M, dim, ffn, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    fn = _oracle_gemv()
    w1, s1 = _weights(ffn, dim, 1)
    w3, s3 = _weights(ffn, dim, 2)
    w2, s2 = _weights(dim, ffn, 3)
    x = torch.from_numpy(np.random.default_rng(9).standard_normal((M, dim)).astype(np.float32))
    t = torch.from_numpy
    # column parallel alone
    col = gemv_tp.ColumnParallelGemv(t(w1), t(s1), dim, rank, world)
    y_col = col(fn, x, torch.empty(M, col.rows))
    # row parallel alone: every rank feeds its slice of a common hidden vector
    h = torch.from_numpy(np.random.default_rng(10).standard_normal((M, ffn)).astype(np.float32))
    row = gemv_tp.RowParallelGemv(t(w2), t(s2), ffn, rank, world)
    y_row = row(fn, h[:, row.c0:row.c0 + row.cols].contiguous(), torch.empty(M, dim))
    # the FFN
    mlp = gemv_tp.TensorParallelMlp(t(w1), t(s1), t(w3), t(s3), t(w2), t(s2), dim, ffn, rank, world)
    y_mlp = mlp(fn, x, torch.empty(M, mlp.cols), torch.empty(M, mlp.cols), torch.empty(M, dim))
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), y_col=y_col.numpy(), off=col.off, rows=col.rows,
             y_row=y_row.numpy(), y_mlp=y_mlp.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("world,M,dim,ffn", [(2, 3, 128, 384), (3, 1, 192, 320)])
def test_tensor_parallel_gemv_equals_unsharded(tmp_path, orc, world, M, dim, ffn):
    mp.spawn(_worker, args=(world, _free_port(), M, dim, ffn, str(tmp_path)), nprocs=world, join=True)
    w1, s1 = _weights(ffn, dim, 1)
    w3, s3 = _weights(ffn, dim, 2)
    w2, s2 = _weights(dim, ffn, 3)
    x = np.random.default_rng(9).standard_normal((M, dim)).astype(np.float32)
    h = np.random.default_rng(10).standard_normal((M, ffn)).astype(np.float32)
    g = lambda a, p2, sc, I, O: np.asarray(orc.ternary_gemv(np.ascontiguousarray(a), p2.view(np.uint32), sc), np.float32).reshape(M, O)
    y1 = g(x, w1, s1, dim, ffn)
    y3 = g(x, w3, s3, dim, ffn)
    y_row = g(h, w2, s2, ffn, dim)
    hid = (y1 / (1.0 + np.exp(-y1.astype(np.float64)))).astype(np.float32) * y3
    y_mlp = g(hid, w2, s2, ffn, dim)
    covered = 0
    for r in range(world):
        d = np.load(tmp_path / f"r{r}.npz")
        off, rows = int(d["off"]), int(d["rows"])
        assert np.array_equal(d["y_col"], y1[:, off:off + rows])          # slices of the same sums: bit-equal
        covered += rows
        # partial sums are added in a different order than one long sum: tolerance, not equality
        assert np.linalg.norm(d["y_row"] - y_row) <= 1e-5 * np.linalg.norm(y_row)
        assert np.linalg.norm(d["y_mlp"] - y_mlp) <= 1e-4 * np.linalg.norm(y_mlp)
    assert covered == ffn


def test_shard_cols_are_whole_blocks():
    for I in (64, 320, 4096, 14336):
        for world in (1, 2, 3, 8):
            parts = [gemv_tp.shard_cols(I, r, world) for r in range(world)]
            assert parts[0][0] == 0 and sum(p[1] for p in parts) == I
            assert all(p[0] % 64 == 0 and p[1] % 64 == 0 for p in parts)
