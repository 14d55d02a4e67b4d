"""Data-parallel plumbing on CPU ranks (gloo, world size 2 and 3): row sharding, reduce-scatter,
row_offset / seed hand-off and all-gather.  The per-shard arithmetic is the CPU checker standing
in for the CUDA update, so the test pins the sharding logic alone: the sharded result must be
bit-identical to ONE unsharded update fed the summed gradient."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from motifcl_b200 import codec, dp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _case(O, I, seed):
    rng = np.random.default_rng(seed)
    state = codec.pack_codes(rng.integers(0, 64, size=(O, I)).astype(np.uint8)).reshape(-1)
    scale = rng.uniform(0.02, 0.2, O).astype(np.float32)
    v = rng.uniform(1e-4, 1e-2, O).astype(np.float32)
    return state, scale, v


def _rank_grad(O, I, seed, rank):
    # multiples of 2^-12 in a small range: sums over ranks are exact in fp32, so the result does
    # not depend on the order in which the backend adds the ranks' gradients
    g = 0.1 * np.random.default_rng(seed * 100 + rank).standard_normal((O, I))
    return (np.round(g * 4096.0) / 4096.0).astype(np.float32)


HY = (0.3, 0.05, 0.9, 1e-3)


def _worker(rank, world, port, O, I, seed, out_dir):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    state, scale, v = _case(O, I, seed)
    p2 = oracle.port.pack2(state, 11, I, O).view(np.int32)
    lin = dp.ShardedLinear(O, I, state, scale, v, p2, rank, world, "cpu")
    lin.grad_w.copy_(torch.from_numpy(_rank_grad(O, I, seed, rank)))

    def update_fn(st, sc, vv, gw, p2s, rows, off, sd):
        ns, nsc, nv, np2 = oracle.port.update_dense(st.numpy(), sc.numpy().copy(), vv.numpy(), gw.numpy(), 11, I,
                                                    rows, off, *HY, sd)
        st.copy_(torch.from_numpy(ns)); sc.copy_(torch.from_numpy(nsc)); vv.copy_(torch.from_numpy(nv))
        p2s.copy_(torch.from_numpy(np2.view(np.int32)))

    for step in range(2):     # two steps: the gathered scales feed the next step's shards
        dp.exchange_and_update(lin, update_fn, 777 + step)
        lin.grad_w.copy_(torch.from_numpy(_rank_grad(O, I, seed + 1, rank)))
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), state=lin.state.numpy(), v=lin.v.numpy(),
             scale=lin.scale.numpy(), packed2=lin.packed2.numpy(), off=lin.off, rows=lin.rows)
    dist.destroy_process_group()


@pytest.mark.parametrize("world,O,I", [(2, 48, 64), (2, 35, 32), (3, 50, 48)])
def test_sharded_update_equals_unsharded(tmp_path, orc, world, O, I):
    seed = O * 7 + world
    mp.spawn(_worker, args=(world, _free_port(), O, I, seed, str(tmp_path)), nprocs=world, join=True)
    # single-device truth: summed gradient, whole layer
    state, scale, v = _case(O, I, seed)
    for step in range(2):
        gsum = np.zeros((O, I), np.float32)
        for r in range(world):
            gsum = gsum + _rank_grad(O, I, seed + step, r)
        state, scale, v, p2 = orc.update_dense(state, scale, v, gsum, 11, I, O, 0, *HY, 777 + step)
    rb = I // 4 * 3
    covered = 0
    for r in range(world):
        d = np.load(tmp_path / f"r{r}.npz")
        off, rows = int(d["off"]), int(d["rows"])
        assert (off, rows) == dp.shard_rows(O, r, world)
        assert np.array_equal(d["state"], state[off * rb:(off + rows) * rb])        # shard, bit-exact
        assert np.array_equal(d["v"].view(np.uint32), v[off:off + rows].view(np.uint32))
        assert np.array_equal(d["scale"].view(np.uint32), scale.view(np.uint32))     # replicated, whole layer
        assert np.array_equal(d["packed2"].view(np.uint32), p2)
        covered += rows
    assert covered == O


def test_shard_rows_partition():
    for O in (1, 7, 35, 288, 1024):
        for world in (1, 2, 3, 8):
            blocks = [dp.shard_rows(O, r, world) for r in range(world)]
            assert blocks[0][0] == 0 and sum(b[1] for b in blocks) == O
            for a, b in zip(blocks, blocks[1:]):
                assert a[0] + a[1] == b[0]
            assert max(b[1] for b in blocks) == dp.max_shard_rows(O, world)
