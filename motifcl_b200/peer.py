"""One-shot sum of small fp32 results over the GPUs of a node, for tensor-parallel decode.

Every rank owns one buffer that all ranks map (CUDA IPC through the library: `mcl_cuda_peer_buffer_*`): 64 flag words
followed by two partial-result areas.  A row-parallel GEMV writes its partial [M, out] straight into `partial(n)`;
`allreduce(out, n)` then launches ONE kernel per rank that announces the partial to the peers, waits (with a limit)
for theirs and adds all of them in rank order with plain peer loads (`mcl_cuda_peer_allreduce_f32`).  No collective
library call is on the path, so a whole decode sweep can be recorded as one batch.

The handles travel once, at construction, through torch.distributed (any backend).  One process per GPU.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

FLAG_WORDS = 64


class _RawCuda:
    """A device range as an object torch can wrap without copying."""

    def __init__(self, ptr: int, floats: int):
        self.__cuda_array_interface__ = {"shape": (floats,), "typestr": "<f4", "data": (ptr, False), "version": 3}


class PeerReducer:
    def __init__(self, ctx, n_max: int, group=None):
        self.ctx, self.group = ctx, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_max = (n_max + 3) // 4 * 4
        self.seq = 0
        lib, h = ctx._lib, ctx._ctx
        own = C.c_void_p()
        handle = C.create_string_buffer(64)
        ctx._check(lib.mcl_cuda_peer_buffer_create(h, (FLAG_WORDS + 2 * self.n_max) * 4, C.byref(own), handle))
        self._own = own.value
        self._opened = []
        ptrs = [0] * self.world
        ptrs[self.rank] = self._own
        if self.world > 1:
            dev = torch.device("cuda", ctx.device)
            mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).to(dev)
            every = [torch.empty(64, dtype=torch.uint8, device=dev) for _ in range(self.world)]
            dist.all_gather(every, mine, group=group)
            failure = None
            for r in range(self.world):
                if r == self.rank:
                    continue
                p = C.c_void_p()
                try:
                    ctx._check(lib.mcl_cuda_peer_buffer_open(h, bytes(every[r].cpu().numpy().tobytes()), C.byref(p)))
                except Exception as exc:      # noqa: BLE001  -- reported below, once every rank knows
                    failure = exc
                    break
                self._opened.append(p.value)
                ptrs[r] = p.value
            # the ranks agree on the outcome, so that a rank that could not map a peer does not leave the others waiting
            ok = torch.tensor([0 if failure else 1], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self.close()
                raise RuntimeError(f"peer buffers could not be mapped on every rank ({failure})")
        vp = C.c_void_p * self.world
        self._flags = vp(*ptrs)
        self._data = vp(*[p + FLAG_WORDS * 4 for p in ptrs])
        self._view = torch.as_tensor(_RawCuda(self._own + FLAG_WORDS * 4, 2 * self.n_max), device=torch.device("cuda", ctx.device))

    def partial(self, n: int) -> torch.Tensor:
        """Where this rank's partial result of the NEXT allreduce goes (n floats)."""
        par = (self.seq + 1) & 1
        return self._view[par * self.n_max: par * self.n_max + n]

    def allreduce(self, out: torch.Tensor, n: int):
        """out[:n] = sum over the ranks of their `partial(n)`, the same bits on every rank.  Calls alternate between the
        two partial areas; a recorded batch must hold an EVEN number of them, so that its replays alternate too."""
        assert n % 4 == 0 and n <= self.n_max and out.is_contiguous() and out.dtype == torch.float32
        self.seq += 1
        self.ctx._check(self.ctx._lib.mcl_cuda_peer_allreduce_f32(
            self.ctx._ctx, self._data, self._flags, self.rank, self.world, n, self.n_max, self.seq & 1,
            C.c_void_p(out.data_ptr())))

    def close(self):
        if self._own is None:
            return
        lib, h = self.ctx._lib, self.ctx._ctx
        for p in self._opened:
            lib.mcl_cuda_peer_buffer_close(h, C.c_void_p(p))
        self._opened = []
        if self.world > 1:
            dist.barrier(self.group)       # every peer has unmapped before the owner frees
        lib.mcl_cuda_peer_buffer_destroy(h, C.c_void_p(self._own))
        self._own = None
