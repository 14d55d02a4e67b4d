"""The allocation-free fused update (mcl_cuda_counter_update_fused_static), checked against the
ordinary entry point.  Some callers of this library may not allocate device memory while they
run (all memory handed to their own arena at start-up, or a latency-critical loop where an
allocation would stall the device); for them the library keeps the gradient row tile in a
fixed 4 MiB array of its own.  This file is collected last on purpose: if it fails under -x,
every other test has already run."""
import ctypes

import numpy as np
import pytest
import torch

from cases import all_cases
from motifcl_b200 import lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CASES = {c["name"]: c for c in all_cases()}


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def test_static_update_equals_ordinary_update_twice_in_a_row(ctx):
    L = lib()
    stream = torch.cuda.current_stream(0).cuda_stream
    for name, seeds in (("cfg1_rebase", (999, 1000)), ("wide", (7, 8)), ("fused_witness", (777, 778))):
        c = CASES[name]
        N, I, O, C = c["N"], c["I"], c["O"], c["C"]
        x, dy = _t(c["x"]), _t(c["dy"])
        a = [_t(c["state"]), _t(c["scale"]), _t(c["v"])]      # ordinary entry point
        b = [_t(c["state"]), _t(c["scale"]), _t(c["v"])]      # allocation-free entry point
        want_p2 = I % 16 == 0
        pa = torch.zeros(O, max(I // 16, 1), dtype=torch.int32, device=DEV) if want_p2 else None
        pb = torch.zeros(O, max(I // 16, 1), dtype=torch.int32, device=DEV) if want_p2 else None
        ctx.set_gemm_mode("exact")
        try:
            for seed in seeds:      # two calls in a row: the second starts from the first's state
                ctx.counter_update_fused(a[0], a[1], a[2], dy, x, pa, C, I, O, N, c["lr"], c["lr_scale"],
                                         c["beta"], c["eps"], seed)
                rc = L.mcl_cuda_counter_update_fused_static(
                    stream, b[0].data_ptr(), b[1].data_ptr(), b[2].data_ptr(), dy.data_ptr(), x.data_ptr(),
                    pb.data_ptr() if want_p2 else None, C, I, O, N, c["lr"], c["lr_scale"], c["beta"],
                    c["eps"], seed)
                assert rc == 0, L.mcl_cuda_static_last_error().decode()
                ctx.finish()
                # bit-exact, the tolerance the update tests use
                assert torch.equal(a[0], b[0]), name
                assert torch.equal(a[1].view(torch.int32), b[1].view(torch.int32)), name
                assert torch.equal(a[2].view(torch.int32), b[2].view(torch.int32)), name
                if want_p2:
                    assert torch.equal(pa, pb), name
        finally:
            ctx.set_gemm_mode("auto")
        assert not np.array_equal(a[0].cpu().numpy(), c["state"])      # and the state did move


def test_static_update_refuses_rows_beyond_its_scratch():
    L = lib()
    cap = L.mcl_cuda_static_scratch_floats()
    assert cap == 1 << 20
    z = torch.zeros(64, dtype=torch.float32, device=DEV)
    s8 = torch.zeros(64, dtype=torch.uint8, device=DEV)
    rc = L.mcl_cuda_counter_update_fused_static(
        torch.cuda.current_stream(0).cuda_stream, s8.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
        z.data_ptr(), None, 11, cap + 4, 1, 1, 0.1, 0.0, 0.9, 1e-3, 1)
    assert rc == 1
    assert b"exceeds the built-in scratch" in L.mcl_cuda_static_last_error()
