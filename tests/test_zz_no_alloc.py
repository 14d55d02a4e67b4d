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


def _multi_tile_case():
    """A layer above the 1,048,576-float array: 640 rows of 2048 weights are updated as a tile of 512
    rows and a tile of 128 rows, so the second tile's state / scale / v / 2-bit offsets and the row
    offset handed to the element hash are exercised."""
    from motifcl_b200 import synth
    N, I, O, C = 32, 2048, 640, 11
    sc, v = synth.scale_v(9, 3, O, I, True)
    return dict(name="multi_tile", N=N, I=I, O=O, C=C, state=synth.counters(9, 3, O, I).reshape(-1), scale=sc, v=v,
                x=synth.activations(9, 3, N, I), dy=synth.upstream_grad(9, 3, N, O, 0.05),
                lr=0.3, lr_scale=0.05, beta=0.9, eps=1e-3, seed=31)


def test_static_update_equals_ordinary_update_twice_in_a_row(ctx, golden):
    L = lib()
    stream = torch.cuda.current_stream(0).cuda_stream
    cases = dict(CASES, multi_tile=_multi_tile_case())
    assert cases["multi_tile"]["I"] * cases["multi_tile"]["O"] > L.mcl_cuda_static_scratch_floats()
    for name, seeds in (("cfg1_rebase", (999, 1000)), ("wide", (7, 8)), ("fused_witness", (777, 778)),
                        ("multi_tile", (31, 32))):
        c = cases[name]
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
                if seed == c["seed"] and f"{name}/dense_state" in golden.files:
                    # the first call is also the compiled reference's own result for this case
                    assert np.array_equal(b[0].cpu().numpy(), golden[f"{name}/dense_state"]), name
                    assert np.array_equal(b[1].cpu().numpy().view(np.uint32),
                                          golden[f"{name}/dense_scale"].view(np.uint32)), name
                    assert np.array_equal(b[2].cpu().numpy().view(np.uint32),
                                          golden[f"{name}/dense_v"].view(np.uint32)), name
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


def test_static_update_refuses_misaligned_tensors():
    """Refused on the host before anything is launched, like the ordinary entry point does."""
    L = lib()
    z = torch.zeros(256, dtype=torch.float32, device=DEV)
    s8 = torch.zeros(256, dtype=torch.uint8, device=DEV)
    p2 = torch.zeros(16, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream(0).cuda_stream
    good = dict(state=s8.data_ptr(), scale=z.data_ptr(), v=z.data_ptr(), grad_out=z.data_ptr(), x=z.data_ptr(),
                packed2=p2.data_ptr())
    for bad in ("scale", "v", "grad_out", "x", "packed2"):
        a = dict(good)
        a[bad] += 2
        rc = L.mcl_cuda_counter_update_fused_static(stream, a["state"], a["scale"], a["v"], a["grad_out"], a["x"],
                                                    a["packed2"], 11, 16, 2, 2, 0.1, 0.0, 0.9, 1e-3, 1)
        assert rc == 1, bad
        assert b"must be 4-byte aligned" in L.mcl_cuda_static_last_error(), bad
