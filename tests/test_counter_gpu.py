"""GPU parity tests of the counter-linear path.  Every call goes through the C ABI
(libmotifcl_cuda.so via ctypes); the CPU oracle and the golden file are the checkers.

Bars: bit-exact for state bytes, 2-bit words, scale and v after the update given identical
fp32 gradients; abs 2e-5 on the reference tests' small shapes and relative L2 1e-5 elsewhere
for forward / grad_x / grad_w (tolerances of MotifCL tests/test_vulkan_counter_fused.cpp:107-118
and tests/test_memory_truth_gate.cpp:86-97)."""
import numpy as np
import pytest
import torch

from cases import all_cases
from motifcl_b200 import MotifclCudaError, codec, synth

pytestmark = pytest.mark.gpu
CASES = {c["name"]: c for c in all_cases()}
DEV = "cuda:0"


def _hy(c):
    return c["lr"], c["lr_scale"], c["beta"], c["eps"], c["seed"]


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def rel_l2(a, ref):
    a, ref = a.astype(np.float64), ref.astype(np.float64)
    return float(np.linalg.norm(a - ref) / max(np.linalg.norm(ref), 1e-30))


def run_dense(ctx, c, gw, rows=None, row_offset=0, want_p2=True):
    I, C = c["I"], c["C"]
    rows = c["O"] if rows is None else rows
    rb = I // 4 * 3
    st = _t(c["state"][row_offset * rb:(row_offset + rows) * rb])
    sc = _t(c["scale"][row_offset:row_offset + rows])
    v = _t(c["v"][row_offset:row_offset + rows])
    g = _t(gw[row_offset:row_offset + rows])
    p2 = torch.zeros(rows, I // 16, dtype=torch.int32, device=DEV) if (want_p2 and I % 16 == 0) else None
    ctx.counter_update_dense(st, sc, v, g, p2, C, I, rows, row_offset, *_hy(c))
    ctx.finish()
    return (st.cpu().numpy(), sc.cpu().numpy(), v.cpu().numpy(),
            None if p2 is None else p2.cpu().numpy().view(np.uint32))


@pytest.mark.parametrize("name", list(CASES))
def test_dense_update_bit_exact_vs_golden_and_oracle(name, ctx, orc, golden):
    c = CASES[name]
    gw = orc.grad_w(c["dy"], c["x"])
    st, sc, v, p2 = run_dense(ctx, c, gw)
    assert np.array_equal(st, golden[f"{name}/dense_state"])
    assert np.array_equal(_bits(sc), _bits(golden[f"{name}/dense_scale"]))
    assert np.array_equal(_bits(v), _bits(golden[f"{name}/dense_v"]))
    o = orc.update_dense(c["state"], c["scale"], c["v"], gw, c["C"], c["I"], c["O"], 0, *_hy(c))
    assert np.array_equal(st, o[0])
    if p2 is not None:
        assert np.array_equal(p2, o[3])


def test_dense_update_row_shard_matches_full(ctx, orc):
    c = CASES["wide"]
    gw = orc.grad_w(c["dy"], c["x"])
    full = orc.update_dense(c["state"], c["scale"], c["v"], gw, c["C"], c["I"], c["O"], 0, *_hy(c))
    rb = c["I"] // 4 * 3
    for r0, nr in [(0, 7), (7, 20), (27, 13)]:
        st, sc, v, p2 = run_dense(ctx, c, gw, rows=nr, row_offset=r0)
        assert np.array_equal(st, full[0][r0 * rb:(r0 + nr) * rb])
        assert np.array_equal(_bits(sc), _bits(full[1][r0:r0 + nr]))
        assert np.array_equal(_bits(v), _bits(full[2][r0:r0 + nr]))
        assert np.array_equal(p2, full[3][r0:r0 + nr])


@pytest.mark.parametrize("O,I,C,lr,lr_scale", [
    (5, 4, 3, 1.0, 0.05),          # one group per row
    (3, 16, 11, 0.5, 0.0),         # one 2-bit word per row
    (130, 64, 11, 3e-3, 0.0),      # 16-byte aligned state rows, ragged row batches
    (33, 2048, 11, 0.2, 0.05),     # eight lane sweeps, q path
    (9, 14336, 11, 3e-3, 0.0),     # the longest row of the 8B-scale configuration
    (6, 5632, 11, 1.0, 0.01),
    (70, 260, 5, 2.0, 0.1),        # in % 16 != 0: byte path, no 2-bit output
    (40, 64, 3, 1.0, 0.05),        # C = 3 with arbitrary bytes: codes whose digit is far outside {-1,0,1}
    (300, 288, 11, 50.0, 0.0),     # huge learning rate: rounded counters far beyond the tick table
])
def test_dense_update_shapes_bit_exact(ctx, orc, O, I, C, lr, lr_scale):
    rng = np.random.default_rng(O * 100003 + I)
    ncodes = 64 if (C == 11 or (O, I) == (40, 64)) else 3 * (2 * C - 1)
    state = codec.pack_codes(rng.integers(0, ncodes, size=(O, I)).astype(np.uint8)).reshape(-1)
    c = dict(I=I, O=O, C=C, state=state, scale=rng.uniform(0.02, 0.2, O).astype(np.float32),
             v=rng.uniform(1e-4, 1e-2, O).astype(np.float32), lr=lr, lr_scale=lr_scale, beta=0.9,
             eps=1e-3, seed=int(rng.integers(0, 2 ** 32)))
    gw = (0.3 * rng.standard_normal((O, I))).astype(np.float32)
    gw[0, :4] = [0.0, -0.0, 1e-30, -1e3]     # zero, negative zero, tiny, huge gradient
    o = orc.update_dense(state, c["scale"], c["v"], gw, C, I, O, 0, *_hy(c))
    st, sc, v, p2 = run_dense(ctx, c, gw)
    assert np.array_equal(st, o[0])
    assert np.array_equal(_bits(sc), _bits(o[1]))
    assert np.array_equal(_bits(v), _bits(o[2]))
    if I % 16 == 0:
        assert np.array_equal(p2, o[3])


def test_two_updates_in_a_row_stay_exact(ctx, orc):
    c = dict(CASES["cfg1_rebase"])
    gw = orc.grad_w(c["dy"], c["x"])
    st, sc, v = c["state"], c["scale"], c["v"]
    dst, dsc, dv = _t(st), _t(sc), _t(v)
    for step in range(3):
        hy = (c["lr"], c["lr_scale"], c["beta"], c["eps"], c["seed"] + step)
        st, sc, v, _ = orc.update_dense(st, sc, v, gw, c["C"], c["I"], c["O"], 0, *hy)
        ctx.counter_update_dense(dst, dsc, dv, _t(gw), None, c["C"], c["I"], c["O"], 0, *hy)
    ctx.finish()
    assert np.array_equal(dst.cpu().numpy(), st)
    assert np.array_equal(_bits(dsc.cpu().numpy()), _bits(sc))
    assert np.array_equal(_bits(dv.cpu().numpy()), _bits(v))


@pytest.mark.parametrize("name", ["fused_witness", "cross_backend"])
def test_decode_forward_grad_x_on_reference_test_shapes(name, ctx, orc, golden):
    c = CASES[name]
    N, I, O, C = c["N"], c["I"], c["O"], c["C"]
    st, sc = _t(c["state"]), _t(c["scale"])
    w = torch.empty(O, I, dtype=torch.float32, device=DEV)
    ctx.counter_decode_weight(st, sc, w, I, O, C)
    assert np.array_equal(w.cpu().numpy(), golden[f"{name}/weight"])     # one multiply: exact
    y = torch.empty(N, O, dtype=torch.float32, device=DEV)
    ctx.counter_forward(_t(c["x"]), st, sc, y, N, I, O, C)
    y_ref = orc.forward(c["x"], c["state"], c["scale"], C, O)
    assert np.abs(y.cpu().numpy() - y_ref).max() <= 2e-5
    gx = torch.empty(N, I, dtype=torch.float32, device=DEV)
    ctx.counter_backward_input(st, sc, _t(c["dy"]), gx, N, I, O, C)
    assert np.abs(gx.cpu().numpy() - golden[f"{name}/grad_x"]).max() <= 2e-5


def test_known_answer_vectors_through_the_abi(ctx):
    """MotifCL tests/test_vulkan_runtime_standalone.cpp:579-640."""
    C = 3
    tern = np.array([[1, 0, -1, 1], [0, 1, 1, -1]])
    st = _t(codec.pack_codes(codec.encode(tern, np.zeros_like(tern), C)).reshape(-1))
    sc = _t(np.array([0.5, 2.0], np.float32))
    w = torch.empty(2, 4, dtype=torch.float32, device=DEV)
    ctx.counter_decode_weight(st, sc, w, 4, 2, C)
    assert w.cpu().numpy().tolist() == [[0.5, 0.0, -0.5, 0.5], [0.0, 2.0, 2.0, -2.0]]
    go = np.array([[1.0, 2.0], [-1.0, 0.5]], np.float32)
    gx = torch.empty(2, 4, dtype=torch.float32, device=DEV)
    ctx.counter_backward_input(st, sc, _t(go), gx, 2, 4, 2, C)
    expect = go[:, :1] * 0.5 * tern[0] + go[:, 1:] * 2.0 * tern[1]
    assert np.allclose(gx.cpu().numpy(), expect, atol=1e-6)


def test_cfg1_forward_backward_grad_w_within_tolerance(ctx, orc):
    c = CASES["cfg1"]
    N, I, O, C = c["N"], c["I"], c["O"], c["C"]
    st, sc = _t(c["state"]), _t(c["scale"])
    y = torch.empty(N, O, dtype=torch.float32, device=DEV)
    ctx.counter_forward(_t(c["x"]), st, sc, y, N, I, O, C)
    assert rel_l2(y.cpu().numpy(), orc.forward(c["x"], c["state"], c["scale"], C, O)) <= 1e-5
    gx = torch.empty(N, I, dtype=torch.float32, device=DEV)
    ctx.counter_backward_input(st, sc, _t(c["dy"]), gx, N, I, O, C)
    assert rel_l2(gx.cpu().numpy(), orc.backward_input(c["dy"], c["state"], c["scale"], C, I)) <= 1e-5
    gw = torch.empty(O, I, dtype=torch.float32, device=DEV)
    ctx.matmul_f32(_t(c["dy"]), _t(c["x"]), gw, O, N, I, trans_a=True)
    assert rel_l2(gw.cpu().numpy(), orc.grad_w(c["dy"], c["x"])) <= 1e-5


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True)])
def test_matmul_f32_multi_tile_odd_shapes(ctx, orc, ta, tb):
    """48 x 40 x 33 as in MotifCL tests/test_vulkan_runtime_standalone.cpp (multi-tile,
    non-multiples); tolerance 1e-4 abs of tests/test_matmul.cpp."""
    M, K, N = 48, 40, 33
    rng = np.random.default_rng(3)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    a = A.T.copy() if ta else A
    b = B.T.copy() if tb else B
    c = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ctx.matmul_f32(_t(a), _t(b), c, M, K, N, ta, tb)
    assert np.abs(c.cpu().numpy() - orc.matmul(a, b, M, K, N, ta, tb)).max() <= 1e-4


@pytest.mark.parametrize("name", ["fused_witness", "cross_backend", "cfg1_rebase"])
def test_fused_update_through_layer_api(name, ctx, orc, golden):
    """The autograd-order transaction of MotifCL src/nn/compact_counter.cpp:40-50: grad_x from
    the pre-update state, then the memory-native update.  State/scale/v must equal the
    compiled reference's exactly when the in-library grad_w equals the r-ascending fp32 sum
    bit for bit."""
    c = CASES[name]
    N, I, O, C = c["N"], c["I"], c["O"], c["C"]
    st, sc, v = _t(c["state"]), _t(c["scale"]), _t(c["v"])
    p2 = torch.zeros(O, max(I // 16, 1), dtype=torch.int32, device=DEV) if I % 16 == 0 else None
    ctx.set_gemm_mode("exact")
    try:
        ctx.counter_update_fused(st, sc, v, _t(c["dy"]), _t(c["x"]), p2, C, I, O, N, *_hy(c))
        ctx.finish()
    finally:
        ctx.set_gemm_mode("auto")
    got = codec.unpack_codes(st.cpu().numpy().reshape(O, -1), I)
    want = codec.unpack_codes(golden[f"{name}/dense_state"].reshape(O, -1), I)
    # exact mode = the CUDA-core contraction (k ascending, unfused multiply-add),
    # so the whole transaction is bit-identical, as MotifCL tests/test_vulkan_counter_fused.cpp:120-133 asks
    assert np.array_equal(got, want)
    assert np.array_equal(_bits(sc.cpu().numpy()), _bits(golden[f"{name}/dense_scale"]))
    assert np.array_equal(_bits(v.cpu().numpy()), _bits(golden[f"{name}/dense_v"]))
    if p2 is not None:
        t, _ = codec.decode(got, C)
        assert np.array_equal(codec.unpack2(p2.cpu().numpy().view(np.uint32), I), (t + 1).astype(np.uint8))


def test_pack2_matches_oracle(ctx, orc):
    c = CASES["cfg1"]
    p2 = torch.empty(c["O"], c["I"] // 16, dtype=torch.int32, device=DEV)
    ctx.counter_pack2(_t(c["state"]), p2, c["I"], c["O"], c["C"])
    assert np.array_equal(p2.cpu().numpy().view(np.uint32), orc.pack2(c["state"], c["C"], c["I"], c["O"]))


@pytest.mark.parametrize("M", [1, 2, 3, 4, 16])
@pytest.mark.parametrize("O,I", [(288, 288), (96, 2048), (40, 5632),         # CUDA-core kernels
                                 (256, 2048), (300, 4160), (1000, 512), (4096, 1024)])   # tensor-core kernel
def test_ternary_gemv_vs_oracle(ctx, orc, M, O, I):
    if M == 3 and O == 4096:
        M = 13      # an activation-row count that is not a multiple of four
    rng = np.random.default_rng(M * 7 + O)
    st = synth.counters(5, O % 97, O, I).reshape(-1)
    p2 = orc.pack2(st, 11, I, O)
    scale = rng.uniform(0.02, 0.2, O).astype(np.float32)
    x = rng.standard_normal((M, I)).astype(np.float32)
    y = torch.empty(M, O, dtype=torch.float32, device=DEV)
    ctx.ternary_gemv(_t(x), _t(p2.view(np.int32)), _t(scale), y, M, I, O)
    ref64 = orc.ternary_gemv(x, p2, scale, f64=True)
    assert rel_l2(y.cpu().numpy(), ref64) <= 1e-5
    assert rel_l2(y.cpu().numpy(), orc.forward(x, st, scale, 11, O)) <= 1e-5


@pytest.mark.parametrize("O,I", [(203, 1024), (33, 4096), (2380, 2048), (64, 256), (500, 3840), (3000, 1280),   # one table for the whole row
                                 (5000, 8192), (100, 6144), (257, 14336)])     # sliced tables, ticket reduction
def test_single_row_gemv_table_kernels_vs_oracle(ctx, orc, O, I):
    """One activation row on the table look-up kernels: row counts that are no multiple of 16 or 256, every field
    value (3 included: random words), repeated launches (the ticket words must come back to zero) and a recorded
    batch replayed several times."""
    rng = np.random.default_rng(O + I)
    words = rng.integers(0, 2 ** 32, size=(O, I // 16), dtype=np.uint64).astype(np.uint32)
    fields = np.zeros((O, I), np.float64)
    for k in range(16):
        fields[:, k::16] = ((words >> np.uint32(2 * k)) & np.uint32(3)).astype(np.float64)
    scale = rng.uniform(0.02, 0.2, O).astype(np.float32)
    xs = [rng.standard_normal((1, I)).astype(np.float32) for _ in range(3)]
    wd, sd = _t(words.view(np.int32)), _t(scale)
    refs = [(x.astype(np.float64) @ (fields - 1.0).T) * scale.astype(np.float64) for x in xs]
    y = torch.full((1, O), 7.0, dtype=torch.float32, device=DEV)
    for x, ref in zip(xs, refs):
        ctx.ternary_gemv(_t(x), wd, sd, y, 1, I, O)
        assert rel_l2(y.cpu().numpy(), ref) <= 1e-5
    first = y.clone()
    ctx.ternary_gemv(_t(xs[2]), wd, sd, y, 1, I, O)
    assert torch.equal(first, y)                      # deterministic, launch after launch
    xd = _t(xs[0])
    ctx.finish()
    ctx.batch_begin()
    try:
        ctx.ternary_gemv(xd, wd, sd, y, 1, I, O)
    finally:
        batch = ctx.batch_end()
    try:
        for x, ref in zip(xs, refs):
            xd.copy_(torch.from_numpy(x).to(DEV))
            y.fill_(3.0)
            torch.cuda.synchronize()
            batch.launch()
            ctx.finish()
            assert rel_l2(y.cpu().numpy(), ref) <= 1e-5
    finally:
        batch.close()


def test_ternary_gemv_calls_in_a_row_leave_no_residue(ctx, orc):
    """Split-K accumulators of the tensor-core GEMV live in the context's workspace: alternate shapes and
    activation counts and repeat the first call at the end."""
    calls = [(4, 4096, 1024), (1, 512, 2048), (16, 1000, 512), (4, 4096, 1024), (1, 256, 4096), (4, 4096, 1024)]
    data = {}
    for M, O, I in calls:
        key = (M, O, I)
        if key not in data:
            rng = np.random.default_rng(M + O + I)
            st = synth.counters(5, (O + I) % 97, O, I).reshape(-1)
            p2 = orc.pack2(st, 11, I, O)
            scale = rng.uniform(0.02, 0.2, O).astype(np.float32)
            x = rng.standard_normal((M, I)).astype(np.float32)
            data[key] = (_t(x), _t(p2.view(np.int32)), _t(scale), orc.ternary_gemv(x, p2, scale, f64=True))
        xd, pd, sd, ref = data[key]
        y = torch.full((M, O), 9.0, dtype=torch.float32, device=DEV)
        ctx.ternary_gemv(xd, pd, sd, y, M, I, O)
        assert rel_l2(y.cpu().numpy(), ref) <= 1e-5, key


def test_argument_checks_mirror_the_reference(ctx):
    """Refusals of MotifCL src/runtime/vulkan_backend.cpp:8497-8521."""
    st = torch.zeros(48, dtype=torch.uint8, device=DEV)
    f = torch.zeros(64, dtype=torch.float32, device=DEV)
    good = dict(C_=3, in_features=8, rows=2, row_offset=0, lr=0.1, lr_scale=0.0, rms_beta=0.9, rms_eps=1e-3, seed=1)

    def call(**kw):
        a = dict(good, **kw)
        ctx.counter_update_dense(st, f, f, f, None, a["C_"], a["in_features"], a["rows"], a["row_offset"],
                                 a["lr"], a["lr_scale"], a["rms_beta"], a["rms_eps"], a["seed"])

    call()
    for bad, frag in [(dict(in_features=6), "in_features % 4"), (dict(C_=0), "non-zero"),
                      (dict(C_=12), "C too large"), (dict(rows=0), "non-zero"),
                      (dict(lr=float("nan")), "finite lr"), (dict(lr_scale=float("inf")), "finite lr_scale"),
                      (dict(rms_beta=float("nan")), "finite rms_beta"), (dict(rms_eps=-1.0), "rms_eps")]:
        with pytest.raises(MotifclCudaError) as e:
            call(**bad)
        assert e.value.code == 1 and frag in e.value.message
    with pytest.raises(MotifclCudaError):
        ctx.ternary_gemv(f, st, f, f, 17, 16, 2)
    ctx.finish()    # the context stays usable after refusals
    call()
    ctx.finish()


def test_layer_mirror_teacher_recovery(ctx):
    """Statistical witness of MotifCL tests/test_counter_state.cpp:17-90 (16x16 teacher, N 256,
    C 11, lr 5e-3, 800 steps of forward + MSE + backward): final MSE <= 5e-3, ternary accuracy
    >= 0.9.  MSE gradient formed with torch; everything else through the library."""
    from motifcl_b200 import CounterStateLinear
    g = torch.Generator(device="cpu").manual_seed(0)
    teacher_t = torch.randint(-1, 2, (16, 16), generator=g).float()
    s0 = float(np.sqrt(3.0 / 32.0))
    teacher = (teacher_t * s0).to(DEV)
    layer = CounterStateLinear(ctx, 16, 16, C=11, lr=5e-3, seed=12345)
    mse = None
    for step in range(800):
        x = torch.randn(256, 16, generator=g).to(DEV)
        y = layer.forward(x)
        target = x @ teacher.T
        diff = y - target
        mse = float((diff * diff).mean())
        grad_out = (2.0 / diff.numel()) * diff
        layer.backward(x, grad_out, layer.next_seed(), need_grad_x=False)
    codes = codec.unpack_codes(layer.state.cpu().numpy().reshape(16, -1), 16)
    t, _ = codec.decode(codes, 11)
    acc = float((t == teacher_t.numpy().astype(np.int64)).mean())
    assert mse <= 5e-3 and acc >= 0.9, (mse, acc)


def test_accumulated_micro_batches_update_once(ctx, orc):
    """Three micro-batches summed into one gradient, then one update: the summed gradient is within 1e-5
    (relative L2) of the float64 sum over all tokens, grad_x comes from the unchanged state every time,
    and the update is bit-identical to the CPU checker's given the summed gradient's bytes."""
    from motifcl_b200 import CounterStateLinear
    I, O, C, N = 96, 64, 11, 160
    layer = CounterStateLinear(ctx, I, O, C=C, lr=3e-3, lr_scale=0.05, seed=7)
    st0 = layer.state.cpu().numpy().copy()
    sc0, v0 = layer.scale.cpu().numpy().copy(), layer.v.cpu().numpy().copy()
    rng = np.random.default_rng(5)
    xs = [rng.standard_normal((N, I)).astype(np.float32) for _ in range(3)]
    dys = [(0.02 * rng.standard_normal((N, O))).astype(np.float32) for _ in range(3)]
    with pytest.raises(RuntimeError):
        layer.apply_accumulated(1)
    for x, dy in zip(xs, dys):
        gx = layer.accumulate_backward(_t(x), _t(dy))
        ctx.finish()
        assert rel_l2(gx.cpu().numpy(), orc.backward_input(dy, st0, sc0, C, I)) <= 1e-5
        assert np.array_equal(layer.state.cpu().numpy(), st0)          # no update between micro-batches
    gw = layer._acc.cpu().numpy().copy()
    ref = sum(dy.astype(np.float64).T @ x.astype(np.float64) for x, dy in zip(xs, dys))
    assert rel_l2(gw, ref) <= 1e-5
    p2 = torch.zeros(O, I // 16, dtype=torch.int32, device=DEV)
    assert layer.apply_accumulated(99, p2) == 3
    ctx.finish()
    e = orc.update_dense(st0, sc0, v0, gw, C, I, O, 0, 3e-3, 0.05, 0.9, 1e-3, 99)
    assert np.array_equal(layer.state.cpu().numpy(), e[0])
    assert np.array_equal(_bits(layer.scale.cpu().numpy()), _bits(e[1]))
    assert np.array_equal(_bits(layer.v.cpu().numpy()), _bits(e[2]))
    assert np.array_equal(p2.cpu().numpy().view(np.uint32), e[3])
    # the buffer starts over
    layer.accumulate_backward(_t(xs[0]), _t(dys[0]), need_grad_x=False)
    ctx.finish()
    assert rel_l2(layer._acc.cpu().numpy(), dys[0].astype(np.float64).T @ xs[0].astype(np.float64)) <= 1e-5


# ---- tensor-core (tcgen05) contractions -----------------------------------------------------

TC_SHAPES = [(256, 288, 288), (512, 768, 288), (300, 288, 768), (1000, 2048, 512), (129, 96, 1032), (4096, 1024, 1024)]


@pytest.mark.parametrize("terms", [(3, 6), (2, 3)])
@pytest.mark.parametrize("N,I,O", TC_SHAPES)
def test_tensor_core_contractions_vs_oracle(ctx, orc, N, I, O, terms):
    """Y, dX and dW on tcgen05 against the fp32 reference sums (relative L2 <= 1e-5, the bound
    the path is specified to) and against float64 accumulation."""
    rng = np.random.default_rng(N + I + O)
    st = synth.counters(7, (N + O) % 89, O, I).reshape(-1)
    scale = rng.uniform(0.02, 0.2, O).astype(np.float32)
    x = rng.standard_normal((N, I)).astype(np.float32)
    dy = (0.02 * rng.standard_normal((N, O))).astype(np.float32)
    ctx.set_gemm_mode("tensor", *terms)
    try:
        d_st, d_sc, d_x, d_dy = _t(st), _t(scale), _t(x), _t(dy)
        y = torch.empty(N, O, dtype=torch.float32, device=DEV)
        gx = torch.empty(N, I, dtype=torch.float32, device=DEV)
        gw = torch.empty(O, I, dtype=torch.float32, device=DEV)
        ctx.counter_forward(d_x, d_st, d_sc, y, N, I, O, 11)
        ctx.counter_backward_input(d_st, d_sc, d_dy, gx, N, I, O, 11)
        ctx.matmul_f32(d_dy, d_x, gw, O, N, I, trans_a=True)
        ctx.finish()
    finally:
        ctx.set_gemm_mode("auto")
    w = orc.decode_weight(st, scale, 11, I, O)
    small = N * I * O <= 300 * 768 * 768
    if small:
        assert rel_l2(y.cpu().numpy(), orc.forward(x, st, scale, 11, O)) <= 1e-5
        assert rel_l2(gx.cpu().numpy(), orc.backward_input(dy, st, scale, 11, I)) <= 1e-5
        assert rel_l2(gw.cpu().numpy(), orc.grad_w(dy, x)) <= 1e-5
    y64 = x.astype(np.float64) @ w.astype(np.float64).T
    gx64 = dy.astype(np.float64) @ w.astype(np.float64)
    gw64 = dy.astype(np.float64).T @ x.astype(np.float64)
    assert rel_l2(y.cpu().numpy(), y64) <= 1e-5
    assert rel_l2(gx.cpu().numpy(), gx64) <= 1e-5
    assert rel_l2(gw.cpu().numpy(), gw64) <= 1e-5


def test_tensor_core_matmul_all_transposes(ctx, orc):
    M, K, N = 200, 520, 136
    rng = np.random.default_rng(17)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    ctx.set_gemm_mode("tensor")
    try:
        for ta, tb in [(False, False), (True, False), (False, True), (True, True)]:
            a = A.T.copy() if ta else A
            b = B.T.copy() if tb else B
            c = torch.empty(M, N, dtype=torch.float32, device=DEV)
            ctx.matmul_f32(_t(a), _t(b), c, M, K, N, ta, tb)
            ctx.finish()
            assert rel_l2(c.cpu().numpy(), ref) <= 1e-5, (ta, tb)
    finally:
        ctx.set_gemm_mode("auto")


@pytest.mark.parametrize("mode", ["tensor", "exact"])
def test_linear_step_matches_separate_calls_and_oracle(ctx, orc, mode):
    """The one-call step: y and grad_x from the PRE-update state, then the dense update fed by
    the step's own grad_w; the update must be bit-exact given that gradient."""
    c = CASES["cfg1_rebase"]
    N, I, O, C = c["N"], c["I"], c["O"], c["C"]
    st, sc, v = _t(c["state"]), _t(c["scale"]), _t(c["v"])
    y = torch.empty(N, O, dtype=torch.float32, device=DEV)
    gx = torch.empty(N, I, dtype=torch.float32, device=DEV)
    gw = torch.empty(O, I, dtype=torch.float32, device=DEV)
    p2 = torch.zeros(O, I // 16, dtype=torch.int32, device=DEV)
    ctx.set_gemm_mode(mode)
    try:
        ctx.counter_linear_step(_t(c["x"]), _t(c["dy"]), st, sc, v, y, gx, gw, p2, C, I, O, N, O, 0, *_hy(c))
        ctx.finish()
    finally:
        ctx.set_gemm_mode("auto")
    assert rel_l2(y.cpu().numpy(), orc.forward(c["x"], c["state"], c["scale"], C, O)) <= 1e-5
    assert rel_l2(gx.cpu().numpy(), orc.backward_input(c["dy"], c["state"], c["scale"], C, I)) <= 1e-5
    gw_h = gw.cpu().numpy()
    assert rel_l2(gw_h, orc.grad_w(c["dy"], c["x"])) <= 1e-5
    o = orc.update_dense(c["state"], c["scale"], c["v"], gw_h, C, I, O, 0, *_hy(c))
    assert np.array_equal(st.cpu().numpy(), o[0])
    assert np.array_equal(_bits(sc.cpu().numpy()), _bits(o[1]))
    assert np.array_equal(_bits(v.cpu().numpy()), _bits(o[2]))
    assert np.array_equal(p2.cpu().numpy().view(np.uint32), o[3])
    if mode == "exact":   # and then the whole transaction equals the reference's
        e = orc.update_fused(c["state"], c["scale"], c["v"], c["dy"], c["x"], C, *_hy(c))
        assert np.array_equal(st.cpu().numpy(), e[0])


@pytest.mark.parametrize("D,N", [(256, 64), (1024, 32), (2048, 64)])
def test_memory_native_update_allocates_less_than_a_quarter_of_a_dense_weight(orc, D, N):
    """MotifCL's memory gate (tests/test_memory_truth_gate.cpp:30-126: D = 256, N = 64) on a context of its own: the
    fused update may allocate less than a quarter of a dense fp32 [D, D] weight, where the dense path needs at least a
    half (here: the whole gradient, which the CALLER of mcl_cuda_counter_update_dense allocates).  The result is still
    the checker's, byte for byte (CUDA-core products: k ascending like the reference's sums)."""
    from motifcl_b200 import Context
    rng = np.random.default_rng(D + N)
    C = 11
    hy = dict(lr=3e-3, lr_scale=0.0, rms_beta=0.9, rms_eps=1e-3, seed=4242)
    state = synth.counters(C, 9, D, D).reshape(-1)
    scale = rng.uniform(0.02, 0.2, D).astype(np.float32)
    v = rng.uniform(0.0, 1e-3, D).astype(np.float32)
    x = rng.standard_normal((N, D)).astype(np.float32)
    dy = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
    own = Context.on_torch_stream(0)
    try:
        own.set_gemm_mode("exact")
        assert own.workspace_bytes == 0
        st, sc, vv = _t(state), _t(scale), _t(v)
        own.counter_update_fused(st, sc, vv, _t(dy), _t(x), None, C, D, D, N, hy["lr"], hy["lr_scale"], hy["rms_beta"],
                                 hy["rms_eps"], hy["seed"])
        own.finish()
        dense_weight = D * D * 4
        print(f"D = {D}: workspace {own.workspace_bytes} bytes = {own.workspace_bytes / dense_weight:.3f} of a dense weight")
        assert 0 < own.workspace_bytes < dense_weight // 4
        e = orc.update_fused(state, scale, v, dy, x, C, hy["lr"], hy["lr_scale"], hy["rms_beta"], hy["rms_eps"], hy["seed"])
        assert np.array_equal(st.cpu().numpy(), e[0])
        assert np.array_equal(_bits(sc.cpu().numpy()), _bits(e[1])) and np.array_equal(_bits(vv.cpu().numpy()), _bits(e[2]))
    finally:
        own.close()


def test_tensor_core_fused_update_flip_rate(ctx, orc):
    """Memory-native update with grad_w formed on tensor cores: grad_w differs from the fp32
    reference sum in its last bits, so a few stochastic roundings may fall the other way.  The
    rate is measured here and must stay small; scale and v agree to 1e-6 as the reference's own
    cross-backend rule asks (MotifCL tests/test_vulkan_backend.cpp:1208-1219)."""
    c = CASES["cfg1_rebase"]
    N, I, O, C = c["N"], c["I"], c["O"], c["C"]
    st, sc, v = _t(c["state"]), _t(c["scale"]), _t(c["v"])
    ctx.set_gemm_mode("tensor")
    try:
        ctx.counter_update_fused(st, sc, v, _t(c["dy"]), _t(c["x"]), None, C, I, O, N, *_hy(c))
        ctx.finish()
    finally:
        ctx.set_gemm_mode("auto")
    e = orc.update_fused(c["state"], c["scale"], c["v"], c["dy"], c["x"], C, *_hy(c))
    got = codec.unpack_codes(st.cpu().numpy().reshape(O, -1), I)
    want = codec.unpack_codes(e[0].reshape(O, -1), I)
    flips = float((got != want).mean())
    print(f"tensor-core fused update: code flip rate {flips:.2e}")
    assert flips <= 1e-3
    assert np.allclose(sc.cpu().numpy(), e[1], rtol=0, atol=1e-6)
    assert np.allclose(v.cpu().numpy(), e[2], rtol=1e-5, atol=1e-9)


def test_recorded_batch_replays_the_step_with_a_per_step_seed(ctx, orc):
    """Two steps replayed from one recorded batch equal two eager steps: the seed of step k is
    base + k through the device seed word (as CounterStateLinear::next_seed() advances,
    MotifCL include/motifcl/nn/compact_counter.hpp:34)."""
    from motifcl_b200.step import CounterLinearState, CounterStack, Hyper
    c = CASES["cfg1"]
    N, I, O = c["N"], c["I"], c["O"]
    shape = synth.LinearShape("l", O, I)
    x, dy = _t(c["x"]), _t(c["dy"])
    results = []
    for recorded in (False, True):
        lin = CounterLinearState(shape, c["state"], c["scale"], c["v"], torch.device(DEV))
        stack = CounterStack(ctx, [lin], Hyper(lr=0.05), N)
        for _ in range(4):
            stack.step([x], [dy], base_seed=100, recorded=recorded)
        ctx.finish()
        results.append((lin.state.cpu().numpy(), lin.scale.cpu().numpy(), lin.v.cpu().numpy(),
                        lin.packed2.cpu().numpy()))
    for a, b in zip(*results):
        assert np.array_equal(a, b)
    # and the first step's update is bit-exact against the checker given the step's own gradient
    lin = CounterLinearState(shape, c["state"], c["scale"], c["v"], torch.device(DEV))
    stack = CounterStack(ctx, [lin], Hyper(lr=0.05), N)
    stack.step([x], [dy], base_seed=100)
    ctx.finish()
    o = orc.update_dense(c["state"], c["scale"], c["v"], lin.grad_w.cpu().numpy(), 11, I, O, 0, 0.05, 0.0, 0.9, 1e-3, 100)
    assert np.array_equal(lin.state.cpu().numpy(), o[0])


@pytest.mark.parametrize("mode", ["tensor", "exact"])
def test_products_from_packed2_equal_products_from_state(ctx, orc, mode):
    """What a data-parallel rank runs for layers whose state it does not own: Y, dX, dW from the
    2-bit words must equal the same products computed from the 6-bit state (bit for bit: the
    ternary digits are identical and so is every kernel that consumes them)."""
    c = CASES["cfg1"]
    N, I, O, C = c["N"], c["I"], c["O"], c["C"]
    st, sc, x, dy = _t(c["state"]), _t(c["scale"]), _t(c["x"]), _t(c["dy"])
    p2 = torch.empty(O, I // 16, dtype=torch.int32, device=DEV)
    ctx.counter_pack2(st, p2, I, O, C)
    outs = []
    ctx.set_gemm_mode(mode)
    try:
        for src in ("state", "packed2"):
            y = torch.empty(N, O, dtype=torch.float32, device=DEV)
            gx = torch.empty(N, I, dtype=torch.float32, device=DEV)
            gw = torch.empty(O, I, dtype=torch.float32, device=DEV)
            if src == "state":
                ctx.counter_linear_step(x, dy, st.clone(), sc.clone(), _t(c["v"]), y, gx, gw, None, C, I, O, N, 0, 0,
                                        *_hy(c))
            else:
                ctx.ternary_linear_products(x, dy, p2, sc, y, gx, gw, I, O, N)
            ctx.finish()
            outs.append((y.cpu().numpy(), gx.cpu().numpy(), gw.cpu().numpy()))
    finally:
        ctx.set_gemm_mode("auto")
    for a, b in zip(*outs):
        assert np.array_equal(a, b)
    assert rel_l2(outs[1][0], orc.forward(c["x"], c["state"], c["scale"], C, O)) <= 1e-5


FUSED_SHAPES = [(256, 64, 64), (1000, 96, 32), (2048, 288, 288), (1024, 288, 768), (1024, 768, 288),
                (516, 1024, 1024), (512, 32, 1024)]


@pytest.mark.parametrize("N,I,O", FUSED_SHAPES)
def test_fused_tf32_products_vs_oracle(ctx, orc, N, I, O):
    """Layers up to 1024 features whose dimensions are multiples of 32 take the kernel that reads the
    fp32 tensors through TMA and multiplies tf32 hi/lo terms (transposed operands in place):
    every product within 1e-5 relative L2 of the fp32 reference sums, ragged token counts included."""
    rng = np.random.default_rng(N + 3 * I + 7 * O)
    C = 11
    state = codec.pack_codes(rng.integers(0, 64, size=(O, I)).astype(np.uint8)).reshape(-1)
    x = rng.standard_normal((N, I)).astype(np.float32)
    dy = (0.02 * rng.standard_normal((N, O))).astype(np.float32)
    sc = rng.uniform(0.02, 0.2, O).astype(np.float32)
    y = torch.full((N, O), 7.0, dtype=torch.float32, device=DEV)
    gx = torch.full((N, I), 7.0, dtype=torch.float32, device=DEV)
    gw = torch.full((O, I), 7.0, dtype=torch.float32, device=DEV)
    v = torch.zeros(O, dtype=torch.float32, device=DEV)
    ctx.set_gemm_mode("tensor")
    try:
        ctx.counter_linear_step(_t(x), _t(dy), _t(state), _t(sc), v, y, gx, gw, None, C, I, O, N, 0, 0,
                                3e-3, 0.0, 0.9, 1e-3, 1)
        ctx.finish()
    finally:
        ctx.set_gemm_mode("auto")
    assert rel_l2(y.cpu().numpy(), orc.forward(x, state, sc, C, O)) <= 1e-5
    assert rel_l2(gx.cpu().numpy(), orc.backward_input(dy, state, sc, C, I)) <= 1e-5
    assert rel_l2(gw.cpu().numpy(), orc.grad_w(dy, x)) <= 1e-5


def test_linear_step_many_equals_layer_by_layer(ctx, orc):
    """mcl_cuda_counter_linear_step_many: grouped launches for the layers that qualify, single calls for
    the rest; each layer's products within tolerance and its update bit-exact given its own grad_w."""
    from motifcl_b200.runtime import linear_descs
    rng = np.random.default_rng(5)
    C, N = 11, 1024
    shapes = [(288, 288), (288, 768), (768, 288), (64, 96), (36, 40)]     # the last one does not qualify
    hy = (0.3, 0.05, 0.9, 1e-3)
    layers, entries = [], []
    for (I, O) in shapes:
        state = codec.pack_codes(rng.integers(0, 64, size=(O, I)).astype(np.uint8)).reshape(-1)
        L = dict(I=I, O=O, state=state, x=rng.standard_normal((N, I)).astype(np.float32),
                 dy=(0.02 * rng.standard_normal((N, O))).astype(np.float32),
                 sc=rng.uniform(0.02, 0.2, O).astype(np.float32), v=rng.uniform(1e-4, 1e-2, O).astype(np.float32))
        L["d"] = dict(x=_t(L["x"]), grad_out=_t(L["dy"]), state=_t(state), scale=_t(L["sc"]), v=_t(L["v"]),
                      y=torch.empty(N, O, dtype=torch.float32, device=DEV),
                      grad_x=torch.empty(N, I, dtype=torch.float32, device=DEV),
                      grad_w=torch.empty(O, I, dtype=torch.float32, device=DEV),
                      packed2_out=torch.zeros(O, (I + 15) // 16, dtype=torch.int32, device=DEV) if I % 16 == 0 else None,
                      in_features=I, out_features=O, batch=N, update_rows=O, row_offset=0)
        layers.append(L)
        entries.append(L["d"])
    ctx.set_gemm_mode("tensor")
    try:
        ctx.counter_linear_step_many(linear_descs(entries), C, *hy, 4242)
        ctx.finish()
    finally:
        ctx.set_gemm_mode("auto")
    for L in layers:
        I, O, d = L["I"], L["O"], L["d"]
        assert rel_l2(d["y"].cpu().numpy(), orc.forward(L["x"], L["state"], L["sc"], C, O)) <= 1e-5
        assert rel_l2(d["grad_x"].cpu().numpy(), orc.backward_input(L["dy"], L["state"], L["sc"], C, I)) <= 1e-5
        gw = d["grad_w"].cpu().numpy()
        assert rel_l2(gw, orc.grad_w(L["dy"], L["x"])) <= 1e-5
        o = orc.update_dense(L["state"], L["sc"], L["v"], gw, C, I, O, 0, *hy, 4242)
        assert np.array_equal(d["state"].cpu().numpy(), o[0])
        assert np.array_equal(_bits(d["scale"].cpu().numpy()), _bits(o[1]))
        assert np.array_equal(_bits(d["v"].cpu().numpy()), _bits(o[2]))
        if d["packed2_out"] is not None:
            assert np.array_equal(d["packed2_out"].cpu().numpy().view(np.uint32), o[3])


# ---- the benchmarked configurations themselves ----------------------------------------------------

def _stack_entry(cfg, idx, shape, N, sigma, randomised=True):
    I, O = shape.in_features, shape.out_features
    sc, v = synth.scale_v(cfg, idx, O, I, randomised)
    L = dict(I=I, O=O, state=synth.counters(cfg, idx, O, I).reshape(-1), sc=sc, v=v,
             x=synth.activations(cfg, idx, N, I), dy=synth.upstream_grad(cfg, idx, N, O, sigma))
    L["d"] = dict(x=_t(L["x"]), grad_out=_t(L["dy"]), state=_t(L["state"]), scale=_t(sc), v=_t(v),
                  y=torch.empty(N, O, dtype=torch.float32, device=DEV),
                  grad_x=torch.empty(N, I, dtype=torch.float32, device=DEV),
                  grad_w=torch.empty(O, I, dtype=torch.float32, device=DEV),
                  packed2_out=torch.zeros(O, I // 16, dtype=torch.int32, device=DEV),
                  in_features=I, out_features=O, batch=N, update_rows=O, row_offset=0)
    return L


def _check_update_given_own_gradient(orc, L, C, hy, seed):
    d = L["d"]
    gw = d["grad_w"].cpu().numpy()
    o = orc.update_dense(L["state"], L["sc"], L["v"], gw, C, L["I"], L["O"], 0, *hy, seed)
    assert np.array_equal(d["state"].cpu().numpy(), o[0])
    assert np.array_equal(_bits(d["scale"].cpu().numpy()), _bits(o[1]))
    assert np.array_equal(_bits(d["v"].cpu().numpy()), _bits(o[2]))
    assert np.array_equal(d["packed2_out"].cpu().numpy().view(np.uint32), o[3])
    return gw


def test_grouped_step_at_the_benchmark_token_count_vs_oracle(ctx, orc):
    """The stories15M-shaped workload as the benchmark runs it: 8192 tokens, so every weight gradient is
    four 2048-token slices added by the grouped split-K reduction.  One layer of each of the three shapes
    against the fp32 reference sums (relative L2 <= 1e-5), update bit-exact given the step's own gradient."""
    from motifcl_b200.runtime import linear_descs
    C, N = 11, 8192
    hy = (3e-3, 0.05, 0.9, 1e-3)
    shapes = [synth.LinearShape("wq", 288, 288), synth.LinearShape("w1", 768, 288), synth.LinearShape("w2", 288, 768)]
    layers = [_stack_entry(2, 50 + i, s, N, 0.02) for i, s in enumerate(shapes)]
    ctx.counter_linear_step_many(linear_descs([L["d"] for L in layers]), C, *hy, 12345)
    ctx.finish()
    for L in layers:
        d = L["d"]
        assert rel_l2(d["y"].cpu().numpy(), orc.forward(L["x"], L["state"], L["sc"], C, L["O"])) <= 1e-5
        assert rel_l2(d["grad_x"].cpu().numpy(), orc.backward_input(L["dy"], L["state"], L["sc"], C, L["I"])) <= 1e-5
        gw = _check_update_given_own_gradient(orc, L, C, hy, 12345)
        assert rel_l2(gw, orc.grad_w(L["dy"], L["x"])) <= 1e-5


def test_grouped_step_of_all_42_linears_at_8192_tokens(ctx, orc):
    """The whole benchmarked call: 42 linears x 8192 tokens in one mcl_cuda_counter_linear_step_many (problem
    tables of 42 and 2 x 42 entries).  Products against float64 sums (relative L2 <= 1e-5); update bit-exact
    given each layer's own gradient."""
    from motifcl_b200.runtime import linear_descs
    C, N = 11, 8192
    hy = (3e-3, 0.0, 0.9, 1e-3)
    shapes = synth.stories15m_linears()
    layers = [_stack_entry(2, i, s, N, 0.02, randomised=False) for i, s in enumerate(shapes)]
    ctx.counter_linear_step_many(linear_descs([L["d"] for L in layers]), C, *hy, 777)
    ctx.finish()
    worst = [0.0, 0.0, 0.0]
    for L in layers:
        d = L["d"]
        w = orc.decode_weight(L["state"], L["sc"], C, L["I"], L["O"]).astype(np.float64)
        x64, dy64 = L["x"].astype(np.float64), L["dy"].astype(np.float64)
        errs = (rel_l2(d["y"].cpu().numpy(), x64 @ w.T), rel_l2(d["grad_x"].cpu().numpy(), dy64 @ w),
                rel_l2(_check_update_given_own_gradient(orc, L, C, hy, 777), dy64.T @ x64))
        worst = [max(a, b) for a, b in zip(worst, errs)]
        del d["x"], d["grad_out"], d["y"], d["grad_x"]
    print(f"42 linears x 8192 tokens: worst relative L2  Y {worst[0]:.2e}  dX {worst[1]:.2e}  dW {worst[2]:.2e}")
    assert max(worst) <= 1e-5, worst


@pytest.mark.parametrize("M", [1, 2, 4, 16])
@pytest.mark.parametrize("O,I", [(14336, 4096), (4096, 14336), (4096, 4096)])
def test_ternary_gemv_on_the_decode_sweep_matrices(ctx, orc, M, O, I):
    """The matrices of the decode-GEMV configuration (w1 / w3, w2, q / o of an 8B-scale block) against float64."""
    rng = np.random.default_rng(M * 11 + O // 1024)
    p2 = rng.integers(0, 3, size=(O, I), dtype=np.uint8)           # fields t + 1
    words = np.zeros((O, I // 16), np.uint32)
    for k in range(16):
        words |= p2[:, k::16].astype(np.uint32) << np.uint32(2 * k)
    scale = rng.uniform(0.02, 0.2, O).astype(np.float32)
    x = rng.standard_normal((M, I)).astype(np.float32)
    y = torch.full((M, O), 3.0, dtype=torch.float32, device=DEV)
    ctx.ternary_gemv(_t(x), _t(words.view(np.int32)), _t(scale), y, M, I, O)
    ref64 = (x.astype(np.float64) @ (p2.astype(np.float64) - 1.0).T) * scale.astype(np.float64)
    assert rel_l2(y.cpu().numpy(), ref64) <= 1e-5
    if M == 1:      # and the checker's own 2-bit decoder agrees with the layout used here
        assert rel_l2(orc.ternary_gemv(x, words, scale, f64=True), ref64) <= 1e-12


def test_workspace_growth_is_refused_while_a_recorded_batch_is_alive(orc):
    """A recorded batch holds addresses inside the context's grow-only workspace; a later call that needs a larger
    workspace must be refused (with the reason) instead of moving the workspace under the batch."""
    from motifcl_b200 import Context
    c2 = Context(0)
    try:
        def products(n_tokens, I, O):
            rng = np.random.default_rng(n_tokens)
            st = synth.counters(7, 3, O, I).reshape(-1)
            x = _t(rng.standard_normal((n_tokens, I)).astype(np.float32))
            y = torch.empty(n_tokens, O, dtype=torch.float32, device=DEV)
            d_st, d_sc = _t(st), _t(np.full(O, 0.1, np.float32))
            torch.cuda.synchronize()
            return lambda: c2.counter_forward(x, d_st, d_sc, y, n_tokens, I, O, 11)
        c2.set_gemm_mode("tensor")
        small, big = products(256, 2048, 256), products(512, 2048, 2048)
        small()
        c2.finish()
        c2.batch_begin()
        small()
        batch = c2.batch_end()
        with pytest.raises(MotifclCudaError) as e:
            big()
        assert "recorded batch" in e.value.message
        batch.launch()
        c2.finish()
        batch.close()
        big()               # with the batch gone the workspace may grow
        c2.finish()
    finally:
        c2.close()



def test_peer_allreduce_of_one_rank_copies_its_partial(ctx):
    """mcl_cuda_peer_allreduce_f32 with a single rank: the hand-shake is with itself and the sum is the partial.  Both
    parities, several calls in a row."""
    from motifcl_b200.peer import PeerReducer
    red = PeerReducer(ctx, 4096)
    try:
        out = torch.zeros(4096, dtype=torch.float32, device=DEV)
        for k in range(5):
            n = 4096 if k % 2 == 0 else 1024
            src = torch.randn(n, device=DEV)
            red.partial(n).copy_(src)
            red.allreduce(out, n)
            ctx.finish()
            assert torch.equal(out[:n], src)
    finally:
        red.close()


def test_peer_allreduce_gives_up_when_a_rank_never_arrives(ctx):
    """A table that names a second rank whose flag nobody writes: the kernel's wait runs out (2 s), the context reports
    code 31 at the next finish, and the context stays usable."""
    import ctypes as C
    from motifcl_b200.peer import PeerReducer, FLAG_WORDS
    red = PeerReducer(ctx, 1024)
    try:
        vp = C.c_void_p * 2
        flags = vp(red._own, red._own + 192)                 # "rank 1": spare words of the flag area; nobody signals for it
        data = vp(red._own + FLAG_WORDS * 4, red._own + FLAG_WORDS * 4)
        out = torch.zeros(1024, dtype=torch.float32, device=DEV)
        ctx._check(ctx._lib.mcl_cuda_peer_allreduce_f32(ctx._ctx, data, flags, 0, 2, 1024, 1024, 1, C.c_void_p(out.data_ptr())))     # parity 1
        with pytest.raises(RuntimeError, match="peer all-reduce"):
            ctx.finish()
        red.seq = 1                                           # the failed call took number 1 and parity 1
        red.partial(1024).fill_(2.0)
        red.allreduce(out, 1024)
        ctx.finish()
        assert torch.all(out == 2.0)
    finally:
        red.close()

