"""CPU tests: the oracle restatement is pinned against (a) outputs of the compiled reference
stored in tests/golden/golden.npz, (b) the reference tests' known-answer vectors, and
(c) the compiled reference itself when oracle/_ref is present."""
import hashlib

import numpy as np
import pytest

from cases import all_cases
from motifcl_b200 import codec

CASES = {c["name"]: c for c in all_cases()}


def _hy(c):
    return c["lr"], c["lr_scale"], c["beta"], c["eps"], c["seed"]


@pytest.mark.parametrize("name", list(CASES))
def test_inputs_match_digest(name, golden):
    c = CASES[name]
    h = hashlib.sha256()
    for k in ("state", "scale", "v", "x", "dy"):
        h.update(np.ascontiguousarray(c[k]).tobytes())
    assert h.digest() == golden[f"{name}/digest"].tobytes(), "input generator drifted from golden"


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_dense_update_matches_reference(name, orc, golden):
    c = CASES[name]
    gw = orc.grad_w(c["dy"], c["x"])
    st, sc, v, p2 = orc.update_dense(c["state"], c["scale"], c["v"], gw, c["C"], c["I"], c["O"], 0, *_hy(c))
    assert np.array_equal(st, golden[f"{name}/dense_state"])       # bit-exact bytes
    assert np.array_equal(sc.view(np.uint32), golden[f"{name}/dense_scale"].view(np.uint32))
    assert np.array_equal(v.view(np.uint32), golden[f"{name}/dense_v"].view(np.uint32))
    assert not np.array_equal(st, c["state"])
    if p2 is not None:   # derived artifact: field == t + 1 of the new state
        t, _ = codec.decode(codec.unpack_codes(st.reshape(c["O"], -1), c["I"]), c["C"])
        assert np.array_equal(codec.unpack2(p2, c["I"]), (t + 1).astype(np.uint8))
        assert np.array_equal(p2, orc.pack2(st, c["C"], c["I"], c["O"]))


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_fused_update_matches_reference(name, orc, golden):
    c = CASES[name]
    st, sc, v, _ = orc.update_fused(c["state"], c["scale"], c["v"], c["dy"], c["x"], c["C"], *_hy(c))
    assert np.array_equal(st, golden[f"{name}/dense_state"])
    assert np.array_equal(sc.view(np.uint32), golden[f"{name}/dense_scale"].view(np.uint32))
    assert np.array_equal(v.view(np.uint32), golden[f"{name}/dense_v"].view(np.uint32))


@pytest.mark.parametrize("name", [n for n in CASES if CASES[n]["O"] * CASES[n]["I"] < 10000])
def test_oracle_decode_and_grad_x_match_reference(name, orc, golden):
    c = CASES[name]
    w = orc.decode_weight(c["state"], c["scale"], c["C"], c["I"], c["O"])
    assert np.array_equal(w, golden[f"{name}/weight"])
    gx = orc.backward_input(c["dy"], c["state"], c["scale"], c["C"], c["I"])
    assert np.array_equal(gx, golden[f"{name}/grad_x"])


def test_row_shard_equals_full_matrix(orc):
    """A row shard with row_offset updates exactly like the same rows of the whole layer."""
    c = CASES["wide"]
    gw = orc.grad_w(c["dy"], c["x"])
    full = orc.update_dense(c["state"], c["scale"], c["v"], gw, c["C"], c["I"], c["O"], 0, *_hy(c))
    rb = c["I"] // 4 * 3
    r0, nr = 16, 12
    part = orc.update_dense(c["state"][r0 * rb:(r0 + nr) * rb], c["scale"][r0:r0 + nr], c["v"][r0:r0 + nr],
                            gw[r0:r0 + nr], c["C"], c["I"], nr, r0, *_hy(c))
    assert np.array_equal(part[0], full[0][r0 * rb:(r0 + nr) * rb])
    assert np.array_equal(part[1], full[1][r0:r0 + nr])
    assert np.array_equal(part[3], full[3][r0:r0 + nr])


def test_known_answer_vectors_of_reference_tests(orc):
    """MotifCL tests/test_vulkan_runtime_standalone.cpp:579-640: hand-packed codes for
    t = {1,0,-1,1 / 0,1,1,-1}, C = 3, scales {0.5, 2.0}."""
    C = 3
    tern = np.array([[1, 0, -1, 1], [0, 1, 1, -1]])
    state = codec.pack_codes(codec.encode(tern, np.zeros_like(tern), C)).reshape(-1)
    scale = np.array([0.5, 2.0], np.float32)
    w = orc.decode_weight(state, scale, C, 4, 2)
    assert np.array_equal(w, np.array([[0.5, 0.0, -0.5, 0.5], [0.0, 2.0, 2.0, -2.0]], np.float32))
    go = np.array([[1.0, 2.0], [-1.0, 0.5]], np.float32)
    gx = orc.backward_input(go, state, scale, C, 4)
    expect = go[:, :1] * scale[0] * tern[0] + go[:, 1:] * scale[1] * tern[1]
    assert np.allclose(gx, expect, atol=1e-6)
    # tests/test_vulkan_backend.cpp:578-645 forward check: y = x w^T within 1e-5
    x = np.array([[1.0, 2.0, -1.0, 0.5], [-0.25, 0.75, 1.5, -2.0]], np.float32)
    y = orc.forward(x, state, scale, C, 2)
    assert np.allclose(y, x @ w.T, atol=1e-5)


def test_code_63_decodes_like_the_reference_formulas(orc):
    """Code 63 is unreachable for C = 11 but defined by the integer formulas
    (MotifCL kernels/compact_counter.cl:7-12): t = 63/21 - 1 = 2, c = 63 % 21 - 10 = -10."""
    state = codec.pack_codes(np.array([[63, 62, 0, 31]], np.uint8)).reshape(-1)
    w = orc.decode_weight(state, np.array([1.0], np.float32), 11, 4, 1)
    assert w.tolist() == [[2.0, 1.0, -1.0, 0.0]]


def test_gemm_restatements_agree_with_float64(orc):
    rng = np.random.default_rng(5)
    A = rng.standard_normal((33, 40)).astype(np.float32)
    B = rng.standard_normal((40, 48)).astype(np.float32)
    for ta, tb in [(False, False), (True, False), (False, True)]:
        a = A.T.copy() if ta else A
        b = B.T.copy() if tb else B
        c = orc.matmul(a, b, 33, 40, 48, ta, tb)
        c64 = orc.matmul(a, b, 33, 40, 48, ta, tb, f64=True)
        assert np.allclose(c, A.astype(np.float64) @ B.astype(np.float64), atol=1e-4)
        assert np.allclose(c64, A.astype(np.float64) @ B.astype(np.float64), atol=1e-12)


def test_ternary_gemv_oracle_equals_forward(orc):
    c = CASES["cfg1"]
    p2 = orc.pack2(c["state"], c["C"], c["I"], c["O"])
    x = c["x"][:4].copy()
    assert np.array_equal(orc.ternary_gemv(x, p2, c["scale"]), orc.forward(x, c["state"], c["scale"], c["C"], c["O"]))


def test_oracle_against_compiled_reference_when_present(orc):
    """Direct comparison with oracle/_ref (only where the reference tree was available to build it)."""
    import oracle
    if oracle.ref is None:
        pytest.skip("compiled reference (oracle/_ref) not built on this machine")
    rng = np.random.default_rng(11)
    O, I, N, C = 19, 132, 9, 7
    state = codec.pack_codes(rng.integers(0, 3 * (2 * C - 1), size=(O, I)).astype(np.uint8)).reshape(-1)
    scale = rng.uniform(0.02, 0.2, O).astype(np.float32)
    v = rng.uniform(1e-4, 1e-2, O).astype(np.float32)
    x = rng.standard_normal((N, I)).astype(np.float32)
    dy = (0.05 * rng.standard_normal((N, O))).astype(np.float32)
    hy = (0.3, 0.02, 0.95, 1e-4, 31337)
    a = orc.update_fused(state, scale, v, dy, x, C, *hy)
    b = oracle.ref.update_fused(state, scale, v, dy, x, C, *hy)
    for u, w in zip(a[:3], b):
        assert np.array_equal(u, w)
    k, n = 31, 17   # tests/test_native_matmul.cpp:54-107 shape
    av = rng.standard_normal(k).astype(np.float32)
    bm = rng.standard_normal((k, n)).astype(np.float32)
    assert np.array_equal(orc.matmul_m1(av, bm), oracle.ref.matmul_m1(av, bm))
