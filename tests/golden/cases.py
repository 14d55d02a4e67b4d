"""Input definitions of the golden parity cases (shared by make_golden.py and the tests).

Each case mirrors a reference test or a benchmark configuration at a size the compiled
reference finishes in seconds.  Inputs are regenerated from seeds; only OUTPUTS of the
compiled reference are stored in golden.npz.
"""
from __future__ import annotations

import numpy as np

from motifcl_b200 import codec, synth
from motifcl_b200.counter import initial_ternary


def lcg_fill(n: int, seed: int, scale: float) -> np.ndarray:
    """fill_deterministic of the reference's test utilities
    (MotifCL tests/vulkan_p0_test_utils.hpp:50-59)."""
    out = np.empty(n, np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        unit = np.float32(np.float32((s >> 8) & 0xFFFF) / np.float32(32767.5)) - np.float32(1.0)
        out[i] = unit * np.float32(scale)
    return out


def layer_init(seed, I, O, C, init_gain=1.0):
    """Initial tensors of a CounterStateLinear (MotifCL src/nn/compact_counter.cpp:64-84)."""
    t = initial_ternary(seed, O * I).reshape(O, I)
    st = codec.pack_codes(codec.encode(t, np.zeros_like(t), C)).reshape(-1)
    s0 = np.float32(init_gain) * np.sqrt(np.float32(3.0) / (np.float32(2.0) * np.float32(I)))
    return st, np.full(O, s0, np.float32), np.zeros(O, np.float32)


def case_fused_witness():
    """tests/test_vulkan_counter_fused.cpp:55-73: rows 37, in 68, out 35, C 3, lr 1, lr_scale .05,
    eps 1e-6, seed 777; inputs from the LCG fill."""
    N, I, O, C = 37, 68, 35, 3
    st, sc, v = layer_init(777, I, O, C)
    return dict(name="fused_witness", N=N, I=I, O=O, C=C, state=st, scale=sc, v=v,
                x=lcg_fill(N * I, 0x1234, 0.8).reshape(N, I), dy=lcg_fill(N * O, 0x5678, 0.9).reshape(N, O),
                lr=1.0, lr_scale=0.05, beta=0.9, eps=1e-6, seed=777)


def case_cross_backend():
    """tests/test_vulkan_backend.cpp:1181-1199: in 8, out 2, C 3, N 2, layer seed 42, update seed 777."""
    N, I, O, C = 2, 8, 2, 3
    st, sc, v = layer_init(42, I, O, C)
    x = np.array([np.float32(0.2) * np.float32(i % 5) - np.float32(0.4) for i in range(N * I)], np.float32)
    dy = np.array([np.float32(0.3) * np.float32(i % 3) - np.float32(0.3) for i in range(N * O)], np.float32)
    return dict(name="cross_backend", N=N, I=I, O=O, C=C, state=st, scale=sc, v=v, x=x.reshape(N, I),
                dy=dy.reshape(N, O), lr=0.05, lr_scale=0.01, beta=0.9, eps=1e-8, seed=777)


def case_cfg1(randomised=False, name="cfg1", lr=3e-3, lr_scale=0.0, sigma=0.02, seed=12345):
    """Single counter linear: X[256,288] ~ N(0,1), counters uniform over the 64 codes
    (including the unreachable code 63), dY ~ N(0, 0.02), reference default hyper-parameters."""
    N, I, O, C = 256, 288, 288, 11
    st = synth.counters(1, 0, O, I).reshape(-1)
    sc, v = synth.scale_v(1, 0, O, I, randomised)
    return dict(name=name, N=N, I=I, O=O, C=C, state=st, scale=sc, v=v,
                x=synth.activations(1, 0, N, I), dy=synth.upstream_grad(1, 0, N, O, sigma),
                lr=lr, lr_scale=lr_scale, beta=0.9, eps=1e-3, seed=seed)


def case_wide():
    """Long rows (in 1024 = four lane sweeps per row) with the rebase term active and a
    learning rate large enough to force carries and clamps."""
    N, I, O, C = 48, 1024, 40, 11
    st = synth.counters(9, 1, O, I).reshape(-1)
    sc, v = synth.scale_v(9, 1, O, I, True)
    return dict(name="wide", N=N, I=I, O=O, C=C, state=st, scale=sc, v=v,
                x=synth.activations(9, 1, N, I), dy=synth.upstream_grad(9, 1, N, O, 0.05),
                lr=0.5, lr_scale=0.05, beta=0.9, eps=1e-3, seed=4242)


def all_cases():
    return [case_fused_witness(), case_cross_backend(), case_cfg1(),
            case_cfg1(True, "cfg1_rebase", lr=0.05, lr_scale=0.05, seed=999), case_wide()]
