"""CPU tests of the host-side logic and of the C-ABI library as a binary (no compute calls)."""
import ctypes
import os
import re

import numpy as np
import pytest

import motifcl_b200 as mb
from motifcl_b200 import codec, synth
from motifcl_b200.counter import initial_ternary


def test_library_builds_loads_and_exports_every_declared_symbol():
    if not os.path.isfile(mb.LIB_PATH):
        mb.build_library()
    L = mb.lib()
    names = mb.declared_symbols()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_header_cites_a_reference_interface_for_every_entry_point():
    text = open(mb._lib.HEADER_PATH).read()
    assert "extern \"C\"" in text and "torch" not in text.lower()
    for cite in ("vulkan_backend.hpp", "compact_counter.cpp", "compact_counter.cl", "matmul.cpp"):
        assert cite in text


def test_no_device_is_reported_not_crashed():
    """Without a GPU, context creation is refused with a message -- the analogue of the
    reference's probe_vulkan_runtime().available() == false."""
    L = mb.lib()
    if L.mcl_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    ctx = ctypes.c_void_p()
    rc = L.mcl_cuda_create(0, ctypes.byref(ctx))
    assert rc == 5 and not ctx.value
    assert b"no CUDA device" in L.mcl_cuda_last_error(None)
    with pytest.raises(mb.MotifclCudaError):
        mb.Context(0)


def test_pack_unpack_roundtrip_and_oracle_agreement(orc):
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 64, size=(7, 36)).astype(np.uint8)
    st = codec.pack_codes(codes)
    assert st.shape == (7, 27)
    assert np.array_equal(codec.unpack_codes(st, 36), codes)
    assert np.array_equal(orc.pack_codes(codes.reshape(-1)), st.reshape(-1))
    t, c = codec.decode(codes, 11)
    assert np.array_equal(codec.encode(t, c, 11), codes)


def test_initial_state_matches_libstdcxx_stream():
    """First digits std::uniform_int_distribution<int>(-1,1) draws from std::mt19937(777),
    generated with g++ 13 / libstdc++ (the reference constructor's stream)."""
    assert initial_ternary(777, 8).tolist() == [-1, 0, -1, -1, -1, 0, 0, -1]


def test_synthetic_shapes_and_weight_counts():
    ls = synth.stories15m_linears()
    assert len(ls) == 42
    assert sum(l.out_features * l.in_features for l in ls) == 5_971_968
    assert sum(l.out_features for l in ls) == 17_856
    big = synth.llama_linears(2048, 5632, 22)
    assert sum(l.out_features * l.in_features for l in big) == 1_130_364_928
    st = synth.counters(1, 0, 288, 288)
    codes = codec.unpack_codes(st, 288)
    assert codes.min() == 0 and codes.max() == 63
    assert synth.seed_for(2, 3, 1) == 20261125 + 2000 + 30 + 1
