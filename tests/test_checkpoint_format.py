"""MotifCL tensor files (.mt) for the counter layers: byte layout as src/serialization.cpp writes it
(magic, dtype index, rank, dims, byte count, four quantisation fields, payload), version-1 files, the
trainer's per-linear file names and the reference's error cases."""
import os
import struct

import numpy as np
import pytest

from motifcl_b200 import checkpoint as ck
from motifcl_b200 import codec, synth


def test_tensor_file_bytes(tmp_path):
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    p = str(tmp_path / "a.mt")
    ck.save_tensor(p, a)
    raw = open(p, "rb").read()
    # the write order of write_tensor_payload (src/serialization.cpp:38-58)
    expect = (b"MCLTEN2\0" + struct.pack("<i", 0) + struct.pack("<Q", 2) + struct.pack("<qq", 2, 3) +
              struct.pack("<Q", 24) + struct.pack("<f", 0.0) + struct.pack("<i", 0) + struct.pack("<i", 0) +
              struct.pack("<q", 0) + a.tobytes())
    assert raw == expect
    back = ck.load_tensor(p)
    assert back.dtype == np.float32 and np.array_equal(back, a)


def test_version1_file_and_types(tmp_path):
    st = np.arange(12, dtype=np.uint8)
    p = str(tmp_path / "v1.mt")
    with open(p, "wb") as f:      # read_tensor_payload_v1: no quantisation fields (src/serialization.cpp:60-73)
        f.write(b"MCLTEN1\0" + struct.pack("<iQ", 3, 1) + struct.pack("<q", 12) + struct.pack("<Q", 12) + st.tobytes())
    back = ck.load_tensor(p)
    assert back.dtype == np.uint8 and np.array_equal(back, st)
    for arr in (np.array([1, -2, 3], dtype=np.int32), np.array([0.5, 2.0], dtype=np.float16)):
        q = str(tmp_path / "t.mt")
        ck.save_tensor(q, arr)
        assert np.array_equal(ck.load_tensor(q), arr) and ck.load_tensor(q).dtype == arr.dtype


def test_rejects_what_the_reference_rejects(tmp_path):
    p = str(tmp_path / "bad.mt")
    open(p, "wb").write(b"NOTMAGIC" + b"\0" * 64)
    with pytest.raises(ck.MotifclFormatError, match="magic"):
        ck.load_tensor(p)
    # byte count that does not match dtype x shape (MCL_CHECK at src/serialization.cpp:67,88)
    open(p, "wb").write(b"MCLTEN2\0" + struct.pack("<iQ", 0, 1) + struct.pack("<q", 4) + struct.pack("<Q", 12) +
                        struct.pack("<fiiq", 0.0, 0, 0, 0) + b"\0" * 12)
    with pytest.raises(ck.MotifclFormatError, match="byte size"):
        ck.load_tensor(p)
    # truncated payload
    open(p, "wb").write(b"MCLTEN2\0" + struct.pack("<iQ", 0, 1) + struct.pack("<q", 4) + struct.pack("<Q", 16) +
                        struct.pack("<fiiq", 0.0, 0, 0, 0) + b"\0" * 8)
    with pytest.raises(ck.MotifclFormatError, match="payload"):
        ck.load_tensor(p)
    with pytest.raises(ck.MotifclFormatError):
        ck.save_tensor(p, np.zeros(3, dtype=np.float64))


def test_counter_linear_files_round_trip(tmp_path):
    O, I = 24, 64
    st = synth.counters(1, 3, O, I).reshape(-1)
    sc, v = synth.scale_v(1, 3, O, I, randomised=True)
    pre = ck.block_prefix(2, "wup")
    assert pre == "l2_wup"
    ck.save_counter_linear(str(tmp_path), pre, st, sc, v)
    assert sorted(os.listdir(tmp_path)) == ["l2_wup_scale.mt", "l2_wup_state.mt", "l2_wup_v.mt"]
    st2, sc2, v2 = ck.load_counter_linear(str(tmp_path), pre)
    assert st2.shape == (O * I // 4 * 3,) and np.array_equal(st2, st)
    assert np.array_equal(sc2.view(np.uint32), sc.view(np.uint32)) and np.array_equal(v2.view(np.uint32), v.view(np.uint32))
    with pytest.raises(KeyError):
        ck.block_prefix(0, "w9")
    with pytest.raises(ck.MotifclFormatError):
        ck.save_counter_linear(str(tmp_path), "x", st[:-1], sc, v)


def test_packed2_export_matches_the_state(tmp_path):
    O, I, C = 8, 64, 11
    st = synth.counters(1, 5, O, I).reshape(-1)
    sc, _ = synth.scale_v(1, 5, O, I, randomised=True)
    t, _ = codec.decode(codec.unpack_codes(st.reshape(O, -1), I), C)
    f = (t + 1).astype(np.uint32).reshape(O, I // 16, 16)
    p2 = np.zeros((O, I // 16), dtype=np.uint32)
    for j in range(16):
        p2 |= f[..., j] << np.uint32(2 * j)
    assert np.array_equal(codec.unpack2(p2, I), (t + 1).astype(np.uint8))
    ck.export_packed2(str(tmp_path), "l0_wq", p2, sc)
    q2, s2 = ck.load_packed2(str(tmp_path), "l0_wq")
    assert q2.dtype == np.uint32 and np.array_equal(q2, p2) and np.array_equal(s2, sc)
    # field of weight m = t + 1 at bits 2(m % 16) of word m / 16
    m = 37
    assert ((q2[3, m // 16] >> (2 * (m % 16))) & 3) == t[3, m] + 1
