"""Host-side (numpy) view of the counter-state byte layout.

Mirrors the packing the reference does on the host when it builds a layer
(MotifCL src/nn/compact_counter.cpp:20-23,64-78) and the unpacking its tests do
(tests/test_counter_state.cpp:64-79): four 6-bit codes per 3 bytes,
code = (t+1)*(2C-1) + (c + C-1).
"""
from __future__ import annotations

import numpy as np


def encode(t: np.ndarray, c: np.ndarray, C: int) -> np.ndarray:
    lv = 2 * C - 1
    return ((t.astype(np.int32) + 1) * lv + (c.astype(np.int32) + (C - 1))).astype(np.uint8)


def decode(codes: np.ndarray, C: int):
    lv = 2 * C - 1
    z = codes.astype(np.int32)
    return z // lv - 1, z % lv - (C - 1)


def pack_codes(codes: np.ndarray) -> np.ndarray:
    """codes uint8 [..., in] (in % 4 == 0) -> bytes uint8 [..., in/4*3]."""
    c = codes.astype(np.uint32).reshape(*codes.shape[:-1], -1, 4)
    w = c[..., 0] | (c[..., 1] << 6) | (c[..., 2] << 12) | (c[..., 3] << 18)
    out = np.stack([w & 0xFF, (w >> 8) & 0xFF, (w >> 16) & 0xFF], axis=-1).astype(np.uint8)
    return out.reshape(*codes.shape[:-1], -1)


def unpack_codes(state: np.ndarray, in_features: int) -> np.ndarray:
    """bytes uint8 [..., in/4*3] -> codes uint8 [..., in]."""
    b = state.astype(np.uint32).reshape(*state.shape[:-1], -1, 3)
    w = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16)
    c = np.stack([(w >> (6 * k)) & 63 for k in range(4)], axis=-1).astype(np.uint8)
    return c.reshape(*state.shape[:-1], in_features)


def unpack2(packed2: np.ndarray, in_features: int) -> np.ndarray:
    """2-bit words uint32 [out, in/16] -> fields (t+1) uint8 [out, in]."""
    f = np.stack([(packed2 >> np.uint32(2 * j)) & np.uint32(3) for j in range(16)], axis=-1)
    return f.astype(np.uint8).reshape(packed2.shape[0], in_features)
