"""MotifCL tensor files (`.mt`) for the counter layers' persistent tensors.

MotifCL's trainer saves every counter linear as three tensor files, `<prefix>_state.mt`,
`<prefix>_scale.mt` and `<prefix>_v.mt` (tools/train_ternary15m.cpp:204-269), written by
`save_tensor` (src/serialization.cpp:38-58,121-126).  This module reads and writes that format
byte for byte, so a run trained through MotifCL (on any backend) can be continued or served from
here and the other way round, and adds an export of the derived 2-bit words for the decode GEMV.

File layout (little endian, no padding):
    char[8]  magic      "MCLTEN2\\0"  ("MCLTEN1\\0" is accepted on read: no quantisation fields)
    int32    dtype      index into MotifCL's DType enum (include/motifcl/core/dtype.hpp:8-22)
    uint64   ndim
    int64    dims[ndim]
    uint64   nbytes     must equal the storage size of dtype x shape
    float32  quant_scale            \\
    int32    has_quant_scales        | version 2 only; zero for the plain types used here
    int32    quant_scale_axis        |
    int64    quant_block_size       /
    bytes    payload[nbytes]
"""
from __future__ import annotations

import os
import struct

import numpy as np

MAGIC_V1 = b"MCLTEN1\0"
MAGIC_V2 = b"MCLTEN2\0"

# MotifCL's DType enum values for the plain (unquantised) types
DTYPE_F32, DTYPE_F16, DTYPE_I32, DTYPE_U8 = 0, 1, 2, 3
_NP_OF = {DTYPE_F32: np.float32, DTYPE_F16: np.float16, DTYPE_I32: np.int32, DTYPE_U8: np.uint8}
_CODE_OF = {np.dtype(np.float32): DTYPE_F32, np.dtype(np.float16): DTYPE_F16, np.dtype(np.int32): DTYPE_I32,
            np.dtype(np.uint8): DTYPE_U8}

LINEAR_NAMES = ("wq", "wk", "wv", "wo", "wup", "wdown")     # the trainer's names inside a block


class MotifclFormatError(ValueError):
    """The file is not a MotifCL tensor file this module can read (the reference raises MCL_CHECK)."""


def save_tensor(path: str, array: np.ndarray) -> None:
    """Write `array` as a version-2 tensor file (src/serialization.cpp:38-58,121-126)."""
    a = np.ascontiguousarray(array)
    if a.dtype not in _CODE_OF:
        raise MotifclFormatError(f"dtype {a.dtype} has no plain MotifCL tensor type (f32, f16, i32, u8)")
    with open(path, "wb") as f:
        f.write(MAGIC_V2)
        f.write(struct.pack("<iQ", _CODE_OF[a.dtype], a.ndim))
        for d in a.shape:
            f.write(struct.pack("<q", d))
        f.write(struct.pack("<Q", a.nbytes))
        f.write(struct.pack("<fiiq", 0.0, 0, 0, 0))
        f.write(a.tobytes())


def load_tensor(path: str) -> np.ndarray:
    """Read a version-1 or version-2 tensor file (src/serialization.cpp:60-103,128-135)."""
    with open(path, "rb") as f:
        buf = f.read()
    if len(buf) < 8:
        raise MotifclFormatError("failed to read serialization magic")
    magic = buf[:8]
    if magic not in (MAGIC_V1, MAGIC_V2):
        raise MotifclFormatError("serialization magic mismatch")
    pos = 8

    def take(fmt):
        nonlocal pos
        size = struct.calcsize(fmt)
        if pos + size > len(buf):
            raise MotifclFormatError("failed to read serialization stream")
        v = struct.unpack_from(fmt, buf, pos)
        pos += size
        return v

    dtype, ndim = take("<iQ")
    if ndim > 8:
        raise MotifclFormatError(f"implausible tensor rank {ndim}")
    dims = [take("<q")[0] for _ in range(ndim)]
    (nbytes,) = take("<Q")
    if magic == MAGIC_V2:
        _, has_scales, _, _ = take("<fiiq")
        if has_scales:
            raise MotifclFormatError("quantised tensors with scale tensors are not part of the counter path")
    if dtype not in _NP_OF:
        raise MotifclFormatError(f"tensor type {dtype} is not a plain type (f32, f16, i32, u8)")
    if any(d < 0 for d in dims):
        raise MotifclFormatError("negative dimension")
    numel = int(np.prod(dims, dtype=np.int64)) if dims else 1
    if numel * np.dtype(_NP_OF[dtype]).itemsize != nbytes:
        raise MotifclFormatError("serialized tensor byte size does not match dtype/shape")
    if pos + nbytes > len(buf):
        raise MotifclFormatError("failed to read tensor payload")
    return np.frombuffer(buf, dtype=_NP_OF[dtype], count=numel, offset=pos).reshape(dims).copy()


def save_counter_linear(directory: str, prefix: str, state: np.ndarray, scale: np.ndarray, v: np.ndarray) -> None:
    """The three files the trainer writes per counter linear (tools/train_ternary15m.cpp:216-222): the packed
    6-bit state as a flat U8 tensor [out * in/4 * 3] (src/nn/compact_counter.cpp:78), scale and v as F32 [out]."""
    st = np.ascontiguousarray(state, dtype=np.uint8).reshape(-1)
    sc = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    vv = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
    if sc.shape != vv.shape or sc.size == 0 or st.size % (3 * sc.size) != 0:
        raise MotifclFormatError("state / scale / v do not describe one counter linear")
    save_tensor(os.path.join(directory, prefix + "_state.mt"), st)
    save_tensor(os.path.join(directory, prefix + "_scale.mt"), sc)
    save_tensor(os.path.join(directory, prefix + "_v.mt"), vv)


def load_counter_linear(directory: str, prefix: str):
    """-> (state u8 [out * in/4 * 3], scale f32 [out], v f32 [out]), checked for consistency."""
    st = load_tensor(os.path.join(directory, prefix + "_state.mt"))
    sc = load_tensor(os.path.join(directory, prefix + "_scale.mt"))
    vv = load_tensor(os.path.join(directory, prefix + "_v.mt"))
    if st.dtype != np.uint8 or sc.dtype != np.float32 or vv.dtype != np.float32:
        raise MotifclFormatError("checkpoint parameter dtype mismatch")
    if sc.ndim != 1 or sc.shape != vv.shape or st.ndim != 1 or sc.size == 0 or st.size % (3 * sc.size) != 0:
        raise MotifclFormatError("checkpoint parameter shape mismatch")
    return st, sc, vv


def block_prefix(layer: int, name: str) -> str:
    """File prefix of linear `name` (one of LINEAR_NAMES) in block `layer`, as the trainer names it."""
    if name not in LINEAR_NAMES:
        raise KeyError(name)
    return f"l{layer}_{name}"


def export_packed2(directory: str, prefix: str, packed2: np.ndarray, scale: np.ndarray) -> None:
    """Inference export of one layer: the 2-bit words (field t + 1, 16 weights per word, weight m in bits
    2(m%16)+1 : 2(m%16) of word m/16: the flat LSB-first layout of docs/BITNET_TERNARY_VULKAN_PLAN.md section
    3.4) as an I32 tensor [out, in/16] and the per-row scale as F32 [out].  MotifCL has no unsigned 32-bit
    tensor type; the bits are what counts."""
    p2 = np.ascontiguousarray(packed2)
    if p2.ndim != 2 or p2.dtype.itemsize != 4:
        raise MotifclFormatError("packed2 must be a [out, in/16] array of 32-bit words")
    sc = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    if sc.size != p2.shape[0]:
        raise MotifclFormatError("one scale per output row expected")
    save_tensor(os.path.join(directory, prefix + "_p2.mt"), p2.view(np.int32))
    save_tensor(os.path.join(directory, prefix + "_scale.mt"), sc)


def load_packed2(directory: str, prefix: str):
    """-> (packed2 u32 [out, in/16], scale f32 [out])"""
    p2 = load_tensor(os.path.join(directory, prefix + "_p2.mt"))
    sc = load_tensor(os.path.join(directory, prefix + "_scale.mt"))
    if p2.dtype != np.int32 or p2.ndim != 2 or sc.dtype != np.float32 or sc.shape != (p2.shape[0],):
        raise MotifclFormatError("not a packed2 export")
    return p2.view(np.uint32), sc
