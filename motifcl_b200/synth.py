"""Seeded synthetic inputs for the counter-linear path.

The reference trains on a tokenised public corpus that is not available here; these
tensors stand in for it with the reference's shapes and value distributions: counters
uniform over the 64 six-bit codes (k ~ U{-32..31}, code = k + 32), fp32 activations ~ N(0,1),
upstream gradients ~ N(0, sigma).  Everything is generated on the host with
numpy.random.default_rng so a CPU checker and the GPU read identical bytes.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import codec

BASE_SEED = 20261125


def seed_for(cfg: int, linear_index: int, tensor_id: int) -> int:
    """tensor_id: 0 counters, 1 X, 2 dY, 3 dW, 4 scale/v."""
    return BASE_SEED + 1000 * cfg + 10 * linear_index + tensor_id


@dataclass
class LinearShape:
    name: str
    out_features: int
    in_features: int


def stories15m_linears() -> list[LinearShape]:
    """stories15M-shaped stack: dim 288, 6 layers, FFN 768; q,k,v,o 288x288, w1,w3 768x288,
    w2 288x768 -- 42 counter linears (the reference trainer fuses w1/w3 into one 288->1536
    layer, tools/train_ternary15m.cpp:174; the weight count is the same)."""
    out = []
    for l in range(6):
        for n in ("wq", "wk", "wv", "wo"):
            out.append(LinearShape(f"l{l}.{n}", 288, 288))
        out.append(LinearShape(f"l{l}.w1", 768, 288))
        out.append(LinearShape(f"l{l}.w3", 768, 288))
        out.append(LinearShape(f"l{l}.w2", 288, 768))
    return out


def llama_linears(dim: int, ffn: int, layers: int, kv_dim: int | None = None) -> list[LinearShape]:
    kv = kv_dim or dim
    out = []
    for l in range(layers):
        out += [LinearShape(f"l{l}.wq", dim, dim), LinearShape(f"l{l}.wk", kv, dim),
                LinearShape(f"l{l}.wv", kv, dim), LinearShape(f"l{l}.wo", dim, dim),
                LinearShape(f"l{l}.w1", ffn, dim), LinearShape(f"l{l}.w3", ffn, dim),
                LinearShape(f"l{l}.w2", dim, ffn)]
    return out


def counters(cfg: int, idx: int, O: int, I: int) -> np.ndarray:
    """Packed state bytes [O, I/4*3]."""
    rng = np.random.default_rng(seed_for(cfg, idx, 0))
    k = rng.integers(-32, 32, size=(O, I), dtype=np.int8)
    return codec.pack_codes((k.astype(np.int16) + 32).astype(np.uint8))


def scale_v(cfg: int, idx: int, O: int, I: int, randomised: bool = False):
    if not randomised:   # the reference's initial values, src/nn/compact_counter.cpp:80-82
        return (np.full(O, np.float32(np.sqrt(np.float32(3.0) / (np.float32(2.0) * np.float32(I)))), np.float32),
                np.zeros(O, np.float32))
    rng = np.random.default_rng(seed_for(cfg, idx, 4))
    return (rng.uniform(0.02, 0.2, O).astype(np.float32), rng.uniform(1e-4, 1e-2, O).astype(np.float32))


def activations(cfg: int, idx: int, N: int, I: int) -> np.ndarray:
    return np.random.default_rng(seed_for(cfg, idx, 1)).standard_normal((N, I), dtype=np.float32)


def upstream_grad(cfg: int, idx: int, N: int, O: int, sigma: float) -> np.ndarray:
    g = np.random.default_rng(seed_for(cfg, idx, 2)).standard_normal((N, O), dtype=np.float32)
    return (g * np.float32(sigma)).astype(np.float32)


def weight_grad(cfg: int, idx: int, O: int, I: int, sigma: float, N: int) -> np.ndarray:
    """Stand-in for dY^T X at sizes where forming it on the CPU is too slow."""
    g = np.random.default_rng(seed_for(cfg, idx, 3)).standard_normal((O, I), dtype=np.float32)
    return (g * np.float32(sigma * np.sqrt(N))).astype(np.float32)
