"""Seeded synthetic tensors in the distributions the benchmark configurations name.

Packed weights: 2/4-bit codes uniform, per-block f16 scales log-normal (mu=-4, sigma=0.5);
activations ~ N(0, 1). numpy's Philox bit generator makes every array a pure function of
(seed, shape), so the CPU oracle and the GPU see identical bytes.
"""
from __future__ import annotations

import numpy as np

from . import _native as N

BLOCK_LEN = 64
BLOCK_BYTES = {N.Q2B64: 18, N.Q4B64: 34}


def _rng(seed: int, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, stream]))


def packed_weights(dtype: int, rows: int, columns: int, seed: int) -> np.ndarray:
    """Row-major canonical blocks [f16 scale LE][code bytes] (quant.rs:117-122,181-186)."""
    bb = BLOCK_BYTES[dtype]
    blocks = rows * (columns // BLOCK_LEN)
    rng = _rng(seed, 1)
    out = np.empty((blocks, bb), dtype=np.uint8)
    out[:, 2:] = rng.integers(0, 256, size=(blocks, bb - 2), dtype=np.uint8)
    scales = np.exp(rng.normal(-4.0, 0.5, size=blocks)).astype(np.float16)
    out[:, :2] = scales.view(np.uint8).reshape(blocks, 2)
    return out.reshape(-1)


def activations(n: int, seed: int, positions: int = 1) -> np.ndarray:
    x = _rng(seed, 2).standard_normal(size=(positions, n)).astype(np.float32)
    return x[0] if positions == 1 else x


def recovery_scales_f16(n: int, seed: int, stream: int) -> np.ndarray:
    """f16 scales ~ U(0.75, 1.25) as little-endian bytes (ScaleSlice::F16Le)."""
    s = _rng(seed, stream).uniform(0.75, 1.25, size=n).astype(np.float16)
    return s.view(np.uint8).copy()


def bias(n: int, seed: int) -> np.ndarray:
    return (_rng(seed, 5).standard_normal(size=n) * 0.1).astype(np.float32)
