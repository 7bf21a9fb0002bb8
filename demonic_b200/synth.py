"""Seeded synthetic inputs with the distributions the benchmark configurations
name: bf16 weights drawn N(0, 0.02) and rounded to nearest-even, f32
activations drawn U(-1, 1).  They stand in for real model weights (no public
dataset is involved).  Default seed 0xDEC0DE, the reference oracle's
(tools/numpy_oracle.py:192)."""
from __future__ import annotations

import numpy as np

DEFAULT_SEED = 0xDEC0DE


def f32_to_bf16_rne(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """Widen bf16 bit patterns (bits << 16; compiler/src/jit.rs:29224-29227)."""
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_weights(rng: np.random.Generator, shape, std: float = 0.02) -> np.ndarray:
    """bf16 bit patterns of N(0, std) values, generated in 64 Mi-element slabs."""
    n = int(np.prod(shape))
    out = np.empty(n, np.uint16)
    step = 1 << 26
    for i in range(0, n, step):
        j = min(n, i + step)
        out[i:j] = f32_to_bf16_rne(rng.standard_normal(j - i, dtype=np.float32) * np.float32(std))
    return out.reshape(shape)


def f32_weights(rng: np.random.Generator, shape, std: float = 0.02) -> np.ndarray:
    return (rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(std)).reshape(shape)


def activations(rng: np.random.Generator, shape) -> np.ndarray:
    """f32 U(-1, 1)."""
    return rng.uniform(-1.0, 1.0, int(np.prod(shape))).astype(np.float32).reshape(shape)


def gemv_bytes(n_out: int, k: int, wbytes: int = 2, m: int = 1) -> int:
    """Algorithmic bytes of one GEMV: weights once + x + y."""
    return n_out * k * wbytes + 4 * k * m + 4 * n_out * m


def gemv_flops(n_out: int, k: int, m: int = 1) -> int:
    return 2 * n_out * k * m
