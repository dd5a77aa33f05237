"""Seeded synthetic inputs of the shapes the benchmarks name.

Real checkpoints are not available offline, so weights are synthesised the way
the benchmark configurations describe them: per output row a 2^bits-entry fp16
palette drawn N(0, sigma) and sorted ascending, indices uniform, packed
LSB-first; payload = all palettes then all index rows, i.e. the byte string
``CImageWriter::append_palettized`` stores (src/quantization/cimage.rs:98-125,
assembled at src/lut/compiler.rs:50-61).  Activations are fp16 ~ N(0, 1).
"""
from __future__ import annotations

import numpy as np

SEED0 = 0xC1A55E5


def payload_bytes(dim_m: int, dim_n: int, bits: int = 4) -> int:
    return dim_m * (2 << bits) + dim_m * (dim_n * bits // 8)


def make_payload(dim_m: int, dim_n: int, bits: int = 4, seed: int = 0, sigma: float = 0.02) -> np.ndarray:
    """Split-block palettized payload as uint8[payload_bytes]."""
    assert bits in (2, 4) and (dim_n * bits) % 32 == 0
    rng = np.random.default_rng([SEED0, seed, dim_m, dim_n, bits])
    n_ent = 1 << bits
    pal = np.sort(rng.normal(0.0, sigma, size=(dim_m, n_ent)).astype(np.float32), axis=1)
    pal16 = pal.astype(np.float16).view(np.uint16)
    idx_bytes = rng.integers(0, 256, size=(dim_m, dim_n * bits // 8), dtype=np.uint8)
    out = np.empty(payload_bytes(dim_m, dim_n, bits), np.uint8)
    out[: dim_m * n_ent * 2] = pal16.astype("<u2").view(np.uint8).reshape(-1)
    out[dim_m * n_ent * 2:] = idx_bytes.reshape(-1)
    return out


def make_activation(n, seed: int = 0, scale: float = 1.0) -> np.ndarray:
    """fp16 ~ N(0, scale) as uint16 bit patterns; ``n`` may be a shape tuple."""
    rng = np.random.default_rng([SEED0, 0xA11, seed])
    return (rng.normal(0.0, scale, size=n).astype(np.float32)).astype(np.float16).view(np.uint16)


def make_prompt(n: int, vocab: int, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng([SEED0, 0x70C, seed])
    return rng.integers(0, vocab, size=n, dtype=np.uint32)


def gemv_algorithmic_bytes(dim_m: int, dim_n: int, bits: int = 4) -> int:
    """Bytes one palettized GEMV must move: indices + palettes + x + y."""
    return dim_m * dim_n * bits // 8 + dim_m * (2 << bits) + 2 * dim_n + 2 * dim_m
