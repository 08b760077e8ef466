"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset is involved: the configurations are synthetic by definition).

Streams are counter-based (numpy Philox), keyed by (config id, tensor id), so any
rank can regenerate exactly its own slice.
"""
from __future__ import annotations

import numpy as np


def _gen(config_id: int, tensor_id: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=config_id * 1000 + tensor_id))


def normal(shape, config_id: int, tensor_id: int, std: float = 1.0) -> np.ndarray:
    return (_gen(config_id, tensor_id).standard_normal(shape, dtype=np.float32) * np.float32(std))


def normal_with_outliers(shape, config_id: int, tensor_id: int, frac: float = 0.01,
                         factor: float = 8.0) -> np.ndarray:
    """N(0,1) with a Bernoulli(frac) subset multiplied by `factor` (independent stream)."""
    x = normal(shape, config_id, tensor_id)
    mask = _gen(config_id, tensor_id + 500).random(shape, dtype=np.float32) < frac
    x[mask] *= np.float32(factor)
    return x


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even BF16 -> fp32, in numpy (for host-side oracles)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(x.shape)
