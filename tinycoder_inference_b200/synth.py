"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (i.i.d. N(0,1) f32, already-rotated Q/K, scale
1/sqrt(hd)); a counter-based generator so any shard can regenerate its slice."""
from __future__ import annotations

import numpy as np

SEED_BASE = 0x7C0DE000

# name -> (nHeads, nKV, hd)
SHAPES = {
    "qwen2.5-0.5b": (14, 2, 64),
    "qwen2.5-7b": (28, 4, 128),
    "qwen2.5-32b": (40, 8, 128),
}


def rng(config: int, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[SEED_BASE + config, stream]))


def normal(config: int, stream: int, shape) -> np.ndarray:
    return rng(config, stream).standard_normal(shape, dtype=np.float32)


def ragged_lengths(config: int, n: int, lo: int = 512, hi: int = 32768) -> np.ndarray:
    """n context lengths uniform in [lo, hi]."""
    r = rng(config, 99)
    return (lo + r.integers(0, hi - lo + 1, size=n)).astype(np.uint32)
