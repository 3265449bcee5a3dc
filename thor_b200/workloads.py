"""Seeded synthetic inputs for the five benchmark configurations.

The reference measures on no dataset; every configuration is defined by a shape, a dtype and a
value distribution, generated here from a counter-based generator (numpy Philox) so that any row
shard can be produced independently and host and device copies agree bit for bit.
"""
from __future__ import annotations

import numpy as np

C1_EDGE_VALUES = np.array(
    [
        0.0, -0.0,
        # fp16 subnormal range, including the exact ties 2^-25 and 3*2^-25
        2.0 ** -25, 3 * 2.0 ** -25, 2.0 ** -24, 5 * 2.0 ** -25, 2.0 ** -20, 2.0 ** -14 * (1 - 2.0 ** -11), 2.0 ** -14, 2.0 ** -26, -(2.0 ** -25), 1e-30,
        # round-to-nearest-even tie patterns k*2^-10 + 2^-11 in [1, 2)
        1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11, 1 + 5 * 2.0 ** -11, 1.5 + 2.0 ** -11, 2 - 2.0 ** -11, -(1 + 2.0 ** -11), -(1 + 3 * 2.0 ** -11),
        # overflow boundary
        65504.0, 65519.996, 65520.0, 1e5, -65504.0, -65519.996, -65520.0, np.inf, -np.inf,
    ],
    dtype=np.float32,
)


def _rng(seed: int, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=seed, counter=[0, 0, 0, stream]))


def cast_input(n: int = 1 << 24, seed: int = 0, edge_density: float = 1e-3) -> np.ndarray:
    """Configuration 1: fp32 values uniform in [-4, 4]; at `edge_density` the value is replaced by
    one of C1_EDGE_VALUES (+-0, fp16-subnormal magnitudes, RNE ties, overflow-to-inf), cycling."""
    x = _rng(seed, 0).uniform(-4.0, 4.0, n).astype(np.float32)
    mask = _rng(seed, 1).random(n) < edge_density
    idx = np.flatnonzero(mask)
    x[idx] = C1_EDGE_VALUES[np.arange(idx.size) % C1_EDGE_VALUES.size]
    return x
