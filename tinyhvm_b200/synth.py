"""Seeded synthetic inputs, identical on every machine and for every backend.

Generator: SplitMix64 in counter mode (element i of tensor t uses the state
seed ^ t, advanced i+1 times), uniform [0,1) from the top 24 bits, Normal(0,1)
by Box-Muller on two uniforms.  Everything is vectorised numpy so a 64 M-element
tensor takes a few seconds.
"""
from __future__ import annotations

import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(seed: int, n: int, start: int = 0) -> np.ndarray:
    """Outputs start+1 .. start+n of the SplitMix64 stream seeded with `seed`."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + _GOLD * np.arange(start + 1, start + n + 1, dtype=np.uint64)
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, tensor_index: int, n: int) -> np.ndarray:
    """U[0,1) as float32: top 24 bits / 2^24."""
    bits = splitmix64(seed ^ tensor_index, n)
    return ((bits >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / (1 << 24))).astype(np.float32)


def normal(seed: int, tensor_index: int, n: int, chunk: int = 1 << 21) -> np.ndarray:
    """N(0,1) as float32 by Box-Muller; element i uses stream outputs 2i+1 and 2i+2.
    Chunks are independent (counter mode), so they are filled by a thread pool."""
    out = np.empty(n, dtype=np.float32)

    def fill(lo: int) -> None:
        m = min(chunk, n - lo)
        bits = splitmix64(seed ^ tensor_index, 2 * m, start=2 * lo)
        u = ((bits >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / (1 << 24))  # (0,1)
        r = np.sqrt(np.float32(-2.0) * np.log(u[0::2]))
        out[lo:lo + m] = r * np.cos(np.float32(2.0 * np.pi) * u[1::2])

    from concurrent.futures import ThreadPoolExecutor
    import os
    with ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 1)) as ex:
        list(ex.map(fill, range(0, n, chunk)))
    return out


def labels(seed: int, tensor_index: int, n: int, classes: int) -> np.ndarray:
    return (splitmix64(seed ^ tensor_index, n) % np.uint64(classes)).astype(np.uint8)


def kaiming_uniform(seed: int, tensor_index: int, n: int, fan_in: int) -> np.ndarray:
    bound = np.float32(np.sqrt(6.0 / fan_in))
    return ((uniform(seed, tensor_index, n) * np.float32(2.0) - np.float32(1.0)) * bound).astype(np.float32)


def kaiming_normal(seed: int, tensor_index: int, n: int, fan_in: int) -> np.ndarray:
    return (normal(seed, tensor_index, n) * np.float32(np.sqrt(2.0 / fan_in))).astype(np.float32)


SEED_BASE = 0x5EED0001
