"""Host-side copy of the runtime's counter-based random numbers, vectorised with NumPy.

Used by callers that prepare a step's inputs in host memory (a data loader feeding token batches):
the numbers are the ones the device kernels draw, so a host-fed run and a device-sampled run see
the same data. Same hash as csrc/anvil_rng.h (reference: anvil/backend/anvil_host.h:17-29).
"""
from __future__ import annotations

import numpy as np

_M32 = np.uint64(0xFFFFFFFF)


def _lowbias32(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint64)
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x7FEB352D)) & _M32
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x846CA68B)) & _M32
    x ^= x >> np.uint64(16)
    return x


def rand_bits(idx, stream: int, salt: int, seed: int) -> np.ndarray:
    k = (stream * 0x85EBCA77 + salt * 0xC2B2AE3D + seed + 0x632BE5AB) & 0xFFFFFFFF
    h = (np.asarray(idx, dtype=np.uint64) * np.uint64(0x9E3779B1) + np.uint64(k)) & _M32
    return _lowbias32(_lowbias32(h)).astype(np.uint32)


def uniform(idx, stream: int, salt: int, seed: int, open_low: bool = False) -> np.ndarray:
    hi = (rand_bits(idx, stream, salt, seed) >> np.uint32(8)).astype(np.float32)
    if open_low:
        hi = hi + np.float32(1.0)
    return hi * np.float32(1.0 / 16777216.0)


def randint(shape, lo: int, hi: int, stream: int, seed: int, base: int = 0) -> np.ndarray:
    """`x: i32[shape] ~ randint(lo, hi)`: lo + floor((hi - lo) * u) in f32, truncated; element i of
    the row-major tensor uses index base + i."""
    n = int(np.prod(shape))
    u = uniform(np.arange(base, base + n, dtype=np.uint64), stream, 0, seed)
    v = np.floor(np.float32(hi - lo) * u)
    if lo:
        v = v + np.float32(lo)
    return v.astype(np.int32).reshape(shape)
