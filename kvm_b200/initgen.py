"""Counter-based initial values of `seeded` buffers, vectorised (host side of the device generator in csrc/kvm_exec.cu).

Spec (reference `runtime/initgen.py:1-58`): draw j of seed s is SplitMix64 at counter j, u = (z >> 40) * 2^-24; element i
uses draws j = i*draws..; acc = u (uniform) or (u0+u1)+(u2+u3) (normal, Irwin-Hall of 4); value = (acc - bias) * coef, every
step one rounded float32 operation.  Bit-exact with the reference by construction (integer hash + float32 numpy ops).
"""
import math

import numpy as np

GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def seeded_params(dist: str, scale: float):
    """(draws, bias, coef) written into bundle metadata (`runtime/initgen.py:28-34`)."""
    if dist == 'uniform':
        return 1, 0.5, float(np.float32(2.0 * scale))
    if dist == 'normal':
        return 4, 2.0, float(np.float32(scale * math.sqrt(3.0)))
    raise ValueError(f"unknown dist {dist!r}; expected 'uniform' or 'normal'")


def splitmix64(seed: int, j: np.ndarray) -> np.ndarray:
    with np.errstate(over='ignore'):
        z = np.uint64(seed & (2**64 - 1)) + (j.astype(np.uint64) + np.uint64(1)) * GOLDEN
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _seeded_range(seed: int, lo: int, hi: int, draws: int, bias: float, coef: float) -> np.ndarray:
    i = np.arange(lo, hi, dtype=np.uint64)
    u = lambda j: (splitmix64(seed, j) >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    if draws == 1:
        acc = u(i)
    else:
        j = i * np.uint64(draws)
        acc = (u(j) + u(j + np.uint64(1))) + (u(j + np.uint64(2)) + u(j + np.uint64(3)))
    return ((acc - np.float32(bias)) * np.float32(coef)).astype(np.float32)


def seeded_values(seed: int, n: int, draws: int, bias: float, coef: float) -> np.ndarray:
    """Elements 0..n-1 of the seeded buffer.  Every element depends on its own index only, so large buffers are generated in
    cache-sized pieces on all host threads (numpy releases the interpreter lock inside its loops)."""
    chunk = 1 << 18
    if n <= 2 * chunk:
        return _seeded_range(seed, 0, n, draws, bias, coef)
    import os
    from concurrent.futures import ThreadPoolExecutor
    out = np.empty(n, np.float32)

    def fill(lo):
        hi = min(lo + chunk, n)
        out[lo:hi] = _seeded_range(seed, lo, hi, draws, bias, coef)
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 1) as pool:
        list(pool.map(fill, range(0, n, chunk)))
    return out
