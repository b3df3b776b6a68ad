"""Small deterministic inputs shared by the tests."""
import numpy as np


def smooth(n, seed=0):
    rng = np.random.default_rng(seed)
    t = np.arange(n, dtype=np.float64) / max(n, 1)
    x = np.zeros(n)
    for _ in range(3):
        x += np.sin(2 * np.pi * rng.uniform(1, 50) * t + rng.uniform(0, 6.28))
    x += rng.normal(0, 1e-3, n)
    return x.astype(np.float32)


def gradient_like(n, seed=0):
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 0.01, n)
    mask = rng.random(n) < 0.01
    x[mask] *= 10
    return x.astype(np.float32)


def sparse_zero(n, seed=0):
    """Mostly exact zeros with a few isolated spikes: zero blocks, outlier blocks with F = 0."""
    rng = np.random.default_rng(seed)
    x = np.zeros(n, dtype=np.float32)
    idx = rng.integers(0, n, max(1, n // 97))
    x[idx] = rng.normal(0, 1, idx.size).astype(np.float32)
    x[(np.arange(n) % 32 == 0) & (rng.random(n) < 0.3)] = 5.0  # element 0 alone -> outlier mode with F = 0
    return x


def wide(n, seed=0):
    """Large dynamic range: F up to ~24 planes."""
    rng = np.random.default_rng(seed)
    return (rng.normal(0, 1, n) * 10 ** rng.uniform(-3, 3, n)).astype(np.float32)


ALL = {"smooth": smooth, "gradient": gradient_like, "sparse": sparse_zero, "wide": wide}
SIZES = [1, 31, 32, 33, 1000, 8192, 8193, 32768, 32769, 100000, 262144 + 17]
