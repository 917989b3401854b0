"""Seeded synthetic inputs shared by the tests (numpy, CPU)."""
from __future__ import annotations

import numpy as np


def gaussian_mixture(N: int, D: int, n_comp: int, seed: int, mean_scale: float = 4.0,
                     sigma: float = 1.0) -> np.ndarray:
    """Isotropic Gaussian mixture with component means ~ N(0, mean_scale^2 I), equal weights."""
    rng = np.random.default_rng(seed)
    means = (mean_scale * rng.standard_normal((n_comp, D))).astype(np.float32)
    comp = rng.integers(0, n_comp, size=N)
    X = means[comp] + sigma * rng.standard_normal((N, D)).astype(np.float32)
    return np.ascontiguousarray(X, dtype=np.float32)


def clustered_jitter(N: int, D: int, seed: int = 42, n_clusters: int = 16) -> np.ndarray:
    """Clustered cloud with small continuous jitter: the data shape of the reference's own
    parity script (tests/test_fps_sharded.py:18-25): N(0, I) centres + 0.05 * noise."""
    rng = np.random.default_rng(seed)
    centres = rng.standard_normal((n_clusters, D)).astype(np.float32)
    ids = rng.integers(0, n_clusters, size=N)
    X = centres[ids] + 0.05 * rng.standard_normal((N, D)).astype(np.float32)
    return np.ascontiguousarray(X, dtype=np.float32)


def with_duplicates(X: np.ndarray, n_dup: int, seed: int) -> np.ndarray:
    """Copy ``n_dup`` random rows over other random rows: exact ties for the arg-max."""
    rng = np.random.default_rng(seed)
    X = X.copy()
    src = rng.integers(0, X.shape[0], size=n_dup)
    dst = rng.integers(0, X.shape[0], size=n_dup)
    X[dst] = X[src]
    return X


def as_dtype(X: np.ndarray, dtype: str) -> np.ndarray:
    """The float32 matrix as a float16 / float64 input.  float64 values get low-order bits that
    do not survive the conversion back to float32, so that rounding is exercised."""
    if dtype == "float32":
        return X
    if dtype == "float16":
        return X.astype(np.float16)
    if dtype == "float64":
        return X.astype(np.float64) * 1.000000123
    raise ValueError(dtype)
