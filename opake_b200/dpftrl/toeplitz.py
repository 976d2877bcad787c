"""Lower-triangular Toeplitz arithmetic used by the correlated-noise (matrix-factorisation) strategies.

A strategy matrix ``C`` (n x n, lower triangular Toeplitz) is represented by its first column ``c``. The mechanism
releases ``A(x + C^{-1} z)`` for the prefix-sum style workload ``A``; its error is governed by
``sens(C)^2 * ||A C^{-1}||_F^2``. This module provides coefficient inversion, workloads, the error functional and the
closed-form banded square-root coefficients (math of packages/opake-dpftrl/src/opake/api/dpftrl/noise/_toeplitz.py,
_bsr.py:47-71 and _blt_math.py:155-294, restated with NumPy).
"""
from __future__ import annotations

import numpy as np


def inverse_coefficients(c: np.ndarray, n: int) -> np.ndarray:
    """First ``n`` coefficients of the inverse of the lower-triangular Toeplitz matrix with first column ``c``."""
    c = np.asarray(c, dtype=np.float64)
    inv = np.zeros(n)
    inv[0] = 1.0 / c[0]
    p = len(c)
    for m in range(1, n):
        k = min(m, p - 1)
        inv[m] = -np.dot(c[1 : k + 1], inv[m - 1 :: -1][:k]) / c[0]
    return inv


def sqrt_series(n: int) -> np.ndarray:
    """r_k = binom(2k, k) / 4^k: coefficients of (1 - x)^(-1/2)."""
    r = np.ones(n)
    for k in range(1, n):
        r[k] = r[k - 1] * (2 * k - 1) / (2 * k)
    return r


def inv_sqrt_series(n: int) -> np.ndarray:
    """Coefficients of (1 - x)^(1/2): 1, -1/2, -1/8, ..."""
    r = np.ones(n)
    for k in range(1, n):
        r[k] = r[k - 1] * (2 * k - 3) / (2 * k)
    return r


def bsr_coefficients(bandwidth: int, alpha: float = 1.0, beta: float = 0.0) -> np.ndarray:
    """Banded square root of the momentum / weight-decay workload with generating function
    1 / ((1 - alpha x)(1 - beta x)): c_k = sum_j alpha^j r_j * beta^(k-j) r_(k-j), truncated to ``bandwidth`` terms."""
    r = sqrt_series(bandwidth)
    a = r * alpha ** np.arange(bandwidth)
    if beta == 0.0:
        return a
    b = r * beta ** np.arange(bandwidth)
    return np.convolve(a, b)[:bandwidth]


def workload_coefficients(n: int, momentum: float = 0.0, weight_decay_alpha: float = 1.0) -> np.ndarray:
    """First column of the workload ``A`` (prefix sums; with momentum beta: sum_j alpha^j beta^(k-j))."""
    a = weight_decay_alpha ** np.arange(n, dtype=np.float64)
    if momentum:
        a = np.convolve(a, momentum ** np.arange(n, dtype=np.float64))[:n]
    return a


def error_squared(c: np.ndarray, n: int, workload: np.ndarray | None = None) -> float:
    """||A C^{-1}||_F^2 for Toeplitz ``C`` (first column ``c``) and Toeplitz workload ``A``."""
    inv = inverse_coefficients(c, n)
    a = workload if workload is not None else np.ones(n)
    b = np.convolve(a[:n], inv)[:n]
    return float(np.dot(b * b, np.arange(n, 0, -1)))


def column_sum_sq(c: np.ndarray, n: int, min_sep: int, k: int | None) -> float:
    """Squared norm of the sum of columns 0, b, 2b, ... (worst participation pattern for non-negative,
    non-increasing coefficients)."""
    from ..accounting._native import native

    return float(native().toeplitz_minsep_sensitivity_squared([float(x) for x in np.abs(c)], int(n), int(min_sep), k))


def blt_coefficients(decay: np.ndarray, scale: np.ndarray, n: int) -> np.ndarray:
    """c_0 = 1, c_i = sum_j scale_j * decay_j^(i-1)."""
    c = np.ones(n)
    if n > 1:
        pw = np.power.outer(np.asarray(decay, float), np.arange(n - 1))
        c[1:] = np.asarray(scale, float) @ pw
    return c


def blt_inverse_params(decay: np.ndarray, scale: np.ndarray):
    """Buffer parameters of ``C^{-1}``, itself a buffered linear Toeplitz operator with coefficients
    c~_0 = 1, c~_i = -sum_j scale~_j decay~_j^(i-1): the decays are the eigenvalues of diag(decay) - 1 scale^T."""
    d, s = np.asarray(decay, float), np.asarray(scale, float)
    M = np.diag(d) - np.outer(np.ones_like(d), s)
    ev, V = np.linalg.eig(M)
    w = np.linalg.solve(V, np.ones_like(d))
    out_scale = (s @ V) * w
    return np.real_if_close(ev), np.real_if_close(out_scale)
