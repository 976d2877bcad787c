"""Correlated-noise strategies for DP-FTRL (matrix-factorisation mechanisms).

Each strategy describes a lower-triangular strategy matrix ``C``; at run time the mechanism adds
``sigma * (C^{-1} z)_t`` at step ``t`` (``z_t`` iid Gaussian), produced by a *streaming* multiply with ``C^{-1}`` that
keeps only a small state. Privacy is accounted as a Gaussian mechanism with noise multiplier ``nm / sens(C)``.

Catalogue and constructor arguments follow packages/opake-dpftrl/src/opake/api/dpftrl/noise/: ``_blt.py:65-203``
(buffered linear Toeplitz, state ``[nbuf, *shape]``), ``_band_mf.py:36-190`` (banded Toeplitz, ring of ``bands-1``
outputs), ``_bsr.py:147-200`` (closed-form banded square root), ``_bisr.py:324-763`` (banded inverse square root: FIR
over the last draws), ``_lambda_cgd.py:192-327`` (``z_t - lambda z_{t-1}``), ``_identity.py`` and
``_streaming_matrix.py:32-309``.
"""
from __future__ import annotations

import math
from collections.abc import Callable
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from ..base.exceptions import ConfigurationError
from ..engine.pytree import tree_map
from . import toeplitz as T


# ------------------------------------------------------------------------------------------------ streaming matrices
@dataclass(frozen=True)
class StreamingMatrix:
    """``y_t = (M x)_t`` computed one row at a time. ``init_multiply(template) -> state``;
    ``multiply_next(x_t, state) -> (y_t, state)`` on pytrees; ``row_norms_squared_fn(n) -> tensor[n]``."""

    init_multiply: Callable[[Any], Any]
    multiply_next: Callable[[Any, Any], tuple[Any, Any]]
    row_norms_squared_fn: Callable[[int], torch.Tensor]

    def row_norms_squared(self, n: int) -> torch.Tensor:
        return self.row_norms_squared_fn(n)

    def __matmul__(self, other: "StreamingMatrix") -> "StreamingMatrix":
        """Product ``self @ other`` (apply ``other`` first). Row norms of a product are not tracked."""
        def init(t):
            return (self.init_multiply(t), other.init_multiply(t))

        def nxt(x, st):
            y, s1 = other.multiply_next(x, st[1])
            z, s0 = self.multiply_next(y, st[0])
            return z, (s0, s1)

        def norms(n):
            raise ConfigurationError("row norms of a streaming product are not available in closed form")

        return StreamingMatrix(init, nxt, norms)


def _zeros_like_stack(template, k: int):
    return tree_map(lambda t: torch.zeros((k, *t.shape), dtype=torch.float32, device=t.device), template)


def identity_matrix() -> StreamingMatrix:
    return StreamingMatrix(lambda t: (), lambda x, s: (x, s), lambda n: torch.ones(n, dtype=torch.float64))


def prefix_sum_matrix() -> StreamingMatrix:
    def nxt(x, s):
        s2 = tree_map(lambda a, b: a + b.to(a.dtype), s, x)
        return s2, s2

    return StreamingMatrix(lambda t: tree_map(lambda a: torch.zeros_like(a, dtype=torch.float32), t), nxt,
                           lambda n: torch.arange(1, n + 1, dtype=torch.float64))


def diagonal_matrix(diag: Callable[[int], float]) -> StreamingMatrix:
    def nxt(x, s):
        return tree_map(lambda a: a * diag(s), x), s + 1

    return StreamingMatrix(lambda t: 0, nxt, lambda n: torch.tensor([diag(i) ** 2 for i in range(n)], dtype=torch.float64))


def momentum_sgd_matrix(momentum: float) -> StreamingMatrix:
    def nxt(x, s):
        s2 = tree_map(lambda m, b: momentum * m + b.to(m.dtype), s, x)
        return s2, s2

    return StreamingMatrix(lambda t: tree_map(lambda a: torch.zeros_like(a, dtype=torch.float32), t), nxt,
                           lambda n: torch.tensor([(1 - momentum ** (2 * (i + 1))) / (1 - momentum**2) for i in range(n)],
                                                  dtype=torch.float64))


def toeplitz_inverse_matrix(c: np.ndarray) -> StreamingMatrix:
    """Streaming multiply by the inverse of the banded Toeplitz matrix with first column ``c``:
    ``y_t = (x_t - sum_{k>=1} c_k y_{t-k}) / c_0`` with a ring of the last ``len(c)-1`` outputs."""
    c = np.asarray(c, dtype=np.float64)
    p = len(c)

    def init(t):
        return (_zeros_like_stack(t, max(p - 1, 1)), 0)

    def nxt(x, st):
        ring, step = st
        if p == 1:
            return tree_map(lambda a: a / c[0], x), (ring, step + 1)
        coef = torch.tensor(c[1:], dtype=torch.float32)

        def one(a, r):
            y = (a.to(torch.float32) - torch.tensordot(coef.to(r.device), r, dims=1)) / c[0]
            r2 = torch.roll(r, 1, 0)
            r2[0] = y
            return y.to(a.dtype), r2

        ys, rs = {}, {}
        from ..engine.pytree import tree_flatten, tree_unflatten

        xl, td = tree_flatten(x)
        rl, _ = tree_flatten(ring)
        pairs = [one(a, r) for a, r in zip(xl, rl)]
        return tree_unflatten(td, [q[0] for q in pairs]), (tree_unflatten(td, [q[1] for q in pairs]), step + 1)

    def norms(n):
        inv = T.inverse_coefficients(c, n)
        return torch.from_numpy(np.cumsum(inv * inv))

    return StreamingMatrix(init, nxt, norms)


def fir_matrix(taps: np.ndarray) -> StreamingMatrix:
    """``y_t = sum_k taps_k x_{t-k}`` with a ring of the last ``len(taps)-1`` inputs."""
    taps = np.asarray(taps, dtype=np.float64)
    p = len(taps)

    def init(t):
        return _zeros_like_stack(t, max(p - 1, 1))

    def nxt(x, ring):
        if p == 1:
            return tree_map(lambda a: a * taps[0], x), ring
        coef = torch.tensor(taps[1:], dtype=torch.float32)

        def one(a, r):
            y = taps[0] * a.to(torch.float32) + torch.tensordot(coef.to(r.device), r, dims=1)
            r2 = torch.roll(r, 1, 0)
            r2[0] = a.to(torch.float32)
            return y.to(a.dtype), r2

        from ..engine.pytree import tree_flatten, tree_unflatten

        xl, td = tree_flatten(x)
        rl, _ = tree_flatten(ring)
        pairs = [one(a, r) for a, r in zip(xl, rl)]
        return tree_unflatten(td, [q[0] for q in pairs]), tree_unflatten(td, [q[1] for q in pairs])

    def norms(n):
        sq = np.cumsum(np.pad(taps * taps, (0, max(0, n - p)))[:n])
        return torch.from_numpy(sq)

    return StreamingMatrix(init, nxt, norms)


def blt_inverse_matrix(decay: np.ndarray, scale: np.ndarray) -> StreamingMatrix:
    """``xhat = x - <scale, state>``; ``state_k = decay_k state_k + xhat`` (state ``[nbuf, *shape]`` fp32)."""
    decay, scale = np.asarray(decay, float), np.asarray(scale, float)
    nb = len(decay)

    def init(t):
        return _zeros_like_stack(t, nb)

    def nxt(x, st):
        d = torch.tensor(decay, dtype=torch.float32)
        s = torch.tensor(scale, dtype=torch.float32)

        def one(a, b):
            xh = a.to(torch.float32) - torch.tensordot(s.to(b.device), b, dims=1)
            b2 = b * d.to(b.device).view(-1, *([1] * a.dim())) + xh.unsqueeze(0)
            return xh.to(a.dtype), b2

        from ..engine.pytree import tree_flatten, tree_unflatten

        xl, td = tree_flatten(x)
        bl, _ = tree_flatten(st)
        pairs = [one(a, b) for a, b in zip(xl, bl)]
        return tree_unflatten(td, [q[0] for q in pairs]), tree_unflatten(td, [q[1] for q in pairs])

    def norms(n):
        inv = T.inverse_coefficients(T.blt_coefficients(decay, scale, n), n)
        return torch.from_numpy(np.cumsum(inv * inv))

    return StreamingMatrix(init, nxt, norms)


# ------------------------------------------------------------------------------------------------ strategies
class MfStrategy:
    """Base of strategy descriptions. Subclasses provide the coefficients of ``C`` and the streaming ``C^{-1}``."""

    name = "strategy"

    def strategy_coefficients(self, n_steps: int) -> np.ndarray:
        raise NotImplementedError

    def streaming_matrix(self, *, n_steps: int, min_sep: int = 1, max_participations: int | None = None) -> StreamingMatrix:
        raise NotImplementedError

    def sensitivity_squared(self, *, n_steps: int, min_sep: int = 1, max_participations: int | None = None) -> float:
        return T.column_sum_sq(self.strategy_coefficients(n_steps), n_steps, min_sep, max_participations)

    def sensitivity(self, **kw) -> float:
        return math.sqrt(self.sensitivity_squared(**kw))

    def gram_matrix(self, *, n_steps: int, num_bins: int, num_epochs: int | None = None, normalized: bool = False):
        from ..accounting._native import native

        c = [float(x) for x in self.strategy_coefficients(n_steps)]
        g = native().toeplitz_gram_matrix(c, int(n_steps), int(num_bins), num_epochs, bool(normalized))
        return np.asarray(g).reshape(num_bins, num_bins)

    def config(self) -> dict:
        return {}


@dataclass(frozen=True)
class IdentityStrategy(MfStrategy):
    name = "identity"

    def strategy_coefficients(self, n_steps):
        return np.array([1.0])

    def streaming_matrix(self, **kw):
        return identity_matrix()

    def config(self):
        return {}


@dataclass(frozen=True)
class BsrStrategy(MfStrategy):
    bandwidth: int
    alpha: float = 1.0
    beta: float = 0.0
    name = "bsr"

    def __post_init__(self):
        if self.bandwidth < 1:
            raise ConfigurationError(f"bandwidth must be >= 1, got {self.bandwidth}")
        if not (0 < self.alpha <= 1 and 0 <= self.beta < 1):
            raise ConfigurationError("need alpha in (0, 1] and beta in [0, 1)")

    def strategy_coefficients(self, n_steps):
        return T.bsr_coefficients(min(self.bandwidth, n_steps), self.alpha, self.beta)

    def streaming_matrix(self, *, n_steps, min_sep=1, max_participations=None):
        return toeplitz_inverse_matrix(self.strategy_coefficients(n_steps))

    def config(self):
        return {"bandwidth": self.bandwidth, "alpha": self.alpha, "beta": self.beta}


@dataclass(frozen=True)
class BandMfStrategy(MfStrategy):
    bands: int
    momentum: float = 1.0
    lr_schedule: Any = None
    coefficients: tuple | None = None     # filled by optimize(); None -> optimized lazily per horizon
    name = "band_mf"

    def __post_init__(self):
        if self.bands < 1:
            raise ConfigurationError(f"bands must be >= 1, got {self.bands}")

    def optimize(self, n_steps: int) -> "BandMfStrategy":
        """Minimise ``sum(c^2) * ||A C^{-1}||_F^2`` over the banded coefficients (L-BFGS from the square-root init)."""
        from dataclasses import replace

        b = min(self.bands, n_steps)
        c0 = T.bsr_coefficients(b)
        if b == 1:
            return replace(self, coefficients=(1.0,))
        # the optimised column is rescaled to unit L2 norm (single-participation sensitivity 1), the normalisation of
        # packages/opake-dpftrl/src/opake/api/dpftrl/noise/_band_mf.py:101-187: streaming states are then interchangeable
        wl = T.workload_coefficients(n_steps, 0.0 if self.momentum in (0.0, 1.0) else self.momentum)
        n_eval = min(n_steps, 4096)

        def loss(free):
            c = np.concatenate([[1.0], free])
            return math.log(np.dot(c, c)) + math.log(T.error_squared(c, n_eval, wl[:n_eval]))

        try:
            from scipy.optimize import minimize

            res = minimize(loss, c0[1:], method="L-BFGS-B", options={"maxiter": 40})
            c = np.concatenate([[1.0], res.x]) if res.fun < loss(c0[1:]) else c0
        except Exception:
            c = c0
        c = np.asarray(c, dtype=np.float64)
        c = c / math.sqrt(float(np.dot(c, c)))
        return replace(self, coefficients=tuple(float(x) for x in c))

    def strategy_coefficients(self, n_steps):
        if self.coefficients is None:
            return np.asarray(self.optimize(n_steps).coefficients)
        return np.asarray(self.coefficients)

    def streaming_matrix(self, *, n_steps, min_sep=1, max_participations=None):
        return toeplitz_inverse_matrix(self.strategy_coefficients(n_steps))

    def sensitivity_squared(self, *, n_steps, min_sep=1, max_participations=None):
        c = self.strategy_coefficients(n_steps)
        if min_sep >= len(c):       # participations never overlap inside a band: columns are orthogonal
            from ..accounting._native import native

            k = native().minsep_true_max_participations(int(n_steps), int(min_sep), max_participations)
            return float(k * np.dot(c, c))
        return T.column_sum_sq(c, n_steps, min_sep, max_participations)

    def config(self):
        return {"bands": self.bands, "momentum": self.momentum,
                "coefficients": list(self.coefficients) if self.coefficients else None}


@dataclass(frozen=True)
class BltStrategy(MfStrategy):
    max_buffers: int = 10
    momentum: float = 1.0
    lr_schedule: Any = None
    buf_decay: tuple | None = None
    output_scale: tuple | None = None
    name = "blt"

    def __post_init__(self):
        if not 1 <= self.max_buffers <= 15:
            raise ConfigurationError(f"max_buffers must be in [1, 15], got {self.max_buffers}")

    def optimize(self, n_steps: int, min_sep: int = 1, max_participations: int | None = None) -> "BltStrategy":
        """Fit decays / scales by minimising ``sens^2 * error`` over log-parametrised buffers, growing the number of
        buffers while it pays (at most ``max_buffers``)."""
        from dataclasses import replace

        n_eval = min(n_steps, 2048)
        wl = T.workload_coefficients(n_eval, 0.0 if self.momentum in (0.0, 1.0) else self.momentum)

        def unpack(v):
            k = len(v) // 2
            decay = 1.0 / (1.0 + np.exp(-v[:k]))          # (0, 1)
            scale = np.exp(v[k:])                          # > 0
            return decay, scale

        def loss(v):
            with np.errstate(all="ignore"):
                decay, scale = unpack(np.clip(v, -30.0, 30.0))
                c = T.blt_coefficients(decay, scale, n_eval)
                s2 = T.column_sum_sq(c, n_eval, min(min_sep, n_eval), max_participations) if min_sep > 1 else float(np.dot(c, c))
                val = math.log(s2) + math.log(T.error_squared(c, n_eval, wl)) if s2 > 0 else math.inf
            return val if math.isfinite(val) else 1e30

        best, best_loss = None, math.inf
        try:
            from scipy.optimize import minimize
        except Exception:
            minimize = None
        for k in range(1, self.max_buffers + 1):
            # spread initial decays geometrically towards 1; scales chosen so that c_1 ~ 1/2 as for the square root
            d0 = 1.0 - 0.5 ** np.arange(1, k + 1) * 0.9
            v0 = np.concatenate([np.log(d0 / (1 - d0)), np.log(np.full(k, 0.5 / k))])
            if minimize is not None:
                res = minimize(loss, v0, method="L-BFGS-B", options={"maxiter": 60})
                v, val = res.x, float(res.fun)
            else:
                v, val = v0, loss(v0)
            if val < best_loss - 1e-3:
                best, best_loss = v, val
            else:
                break
            if k >= 4 and n_steps <= 4096:
                break
        decay, scale = unpack(np.clip(best, -30.0, 30.0))
        return replace(self, buf_decay=tuple(map(float, decay)), output_scale=tuple(map(float, scale)))

    def _params(self, n_steps, min_sep=1, max_participations=None):
        s = self if self.buf_decay is not None else self.optimize(n_steps, min_sep, max_participations)
        return np.asarray(s.buf_decay), np.asarray(s.output_scale)

    def strategy_coefficients(self, n_steps):
        d, s = self._params(n_steps)
        return T.blt_coefficients(d, s, n_steps)

    def streaming_matrix(self, *, n_steps, min_sep=1, max_participations=None):
        d, s = self._params(n_steps, min_sep, max_participations)
        return blt_inverse_matrix(d, s)

    def sensitivity_squared(self, *, n_steps, min_sep=1, max_participations=None):
        d, s = self._params(n_steps, min_sep, max_participations)
        if min_sep <= 1 and (max_participations in (None, 1)) and max_participations == 1:
            from ..accounting._native import native

            return float(native().blt_sensitivity_squared(list(map(float, d)), list(map(float, s)), float(n_steps)))
        return T.column_sum_sq(T.blt_coefficients(d, s, n_steps), n_steps, min_sep, max_participations)

    def config(self):
        return {"max_buffers": self.max_buffers, "momentum": self.momentum,
                "buf_decay": list(self.buf_decay) if self.buf_decay else None,
                "output_scale": list(self.output_scale) if self.output_scale else None}


@dataclass(frozen=True)
class BisrStrategy(MfStrategy):
    bandwidth: int
    normalized: bool = True
    momentum: float = 0.0
    lr_schedule: Any = None
    inv_coefficients: tuple | None = None
    name = "bisr"

    def __post_init__(self):
        if self.bandwidth < 1:
            raise ConfigurationError(f"bandwidth must be >= 1, got {self.bandwidth}")

    def inverse_taps(self) -> np.ndarray:
        if self.inv_coefficients is not None:
            return np.asarray(self.inv_coefficients, float)
        return T.inv_sqrt_series(self.bandwidth)

    def strategy_coefficients(self, n_steps):
        from ..accounting._native import native

        return np.asarray(native().bisr_strategy_coefficients([float(x) for x in self.inverse_taps()], int(n_steps)))

    def streaming_matrix(self, *, n_steps, min_sep=1, max_participations=None):
        taps = self.inverse_taps()[: max(1, min(self.bandwidth, n_steps))]
        return fir_matrix(taps)

    def config(self):
        return {"bandwidth": self.bandwidth, "normalized": self.normalized, "momentum": self.momentum,
                "inv_coefficients": list(self.inv_coefficients) if self.inv_coefficients else None}


@dataclass(frozen=True)
class LambdaCgdStrategy(MfStrategy):
    lambda_: float
    normalized: bool = True
    lr_schedule: Any = None
    name = "lambda_cgd"

    def __post_init__(self):
        if not 0 <= self.lambda_ < 1:
            raise ConfigurationError(f"lambda_ must be in [0, 1), got {self.lambda_}")

    def strategy_coefficients(self, n_steps):
        return self.lambda_ ** np.arange(n_steps, dtype=np.float64)

    def column_norm(self, col: int, n_steps: int) -> float:
        lam = self.lambda_
        return 1.0 if lam == 0 else math.sqrt((1 - lam ** (2 * (n_steps - col))) / (1 - lam * lam))

    def streaming_matrix(self, *, n_steps, min_sep=1, max_participations=None):
        lam = self.lambda_
        base = fir_matrix(np.array([1.0, -lam]) if lam else np.array([1.0]))
        if not self.normalized:
            return base
        # column-normalised C~ = C D^{-1}  =>  C~^{-1} = D C^{-1}: scale output row t by the norm of column t
        def nxt(x, st):
            ring, t = st
            y, ring = base.multiply_next(x, ring)
            d = self.column_norm(t, n_steps)
            return tree_map(lambda a: a * d, y), (ring, t + 1)

        def norms(n):
            r = base.row_norms_squared(n)
            return r * torch.tensor([self.column_norm(t, n_steps) ** 2 for t in range(n)], dtype=r.dtype)

        return StreamingMatrix(lambda t: (base.init_multiply(t), 0), nxt, norms)

    def sensitivity_squared(self, *, n_steps, min_sep=1, max_participations=None):
        from ..accounting._native import native

        fn = native().lambda_cgd_normalized_sensitivity_squared if self.normalized else native().lambda_cgd_sensitivity_squared
        return float(fn(float(self.lambda_), int(n_steps), int(min_sep), max_participations))

    def config(self):
        return {"lambda_": self.lambda_, "normalized": self.normalized}


def identity_strategy() -> IdentityStrategy:
    return IdentityStrategy()


def blt_strategy(*, max_buffers: int = 10, momentum: float = 1.0, lr_schedule=None) -> BltStrategy:
    return BltStrategy(max_buffers, momentum, lr_schedule)


def band_mf_strategy(*, bands: int, momentum: float = 1.0, lr_schedule=None) -> BandMfStrategy:
    return BandMfStrategy(bands, momentum, lr_schedule)


def bsr_strategy(*, bandwidth: int, alpha: float, beta: float) -> BsrStrategy:
    return BsrStrategy(bandwidth, alpha, beta)


def bisr_strategy(*, bandwidth: int, normalized: bool = True, momentum: float = 0.0, lr_schedule=None,
                  inv_coefficients=None) -> BisrStrategy:
    return BisrStrategy(bandwidth, normalized, momentum, lr_schedule,
                        tuple(inv_coefficients) if inv_coefficients is not None else None)


def lambda_cgd_strategy(*, lambda_: float, normalized: bool = True, lr_schedule=None) -> LambdaCgdStrategy:
    return LambdaCgdStrategy(lambda_, normalized, lr_schedule)


# ------------------------------------------------------------------------------------------------ strategy codec
_STRATEGIES: dict[str, type] = {}


def register_strategy(cls: type) -> type:
    _STRATEGIES[cls.name] = cls
    return cls


for _c in (IdentityStrategy, BsrStrategy, BandMfStrategy, BltStrategy, BisrStrategy, LambdaCgdStrategy):
    register_strategy(_c)


def serialize_strategy(s: MfStrategy) -> dict:
    return {"kind": s.name, **{k: v for k, v in s.config().items()}}


def deserialize_strategy(d: dict) -> MfStrategy:
    d = dict(d)
    kind = d.pop("kind")
    cls = _STRATEGIES.get(kind)
    if cls is None:
        raise ConfigurationError(f"unknown strategy kind {kind!r}")
    kw = {k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items()}
    return cls(**kw)


__all__ = ["StreamingMatrix", "MfStrategy", "IdentityStrategy", "BsrStrategy", "BandMfStrategy", "BltStrategy",
           "BisrStrategy", "LambdaCgdStrategy", "identity_strategy", "blt_strategy", "band_mf_strategy", "bsr_strategy",
           "bisr_strategy", "lambda_cgd_strategy", "register_strategy", "serialize_strategy", "deserialize_strategy",
           "identity_matrix", "prefix_sum_matrix", "diagonal_matrix", "momentum_sgd_matrix"]
