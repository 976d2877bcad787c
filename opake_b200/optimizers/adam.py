"""DP-aware Adam / AdamW with noise bias correction ("AdamW-BC").

Update rule of packages/opake-optimizers/src/opake/api/optimizers/_adam.py:122-267:
``m = b1 m + (1-b1) g``, ``v = b2 v + (1-b2) g^2``; with ``noise_bias_correction`` the EMA ``phi`` of the noise
variance ``sigma^2`` (from ``NoisedPytree.noise_stddev``; per group when it is a ``PerGroup``) is subtracted from the
bias-corrected second moment where the difference stays positive: ``denom = sqrt(where(v_hat - phi_hat > 0,
v_hat - phi_hat, v_hat)) + eps``. With a private second-moment stream ``v`` tracks the noisy squared gradients and
``v_eff = where(v_hat > 0, v_hat, m_hat^2).clamp(min=eps^2)``. The sharded engine runs the same arithmetic inside
its fused step kernel (csrc/kernels/dp_step.cu).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..base.exceptions import ConfigurationError
from ..engine.pytree import tree_flatten_with_paths, tree_map, tree_unflatten
from ..engine.types import PerGroup
from .chain import GradientTransformation, make_optimizer_chain


@dataclass(frozen=True)
class AdamState:
    mu: Any
    nu: Any
    phi: Any      # dict[ParamPath -> float]: EMA of the noise variance per leaf (None without bias correction)
    step: int


def update_phi_ema(phi, noise_stddev, beta2: float, paths):
    """EMA of the noise variance, one entry per parameter leaf keyed by its path (the layout of
    packages/opake-optimizers/src/opake/api/optimizers/_bias_correction.py:53-152, which serializes as
    ``phi.<path>``); the entries are equal when the noise is isotropic."""
    if isinstance(phi, dict):
        old = phi
    else:
        old = {p: float(phi or 0.0) for p in paths}
    if isinstance(noise_stddev, PerGroup):
        return {p: beta2 * old.get(p, 0.0) + (1 - beta2) * noise_stddev.for_path(p) ** 2 for p in paths}
    s = 0.0 if noise_stddev is None else float(noise_stddev)
    return {p: beta2 * old.get(p, 0.0) + (1 - beta2) * s * s for p in paths}


def scale_by_adam(b1: float, b2: float, eps: float, noise_bias_correction: bool) -> GradientTransformation:
    bc_floor = eps * eps

    def init(params):
        z = (lambda p: torch.zeros_like(p, dtype=torch.float32 if p.dtype in (torch.bfloat16, torch.float16) else p.dtype))
        phi = {p: 0.0 for p in tree_flatten_with_paths(params)[0]} if noise_bias_correction else None
        return AdamState(tree_map(z, params), tree_map(z, params), phi, 0)

    def update(grads, state: AdamState, *, params=None, noise_stddev=None, noisy_squared_grads=None):
        t = state.step + 1
        bc1, bc2 = 1 - b1**t, 1 - b2**t
        paths, g_leaves, td = tree_flatten_with_paths(grads)
        mu = tree_flatten_with_paths(state.mu)[1]
        nu = tree_flatten_with_paths(state.nu)[1]
        sq = tree_flatten_with_paths(noisy_squared_grads)[1] if noisy_squared_grads is not None else None
        phi = state.phi
        if noise_bias_correction and noisy_squared_grads is None:
            phi = update_phi_ema(phi, noise_stddev, b2, paths)
        out, new_mu, new_nu = [], [], []
        for i, (p, g) in enumerate(zip(paths, g_leaves)):
            g32 = g.to(mu[i].dtype)
            m = b1 * mu[i] + (1 - b1) * g32
            second = sq[i].to(m.dtype) if sq is not None else g32 * g32
            v = b2 * nu[i] + (1 - b2) * second
            m_hat, v_hat = m / bc1, v / bc2
            if sq is not None:
                v_eff = torch.where(v_hat > 0, v_hat, m_hat * m_hat).clamp(min=bc_floor)
                den = v_eff.sqrt() + eps
            elif noise_bias_correction:
                ph = (phi[p] if isinstance(phi, dict) else phi) / bc2
                d = v_hat - ph
                den = torch.where(d > 0, d, v_hat).sqrt() + eps
            else:
                den = v_hat.sqrt() + eps
            out.append((m_hat / den).to(g.dtype))
            new_mu.append(m)
            new_nu.append(v)
        return tree_unflatten(td, out), AdamState(tree_unflatten(td, new_mu), tree_unflatten(td, new_nu), phi, t)

    return GradientTransformation(init, update)


def _check(lr, betas, eps, weight_decay):
    b1, b2 = betas
    if not (0 <= b1 < 1 and 0 <= b2 < 1):
        raise ConfigurationError(f"betas must be in [0, 1), got {betas}")
    if eps <= 0:
        raise ConfigurationError(f"eps must be > 0, got {eps}")
    if weight_decay < 0:
        raise ConfigurationError(f"weight_decay must be >= 0, got {weight_decay}")


def adam(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, *, update_rms_clip=None,
         noise_bias_correction=False):
    _check(lr, betas, eps, weight_decay)
    return make_optimizer_chain(scale_by_adam(betas[0], betas[1], eps, noise_bias_correction), lr, weight_decay,
                                optimizer_name="adam", decoupled_weight_decay=False, update_rms_clip=update_rms_clip)


def adamw(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, *, decoupled_weight_decay=True,
          update_rms_clip=None, noise_bias_correction=False):
    _check(lr, betas, eps, weight_decay)
    return make_optimizer_chain(scale_by_adam(betas[0], betas[1], eps, noise_bias_correction), lr, weight_decay,
                                optimizer_name="adamw", decoupled_weight_decay=decoupled_weight_decay,
                                update_rms_clip=update_rms_clip)


__all__ = ["AdamState", "adam", "adamw", "scale_by_adam", "update_phi_ema"]
