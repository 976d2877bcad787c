"""The remaining optimizers, each as ``moment scaler + make_optimizer_chain``: SGD (momentum / Nesterov), Adagrad,
Adadelta, RMSprop, Lion, RAdam, AdEMAMix, Adafactor and schedule-free SGD/AdamW.

Same catalogue and argument names as packages/opake-optimizers/src/opake/api/optimizers/_sgd.py:41-84, _adagrad.py,
_adadelta.py, _rmsprop.py, _lion.py, _radam.py, _ademamix.py, _adafactor.py, _schedule_free.py. Optimizers with a
second-moment accumulator accept ``noisy_squared_grads`` (a private second-moment stream); the others reject it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch

from ..base.exceptions import ConfigurationError
from ..engine.pytree import tree_map
from .chain import GradientTransformation, make_optimizer_chain, resolve_lr


def _f32(p):
    return torch.zeros_like(p, dtype=torch.float32 if p.dtype in (torch.bfloat16, torch.float16) else p.dtype)


def _zeros(params):
    return tree_map(_f32, params)


# ------------------------------------------------------------------------------------------------ SGD
@dataclass(frozen=True)
class MomentumState:
    trace: Any
    step: int = 0


def sgd(lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, *, moment_requires_grad=False,
        maximize=False):
    if momentum < 0 or weight_decay < 0:
        raise ConfigurationError("momentum and weight_decay must be >= 0")
    if nesterov and (momentum <= 0 or dampening != 0):
        raise ConfigurationError("Nesterov momentum requires a momentum and zero dampening")

    def init(params):
        return MomentumState(_zeros(params) if momentum else None, 0)

    def update(g, st: MomentumState, *, params=None):
        if maximize:
            g = tree_map(lambda x: -x, g)
        if not momentum:
            return g, MomentumState(None, st.step + 1)
        if st.step == 0:
            tr = tree_map(lambda x: x.to(torch.float32).clone() if x.dtype in (torch.bfloat16, torch.float16) else x.clone(), g)
        else:
            tr = tree_map(lambda b, x: momentum * b + (1 - dampening) * x.to(b.dtype), st.trace, g)
        d = tree_map(lambda x, b: (x.to(b.dtype) + momentum * b).to(x.dtype), g, tr) if nesterov else \
            tree_map(lambda x, b: b.to(x.dtype), g, tr)
        return d, MomentumState(tr, st.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="sgd",
                                decoupled_weight_decay=False)


# ------------------------------------------------------------------------------------------------ Adagrad / RMSprop / Adadelta
@dataclass(frozen=True)
class AccumState:
    acc: Any
    aux: Any = None
    step: int = 0


def adagrad(lr=1e-2, lr_decay=0.0, weight_decay=0.0, initial_accumulator_value=0.0, eps=1e-10):
    def init(params):
        return AccumState(tree_map(lambda p: _f32(p) + initial_accumulator_value, params))

    def update(g, st, *, params=None, noisy_squared_grads=None):
        sq = noisy_squared_grads if noisy_squared_grads is not None else tree_map(lambda x: x.float() ** 2, g)
        acc = tree_map(lambda a, s: a + s.to(a.dtype), st.acc, sq)
        clr = 1.0 / (1.0 + st.step * lr_decay)
        d = tree_map(lambda x, a: (clr * x.to(a.dtype) / (a.clamp(min=0).sqrt() + eps)).to(x.dtype), g, acc)
        return d, AccumState(acc, None, st.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="adagrad",
                                decoupled_weight_decay=False)


def rmsprop(lr=1e-2, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0, centered=False):
    def init(params):
        return AccumState(_zeros(params), (_zeros(params) if centered else None, _zeros(params) if momentum else None))

    def update(g, st, *, params=None, noisy_squared_grads=None):
        sq = noisy_squared_grads if noisy_squared_grads is not None else tree_map(lambda x: x.float() ** 2, g)
        acc = tree_map(lambda a, s: alpha * a + (1 - alpha) * s.to(a.dtype), st.acc, sq)
        avg, buf = st.aux
        if centered:
            avg = tree_map(lambda m, x: alpha * m + (1 - alpha) * x.to(m.dtype), avg, g)
            den = tree_map(lambda a, m: (a - m * m).clamp(min=0).sqrt() + eps, acc, avg)
        else:
            den = tree_map(lambda a: a.clamp(min=0).sqrt() + eps, acc)
        d = tree_map(lambda x, dn: x.to(dn.dtype) / dn, g, den)
        if momentum:
            buf = tree_map(lambda b, x: momentum * b + x, buf, d)
            d = buf
        d = tree_map(lambda x, y: y.to(x.dtype), g, d)
        return d, AccumState(acc, (avg, buf), st.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="rmsprop",
                                decoupled_weight_decay=False)


def adadelta(lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0):
    def init(params):
        return AccumState(_zeros(params), _zeros(params))

    def update(g, st, *, params=None, noisy_squared_grads=None):
        sq = noisy_squared_grads if noisy_squared_grads is not None else tree_map(lambda x: x.float() ** 2, g)
        acc = tree_map(lambda a, s: rho * a + (1 - rho) * s.to(a.dtype), st.acc, sq)
        d = tree_map(lambda x, a, u: x.to(a.dtype) * (u + eps).sqrt() / (a.clamp(min=0) + eps).sqrt(), g, acc, st.aux)
        dacc = tree_map(lambda u, y: rho * u + (1 - rho) * y * y, st.aux, d)
        return tree_map(lambda x, y: y.to(x.dtype), g, d), AccumState(acc, dacc, st.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="adadelta",
                                decoupled_weight_decay=False)


# ------------------------------------------------------------------------------------------------ Lion / RAdam / AdEMAMix
def lion(lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
    b1, b2 = betas

    def init(params):
        return MomentumState(_zeros(params))

    def update(g, st, *, params=None):
        d = tree_map(lambda m, x: torch.sign(b1 * m + (1 - b1) * x.to(m.dtype)).to(x.dtype), st.trace, g)
        tr = tree_map(lambda m, x: b2 * m + (1 - b2) * x.to(m.dtype), st.trace, g)
        return d, MomentumState(tr, st.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="lion")


@dataclass(frozen=True)
class TwoMomentState:
    mu: Any
    nu: Any
    slow: Any = None
    step: int = 0


def radam(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, *, decoupled_weight_decay=False):
    b1, b2 = betas
    rho_inf = 2.0 / (1.0 - b2) - 1.0

    def init(params):
        return TwoMomentState(_zeros(params), _zeros(params))

    def update(g, st, *, params=None, noisy_squared_grads=None):
        t = st.step + 1
        sq = noisy_squared_grads if noisy_squared_grads is not None else tree_map(lambda x: x.float() ** 2, g)
        mu = tree_map(lambda m, x: b1 * m + (1 - b1) * x.to(m.dtype), st.mu, g)
        nu = tree_map(lambda v, s: b2 * v + (1 - b2) * s.to(v.dtype), st.nu, sq)
        bc1, bc2 = 1 - b1**t, 1 - b2**t
        rho_t = rho_inf - 2.0 * t * b2**t / bc2
        if rho_t > 5.0:
            r = math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t))
            d = tree_map(lambda x, m, v: (r * (m / bc1) / ((v.clamp(min=0) / bc2).sqrt() + eps)).to(x.dtype), g, mu, nu)
        else:
            d = tree_map(lambda x, m: (m / bc1).to(x.dtype), g, mu)
        return d, TwoMomentState(mu, nu, None, t)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="radam",
                                decoupled_weight_decay=decoupled_weight_decay)


def ademamix(lr=1e-3, betas=(0.9, 0.999, 0.9999), alpha=5.0, eps=1e-8, weight_decay=0.0, *, t_alpha=None,
             t_beta3=None):
    b1, b2, b3 = betas

    def init(params):
        return TwoMomentState(_zeros(params), _zeros(params), _zeros(params))

    def update(g, st, *, params=None, noisy_squared_grads=None):
        t = st.step + 1
        a_t = alpha if not t_alpha else min(t * alpha / t_alpha, alpha)
        if t_beta3:
            ln1, ln3 = math.log(b1), math.log(b3)
            frac = min(t / t_beta3, 1.0)
            b3_t = min(math.exp(ln1 * ln3 / ((1 - frac) * ln3 + frac * ln1)), b3)
        else:
            b3_t = b3
        sq = noisy_squared_grads if noisy_squared_grads is not None else tree_map(lambda x: x.float() ** 2, g)
        mu = tree_map(lambda m, x: b1 * m + (1 - b1) * x.to(m.dtype), st.mu, g)
        slow = tree_map(lambda m, x: b3_t * m + (1 - b3_t) * x.to(m.dtype), st.slow, g)
        nu = tree_map(lambda v, s: b2 * v + (1 - b2) * s.to(v.dtype), st.nu, sq)
        bc1, bc2 = 1 - b1**t, 1 - b2**t
        d = tree_map(lambda x, m, s, v: ((m / bc1 + a_t * s) / ((v.clamp(min=0) / bc2).sqrt() + eps)).to(x.dtype), g, mu, slow, nu)
        return d, TwoMomentState(mu, nu, slow, t)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="ademamix")


# ------------------------------------------------------------------------------------------------ Adafactor
@dataclass(frozen=True)
class AdafactorState:
    row: Any
    col: Any
    full: Any
    step: int = 0


def adafactor(lr=1e-3, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8, weight_decay=0.0, *,
              scale_parameter=False):
    e1, e2 = eps

    def factored(p):
        return p.dim() >= 2

    def init(params):
        row = tree_map(lambda p: torch.zeros(p.shape[:-1], dtype=torch.float32, device=p.device) if factored(p) else None, params)
        col = tree_map(lambda p: torch.zeros(p.shape[:-2] + p.shape[-1:], dtype=torch.float32, device=p.device) if factored(p) else None, params)
        full = tree_map(lambda p: None if factored(p) else _f32(p), params)
        return AdafactorState(row, col, full)

    def update(g, st, *, params=None):
        from ..engine.pytree import tree_flatten_with_paths, tree_unflatten

        t = st.step + 1
        beta2 = 1.0 - t**decay_rate
        paths, gl, td = tree_flatten_with_paths(g)

        def leaves_with_none(tree):
            # None entries disappear on flatten; rebuild aligned lists by walking the gradient paths
            out = []
            for p in paths:
                node = tree
                for k in p:
                    node = node[k]
                out.append(node)
            return out

        rows, cols, fulls = leaves_with_none(st.row), leaves_with_none(st.col), leaves_with_none(st.full)
        pl = leaves_with_none(params) if (scale_parameter and params is not None) else [None] * len(gl)
        outs, nr, nc, nf = [], [], [], []
        for x, r, c, f, p in zip(gl, rows, cols, fulls, pl):
            x32 = x.float()
            sq = x32 * x32 + e1
            if r is not None:
                r = beta2 * r + (1 - beta2) * sq.mean(-1)
                c = beta2 * c + (1 - beta2) * sq.mean(-2)
                rf = (r / r.mean(-1, keepdim=True)).rsqrt().unsqueeze(-1)
                u = x32 * rf * c.rsqrt().unsqueeze(-2)
            else:
                f = beta2 * f + (1 - beta2) * sq
                u = x32 * f.rsqrt()
            u = u / max(1.0, float((u.pow(2).mean().sqrt() / clip_threshold)))
            if p is not None:
                u = u * max(e2, float(p.float().pow(2).mean().sqrt()))
            outs.append(u.to(x.dtype))
            nr.append(r); nc.append(c); nf.append(f)

        def rebuild(vals):
            # same container structure as the gradient tree, with None where a slot is unused
            def build(node, it):
                if isinstance(node, dict):
                    return {k: build(node[k], it) for k in sorted(node)}
                if isinstance(node, (list, tuple)):
                    return type(node)(build(v, it) for v in node)
                return next(it)

            return build(g, iter(vals))

        return tree_unflatten(td, outs), AdafactorState(rebuild(nr), rebuild(nc), rebuild(nf), t)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay, optimizer_name="adafactor")


# ------------------------------------------------------------------------------------------------ schedule-free
@dataclass(frozen=True)
class ScheduleFreeState:
    z: Any          # base iterate
    x: Any          # averaged iterate (evaluation point)
    nu: Any
    weight_sum: float = 0.0
    step: int = 0


def schedule_free(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, *, warmup_steps=0, adam: bool = True):
    """Schedule-free AdamW / SGD (Defazio et al.): parameters handed to the model are ``y = (1-b1) z + b1 x``.

    ``update`` returns the difference ``y_new - y_old`` so that ``apply_updates`` keeps the usual contract; the
    averaged iterate for evaluation is ``state.moment.x``.
    """
    b1, b2 = betas

    def init(params):
        c = (lambda p: p.detach().clone().float())
        return ScheduleFreeState(tree_map(c, params), tree_map(c, params), _zeros(params) if adam else None)

    def update(g, st, *, params=None, noisy_squared_grads=None):
        t = st.step + 1
        sched = min(1.0, t / warmup_steps) if warmup_steps else 1.0
        step_lr = resolve_lr(lr, st.step) * sched
        if adam:
            sq = noisy_squared_grads if noisy_squared_grads is not None else tree_map(lambda x: x.float() ** 2, g)
            nu = tree_map(lambda v, s: b2 * v + (1 - b2) * s.to(v.dtype), st.nu, sq)
            bc2 = 1 - b2**t
            d = tree_map(lambda x, v: x.float() / ((v.clamp(min=0) / bc2).sqrt() + eps), g, nu)
        else:
            nu, d = None, tree_map(lambda x: x.float(), g)
        y_old = tree_map(lambda z, x: (1 - b1) * z + b1 * x, st.z, st.x)
        if weight_decay:
            d = tree_map(lambda u, y: u + weight_decay * y, d, y_old)
        z = tree_map(lambda zz, u: zz - step_lr * u, st.z, d)
        w = step_lr**2
        wsum = st.weight_sum + w
        ck = w / wsum if wsum > 0 else 0.0
        x = tree_map(lambda xx, zz: (1 - ck) * xx + ck * zz, st.x, z)
        y_new = tree_map(lambda zz, xx: (1 - b1) * zz + b1 * xx, z, x)
        delta = tree_map(lambda a, b, gg: (a - b).to(gg.dtype), y_new, y_old, g)
        return delta, ScheduleFreeState(z, x, nu, wsum, t)

    # the scaler already contains lr and weight decay: chain with lr = -1 so the final sign flip cancels
    return make_optimizer_chain(GradientTransformation(init, update), -1.0, 0.0, optimizer_name="schedule_free")


__all__ = ["sgd", "adagrad", "rmsprop", "adadelta", "lion", "radam", "ademamix", "adafactor", "schedule_free"]
