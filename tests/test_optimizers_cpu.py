"""Every optimizer of ``opake_b200.optimizers`` on its own: trajectory against ``torch.optim`` where PyTorch has the
same algorithm, hand-written recurrences for the others, state round trips that continue the trajectory exactly,
learning-rate schedules, weight decay, refusal of un-noised input (the layout of packages/opake-optimizers/tests/)."""
import math

import pytest
import torch

from opake_b200 import optimizers as O
from opake_b200.base.serialization import from_state_dict, state_dict
from opake_b200.engine.types import clipped, noised


def _grads(step: int):
    g = torch.Generator().manual_seed(100 + step)
    return {"w": torch.randn(7, generator=g), "m": torch.randn(3, 4, generator=g)}


def _run(opt, steps: int, params=None, state=None, start: int = 0):
    p = params or {"w": torch.linspace(-1, 1, 7), "m": torch.ones(3, 4) * 0.5}
    st = opt.init(p) if state is None else state
    for t in range(start, start + steps):
        upd, st = opt.update(noised(_grads(t), max_norm=1.0, noise_stddev=0.0), st, params=p)
        p = O.apply_updates(p, upd)
    return p, st


def _run_torch(cls, steps: int, **kw):
    p = [torch.nn.Parameter(torch.linspace(-1, 1, 7)), torch.nn.Parameter(torch.ones(3, 4) * 0.5)]
    opt = cls(p, **kw)
    for t in range(steps):
        g = _grads(t)
        p[0].grad, p[1].grad = g["w"].clone(), g["m"].clone()
        opt.step()
    return {"w": p[0].detach(), "m": p[1].detach()}


_TORCH_PAIRS = [
    ("sgd", dict(lr=0.1), torch.optim.SGD, dict(lr=0.1)),
    ("sgd", dict(lr=0.05, momentum=0.9, weight_decay=0.01), torch.optim.SGD, dict(lr=0.05, momentum=0.9, weight_decay=0.01)),
    ("sgd", dict(lr=0.05, momentum=0.8, nesterov=True), torch.optim.SGD, dict(lr=0.05, momentum=0.8, nesterov=True)),
    ("sgd", dict(lr=0.05, momentum=0.8, dampening=0.3), torch.optim.SGD, dict(lr=0.05, momentum=0.8, dampening=0.3)),
    ("adam", dict(lr=0.01), torch.optim.Adam, dict(lr=0.01)),
    ("adam", dict(lr=0.01, weight_decay=0.1), torch.optim.Adam, dict(lr=0.01, weight_decay=0.1)),
    ("adamw", dict(lr=0.01, weight_decay=0.1, betas=(0.8, 0.95)), torch.optim.AdamW, dict(lr=0.01, weight_decay=0.1, betas=(0.8, 0.95))),
    ("adagrad", dict(lr=0.1), torch.optim.Adagrad, dict(lr=0.1)),
    ("adagrad", dict(lr=0.1, lr_decay=0.05, initial_accumulator_value=0.1, weight_decay=0.01), torch.optim.Adagrad,
     dict(lr=0.1, lr_decay=0.05, initial_accumulator_value=0.1, weight_decay=0.01)),
    ("rmsprop", dict(lr=0.01), torch.optim.RMSprop, dict(lr=0.01)),
    ("rmsprop", dict(lr=0.01, momentum=0.5, centered=True), torch.optim.RMSprop, dict(lr=0.01, momentum=0.5, centered=True)),
    ("adadelta", dict(lr=1.0, rho=0.9), torch.optim.Adadelta, dict(lr=1.0, rho=0.9)),
    ("radam", dict(lr=0.01), torch.optim.RAdam, dict(lr=0.01)),
    ("radam", dict(lr=0.01, weight_decay=0.1, decoupled_weight_decay=True), torch.optim.RAdam,
     dict(lr=0.01, weight_decay=0.1, decoupled_weight_decay=True)),
]


@pytest.mark.parametrize("name,kw,tcls,tkw", _TORCH_PAIRS, ids=[f"{a}-{i}" for i, (a, *_r) in enumerate(_TORCH_PAIRS)])
def test_trajectory_matches_torch_optim(name, kw, tcls, tkw):
    got, _ = _run(getattr(O, name)(**kw), 12)
    want = _run_torch(tcls, 12, **tkw)
    for k in want:
        assert torch.allclose(got[k], want[k], rtol=2e-5, atol=2e-6), (name, kw, k, (got[k] - want[k]).abs().max())


def test_lion_recurrence():
    lr, (b1, b2), wd = 0.01, (0.9, 0.99), 0.1
    got, _ = _run(O.lion(lr=lr, betas=(b1, b2), weight_decay=wd), 8)
    p = {"w": torch.linspace(-1, 1, 7), "m": torch.ones(3, 4) * 0.5}
    m = {k: torch.zeros_like(v) for k, v in p.items()}
    for t in range(8):
        g = _grads(t)
        for k in p:
            u = torch.sign(b1 * m[k] + (1 - b1) * g[k])
            p[k] = p[k] - lr * (u + wd * p[k])
            m[k] = b2 * m[k] + (1 - b2) * g[k]
    for k in p:
        assert torch.allclose(got[k], p[k], atol=1e-6), k


def test_ademamix_recurrence():
    lr, (b1, b2, b3), alpha, eps = 0.01, (0.9, 0.999, 0.9999), 5.0, 1e-8
    got, _ = _run(O.ademamix(lr=lr, betas=(b1, b2, b3), alpha=alpha, eps=eps), 6)
    p = {"w": torch.linspace(-1, 1, 7), "m": torch.ones(3, 4) * 0.5}
    m1 = {k: torch.zeros_like(v) for k, v in p.items()}
    m2 = {k: torch.zeros_like(v) for k, v in p.items()}
    v = {k: torch.zeros_like(x) for k, x in p.items()}
    for t in range(1, 7):
        g = _grads(t - 1)
        for k in p:
            m1[k] = b1 * m1[k] + (1 - b1) * g[k]
            m2[k] = b3 * m2[k] + (1 - b3) * g[k]
            v[k] = b2 * v[k] + (1 - b2) * g[k] ** 2
            upd = (m1[k] / (1 - b1**t) + alpha * m2[k]) / ((v[k] / (1 - b2**t)).sqrt() + eps)
            p[k] = p[k] - lr * upd
    for k in p:
        assert torch.allclose(got[k], p[k], rtol=1e-5, atol=1e-6), k


def test_adafactor_factored_and_unfactored_statistics():
    opt = O.adafactor(lr=0.01)
    p = {"w": torch.linspace(-1, 1, 7), "m": torch.ones(3, 4) * 0.5}
    st = opt.init(p)
    flat = state_dict(st)
    # the matrix keeps a row and a column statistic, the vector a full one
    assert any(tuple(v.shape) == (3,) for v in flat.values() if isinstance(v, torch.Tensor))
    assert any(tuple(v.shape) == (4,) for v in flat.values() if isinstance(v, torch.Tensor))
    assert any(tuple(v.shape) == (7,) for v in flat.values() if isinstance(v, torch.Tensor))
    assert not any(tuple(v.shape) == (3, 4) for v in flat.values() if isinstance(v, torch.Tensor))
    out, _ = _run(opt, 5)
    assert all(torch.isfinite(v).all() for v in out.values())
    # update RMS is clipped to clip_threshold: one step moves no coordinate further than lr * sqrt(n) * threshold
    upd, _ = opt.update(noised({"w": torch.full((7,), 1e6), "m": torch.full((3, 4), 1e6)}, max_norm=1.0, noise_stddev=0.0), st, params=p)
    assert float(upd["w"].pow(2).mean().sqrt()) <= 0.01 * 1.0 * 1.001


def test_schedule_free_interpolates_and_exposes_eval_point():
    opt = O.schedule_free(lr=0.05, warmup_steps=3)
    target = torch.linspace(-1, 1, 7)
    p = {"w": torch.zeros(7)}
    st = opt.init(p)
    for _ in range(400):
        upd, st = opt.update(noised({"w": p["w"] - target}, max_norm=1.0, noise_stddev=0.0), st, params=p)
        p = O.apply_updates(p, upd)
    assert (p["w"] - target).abs().max() < 0.05


@pytest.mark.parametrize("name", ["sgd", "adam", "adamw", "adagrad", "rmsprop", "adadelta", "lion", "radam", "ademamix", "adafactor",
                                  "schedule_free"])
def test_state_round_trip_continues_the_trajectory(name):
    kw = dict(lr=0.02)
    if name == "sgd":
        kw["momentum"] = 0.9
    opt = getattr(O, name)(**kw)
    full, _ = _run(opt, 9)
    half, st = _run(opt, 4)
    flat = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in state_dict(st).items()}
    fresh = getattr(O, name)(**kw)
    restored = from_state_dict(fresh.init({k: torch.zeros_like(v) for k, v in half.items()}), flat)
    resumed, _ = _run(fresh, 5, params=half, state=restored, start=4)
    for k in full:
        assert torch.equal(resumed[k], full[k]), (name, k)


@pytest.mark.parametrize("name", ["sgd", "adamw", "lion", "rmsprop"])
def test_learning_rate_schedule_is_read_per_step(name):
    seen = []

    def lr(step):
        seen.append(step)
        return 0.1 if step < 2 else 0.0

    opt = getattr(O, name)(lr=lr)
    p0 = {"w": torch.linspace(-1, 1, 7), "m": torch.ones(3, 4) * 0.5}
    p2, st = _run(opt, 2, params=p0)
    p5, _ = _run(opt, 3, params=p2, state=st, start=2)
    assert seen[:5] == [0, 1, 2, 3, 4]
    assert not torch.equal(p2["w"], p0["w"]) and torch.equal(p5["w"], p2["w"])          # zero rate: frozen


@pytest.mark.parametrize("name", ["sgd", "adam", "adamw", "adagrad", "rmsprop", "adadelta", "lion", "radam", "ademamix", "adafactor",
                                  "schedule_free"])
def test_optimizers_refuse_gradients_without_noise(name):
    opt = getattr(O, name)(lr=0.01)
    p = {"w": torch.zeros(3)}
    with pytest.raises(TypeError):
        opt.update(clipped({"w": torch.ones(3)}, max_norm=1.0), opt.init(p), params=p)
    # a plain pytree is the non-private use of the same transformation
    upd, _ = opt.update({"w": torch.ones(3)}, opt.init(p), params=p)
    assert torch.isfinite(upd["w"]).all()


def test_noise_bias_correction_subtracts_the_noise_second_moment():
    b2, sigma, lr = 0.99, 0.3, 0.01
    opt = O.adamw(lr, betas=(0.9, b2), weight_decay=0.0, noise_bias_correction=True)
    plain = O.adamw(lr, betas=(0.9, b2), weight_decay=0.0)
    p = {"w": torch.zeros(5)}
    st, st0 = opt.init(p), plain.init(p)
    phi = 0.0
    for t in range(1, 6):
        g = {"w": torch.full((5,), 0.5 + 0.1 * t)}
        u, st = opt.update(noised(g, max_norm=1.0, noise_stddev=sigma), st, params=p)
        u0, st0 = plain.update(noised(g, max_norm=1.0, noise_stddev=sigma), st0, params=p)
        phi = b2 * phi + (1 - b2) * sigma**2
        assert all(v == pytest.approx(phi) for v in st.moment.phi.values())
        assert (u["w"].abs() > u0["w"].abs()).all()           # a smaller denominator: the corrected step is longer
    flat = state_dict(st)
    assert any("phi" in k for k in flat)
