"""DP-SGD / DP-FTRL / accounting / optimizers on CPU, plus benchmark configuration (a): a complete functional DP-SGD loop."""
import json
import math

import numpy as np
import pytest
import torch
from scipy.optimize import brentq
from scipy.stats import kstest, norm

import opake_b200.accounting as acc
from opake_b200 import optimizers as O
from opake_b200.base.serialization import from_state_dict, state_dict
from opake_b200.dpftrl import accounting as facc
from opake_b200.dpftrl.noise import mf_gaussian_noise
from opake_b200.dpftrl.sampling import BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler, SequentialBatchSampler
from opake_b200.dpftrl.strategies import (band_mf_strategy, bisr_strategy, blt_strategy, bsr_strategy, deserialize_strategy,
                                          identity_strategy, lambda_cgd_strategy, serialize_strategy)
from opake_b200.dpsgd import accounting as sacc
from opake_b200.dpsgd import adaptive_clipped_grad, clipped_grad, gaussian_noise
from opake_b200.dpsgd.sampling import KOutOfTSampler, PoissonSampler
from opake_b200.engine.random import key
from opake_b200.engine.types import NoisedPytree, clipped, noised
from opake_b200.ops.philox_ref import normal as philox_normal


def _gauss_eps(nm, delta):
    d = lambda e: norm.cdf(0.5 / nm - e * nm) - math.exp(e) * norm.cdf(-0.5 / nm - e * nm)  # noqa: E731
    return brentq(lambda e: d(e) - delta, 0, 500)


def test_gaussian_mechanism_statistics_and_reproducibility():
    fn, st = gaussian_noise(noise_multiplier=2.0, key=key(1))
    g = clipped({"a": torch.zeros(200000), "b": torch.zeros(7)}, max_norm=0.5)
    n1, st1 = fn(g, st)
    n2, _ = fn(g, st)
    assert torch.equal(n1.pytree["a"], n2.pytree["a"]) and st1._step_counter == 1
    n3, _ = fn(g, st1)
    assert not torch.equal(n1.pytree["a"], n3.pytree["a"])
    assert n1.noise_stddev == 1.0 and abs(n1.pytree["a"].std().item() - 1.0) < 0.01
    assert kstest(n1.pytree["a"].numpy(), "norm").pvalue > 1e-3
    with pytest.raises(TypeError):
        fn(n1, st)
    with pytest.raises(TypeError):
        fn({"a": torch.zeros(3)}, st)
    fnp, stp = gaussian_noise(noise_multiplier=2.0, key=key(1), backend="philox")
    p, _ = fnp(g, stp)
    assert kstest(p.pytree["a"].numpy(), "norm").pvalue > 1e-3
    assert state_dict(st1) == {"_step_counter": 1, "_rng_key.seed": 1, "_rng_key.impl": "opake_threefry_like"}


def test_philox_restatement_is_shard_invariant():
    full = philox_normal(1000, 123456789, 3)
    assert np.array_equal(philox_normal(100, 123456789, 3, offset=333), full[333:433])
    assert not np.array_equal(philox_normal(100, 123456789, 4), full[:100])


def test_samplers_resume_and_properties():
    ds = list(range(2000))
    s = PoissonSampler(ds, 0.01, n_steps=20, key=key(3))
    it = iter(s)
    first = [next(it) for _ in range(6)]
    sd = state_dict(s)
    assert sd["consumed"] == 6 and sd["num_samples"] == 2000
    rest = list(it)
    s2 = from_state_dict(PoissonSampler(ds, 0.5, n_steps=20, key=key(99)), sd)
    assert list(s2) == rest
    with pytest.raises(ValueError):
        from_state_dict(PoissonSampler(ds[:10], 0.5, key=key(0)), sd)
    sizes = [len(b) for b in PoissonSampler(ds, 0.05, n_steps=200, key=key(4))]
    assert abs(np.mean(sizes) - 100) < 5
    assert max(len(b) for b in PoissonSampler(ds, 0.05, n_steps=50, truncated_batch_size=90, key=key(4))) <= 90
    for alloc in ("block", "total"):
        counts = np.zeros(2000, int)
        for b in KOutOfTSampler(ds, k=3, t=10, allocation=alloc, key=key(5)):
            counts[b] += 1
        assert (counts == 3).all()
    for mk in (lambda k: CyclicPoissonSampler(ds, 0.1, bands=4, n_steps=12, key=k), lambda k: BMinSepSampler(ds[:300], 3, 0.1, 12, key=k),
               lambda k: BallsInBinsSampler(ds, 4, 12, key=k), lambda k: SequentialBatchSampler(ds, 64, 12)):
        s = mk(key(1))
        it = iter(s)
        [next(it) for _ in range(5)]
        sd = state_dict(s)
        rest = list(it)
        assert list(from_state_dict(mk(key(7)), sd)) == rest
    bins = list(BallsInBinsSampler(ds, 4, 8, key=key(2)))
    assert bins[:4] == bins[4:] and sorted(i for b in bins[:4] for i in b) == ds


def test_accountant_closed_forms_and_codec():
    g = sacc.gaussian(1.0)
    assert g.epsilon_at(1e-5) == pytest.approx(_gauss_eps(1.0, 1e-5), abs=1e-6)
    assert (g * 100).epsilon_at(1e-5) == pytest.approx(_gauss_eps(0.1, 1e-5), rel=1e-6)
    assert (sacc.gaussian(2.0) | sacc.gaussian(2.0)).epsilon_at(1e-6) == pytest.approx(_gauss_eps(math.sqrt(2), 1e-6), abs=1e-6)
    assert g.advantage() == pytest.approx(2 * norm.cdf(0.5) - 1, abs=1e-7)
    assert g.beta_at(0.05) == pytest.approx(norm.cdf(norm.ppf(0.95) - 1.0), abs=1e-6)
    step = sacc.poisson(sacc.gaussian(1.1), 256 / 60000)
    exact = sacc.parallel_poisson(sacc.gaussian(1.1), 256 / 60000, 1)
    assert step.epsilon_at(1e-5) == pytest.approx(exact.epsilon_at(1e-5), abs=1e-8)
    assert (step * 200).epsilon_at(1e-5) < (sacc.gaussian(1.1) * 200).epsilon_at(1e-5)
    a = acc.Accountant(budget=acc.epsilon_budget(3.0, 1e-5))
    for _ in range(50):
        a = a | step
    assert isinstance(a.process, acc.Repeated) and a.process.count == 50 and not a.budget_exceeded
    a = a | sacc.poisson(sacc.gaussian(0.9), 0.01) * 3 | acc.eps_delta(0.1)
    js = json.dumps(state_dict(a))
    b = from_state_dict(acc.Accountant(), json.loads(js))
    assert b.process == a.process and b.budget == a.budget
    assert b.epsilon_at(1e-5) == pytest.approx(a.epsilon_at(1e-5))
    assert (acc.identity() | g) == g and acc.nonprivate().epsilon_at(1e-5) == math.inf
    with pytest.raises(ValueError):
        g * 0
    assert sacc.adaclip(sacc.gaussian(1.0), fraction_noise_std=0.5, expected_batch_size=1.0).effective_noise_multiplier == \
        pytest.approx(1 / math.sqrt(2))


def test_calibrate_is_one_sided():
    r = acc.calibrate(acc.epsilon_budget(2.0, 1e-5), lambda nm: sacc.gaussian(nm) * 10, 0.5, 50.0)
    assert r.converged and r.achieved <= 2.0 and r.achieved == pytest.approx(2.0, rel=1e-5)
    assert _gauss_eps(r.param / math.sqrt(10), 1e-5) == pytest.approx(r.achieved, abs=1e-4)
    with pytest.raises(acc.calibration.CalibrationError):
        acc.calibrate(acc.epsilon_budget(2.0, 1e-5), lambda nm: sacc.gaussian(nm), 50.0, 60.0)
    r2 = acc.calibrate(acc.epsilon_budget(1.0, 1e-5), lambda q: sacc.poisson(sacc.gaussian(1.0), q) * 100, 1e-4, 0.5)
    assert r2.achieved <= 1.0


def test_mf_strategies_invert_and_account():
    n = 64
    for s in (identity_strategy(), bsr_strategy(bandwidth=8, alpha=1.0, beta=0.0), band_mf_strategy(bands=4),
              blt_strategy(max_buffers=2), bisr_strategy(bandwidth=4)):
        sm = s.streaming_matrix(n_steps=n)
        st = sm.init_multiply({"w": torch.zeros(3)})
        torch.manual_seed(0)
        zs, ys = [torch.randn(3) for _ in range(n)], []
        for z in zs:
            y, st = sm.multiply_next({"w": z}, st)
            ys.append(y["w"])
        c = s.strategy_coefficients(n)
        Y, Z = torch.stack(ys).double().numpy(), torch.stack(zs).double().numpy()
        rec = np.stack([np.convolve(c, Y[:, j])[:n] for j in range(3)], 1)
        assert np.abs(rec - Z).max() < 1e-4, s.name
        assert deserialize_strategy(serialize_strategy(s)).name == s.name
    tmpl = {"w": torch.zeros(20000)}
    fn, st = mf_gaussian_noise(tmpl, bsr_strategy(bandwidth=8, alpha=1.0, beta=0.0), n_steps=8, noise_multiplier=2.0, key=key(0))
    tot = torch.zeros(20000)
    for t in range(8):
        nz, st = fn(clipped(tmpl, max_norm=0.5), st)
        tot += nz.pytree["w"]
        assert abs(nz.pytree["w"].std().item() - nz.noise_stddev) < 0.03
    assert tot.std().item() < 0.75 * math.sqrt(8)          # anti-correlated: prefix sums grow slower than iid noise
    st2 = from_state_dict(st, state_dict(st))
    assert st2._step_counter == 8
    with pytest.raises(RuntimeError):
        fn(clipped(tmpl, max_norm=0.5), st)
    m = facc.mf_gaussian(5.0, bsr_strategy(bandwidth=8, alpha=1.0, beta=0.0), n_steps=128, min_sep=32, max_participations=4)
    assert m.epsilon_at(1e-5) == pytest.approx(_gauss_eps(5.0 / m.sensitivity(), 1e-5), abs=1e-5)
    a = acc.Accountant() | m
    assert from_state_dict(acc.Accountant(), json.loads(json.dumps(state_dict(a)))).process == m
    cyc = facc.poisson(facc.mf_gaussian(2.0, band_mf_strategy(bands=4)), 0.05, n_steps=64)
    assert 0 < cyc.epsilon_at(1e-5) < facc.mf_gaussian(2.0, band_mf_strategy(bands=4), n_steps=64, min_sep=4).epsilon_at(1e-5)
    assert lambda_cgd_strategy(lambda_=0.5).sensitivity_squared(n_steps=16, min_sep=16) == pytest.approx(1.0)


def test_optimizers_converge_and_route_metadata():
    torch.manual_seed(0)
    target = torch.randn(10)
    for name in ("sgd", "adam", "adamw", "rmsprop", "lion", "radam", "ademamix", "adafactor", "schedule_free"):
        p = {"w": torch.zeros(10), "m": torch.zeros(4, 5)}
        opt = getattr(O, name)(lr=0.05)
        st = opt.init(p)
        for _ in range(300):
            g = {"w": p["w"] - target, "m": p["m"] - 1.0}
            upd, st = opt.update(noised(g, max_norm=1.0, noise_stddev=0.0), st, params=p)
            p = O.apply_updates(p, upd)
        assert (p["w"] - target).abs().max() < 0.06, name
    opt = O.adamw(1e-2, noise_bias_correction=True)
    st = opt.init({"w": torch.zeros(3)})
    u, st = opt.update(noised({"w": torch.ones(3)}, max_norm=1.0, noise_stddev=0.5), st, params={"w": torch.zeros(3)})
    assert all(v == pytest.approx((1 - 0.999) * 0.25) for v in st.moment.phi.values())
    # first step: v_hat = g^2 = 1, phi_hat = 0.25 -> update = -lr * 1 / sqrt(0.75)
    assert u["w"][0].item() == pytest.approx(-1e-2 / math.sqrt(0.75), rel=1e-4)
    with pytest.raises(TypeError):
        opt.update(clipped({"w": torch.ones(3)}, max_norm=1.0), st, params={"w": torch.zeros(3)})
    with pytest.raises(TypeError):
        O.lion(1e-3).update(__import__("opake_b200.engine.types", fromlist=["x"]).SecondMomentNoiseOutput(
            noised({"w": torch.ones(3)}, max_norm=1.0, noise_stddev=0.1), noised({"w": torch.ones(3)}, max_norm=1.0, noise_stddev=0.1)),
            O.lion(1e-3).init({"w": torch.zeros(3)}), params={"w": torch.zeros(3)})


def test_adaptive_clipping_tracks_quantile():
    torch.manual_seed(0)
    w = {"w": torch.randn(3, 4)}
    loss = lambda p, x, y: ((p["w"] @ x - y) ** 2).sum()  # noqa: E731
    x, y = torch.randn(64, 4), torch.randn(64, 3)
    fn, st = adaptive_clipped_grad(loss, initial_clipping_norm=0.01, key=key(0), batch_argnums=(1, 2), normalize_by=64.0,
                                   learning_rate=0.5, fraction_noise_std=0.01, return_stats=True)
    for _ in range(40):
        (g, stats), st = fn(w, x, y, state=st)
    assert 0.2 < stats.clipping_rate < 0.8 and st._step == 40 and g.max_norm == pytest.approx(st._current_clipping_norm / 64)


def test_baseline_config_a_functional_dpsgd_loop():
    """MLP 784->512->10 on synthetic data, Poisson q = 256/60000, C = 1, sigma = 1.1, SGD 0.1 (shortened to 25 steps)."""
    torch.manual_seed(0)
    N = 6000
    X, Y = torch.randn(N, 784), torch.randint(0, 10, (N,))
    model = torch.nn.Sequential(torch.nn.Linear(784, 512), torch.nn.ReLU(), torch.nn.Linear(512, 10))
    from opake_b200.engine.functional import make_functional

    fmodel, params = make_functional(model, disable_autograd_tracking=True)
    loss_fn = lambda p, x, y: torch.nn.functional.cross_entropy(fmodel(p, x.unsqueeze(0)), y.unsqueeze(0))  # noqa: E731
    q, B = 256 / N, 256.0
    grad_fn, cst = clipped_grad(loss_fn, clipping_norm=1.0, normalize_by=B, batch_argnums=(1, 2), microbatch_size=128)
    noise_fn, nst = gaussian_noise(noise_multiplier=1.1, key=key(0))
    opt = O.sgd(0.1)
    ost = opt.init(params)
    acct = acc.Accountant()
    step_proc = sacc.poisson(sacc.gaussian(1.1), q)
    losses = []
    for idx in PoissonSampler(range(N), q, n_steps=25, key=key(1)):
        xb, yb = X[idx], Y[idx]
        g, cst = grad_fn(params, xb, yb, state=cst)
        assert g.max_norm == pytest.approx(1.0 / B)
        ng, nst = noise_fn(g, nst)
        assert isinstance(ng, NoisedPytree) and ng.noise_stddev == pytest.approx(1.1 / B)
        upd, ost = opt.update(ng, ost, params=params)
        params = O.apply_updates(params, upd)
        acct = acct | step_proc
        with torch.no_grad():
            losses.append(torch.nn.functional.cross_entropy(fmodel(params, X[:512]), Y[:512]).item())
    eps = acct.epsilon_at(1e-5)
    assert 0 < eps < 3.0 and acct.process.count == 25 and all(math.isfinite(l) for l in losses)
