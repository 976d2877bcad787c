"""Every matrix-factorisation strategy on its own (the layout of packages/opake-dpftrl/tests/noise): the streaming
``C^{-1}`` inverts the strategy's Toeplitz ``C``, sensitivities against a dense construction, codec round trips, the
realised per-step noise scale, state round trips that continue the correlated stream."""
import math

import numpy as np
import pytest
import torch

from opake_b200.base.serialization import from_state_dict, state_dict
from opake_b200.dpftrl.noise import mf_gaussian_noise
from opake_b200.dpftrl.strategies import (band_mf_strategy, bisr_strategy, blt_strategy, bsr_strategy, deserialize_strategy,
                                          identity_strategy, lambda_cgd_strategy, serialize_strategy)
from opake_b200.engine.random import key
from opake_b200.engine.types import clipped

_STRATEGIES = {
    "identity": identity_strategy,
    "bsr": lambda: bsr_strategy(bandwidth=6, alpha=1.0, beta=0.0),
    "bsr_momentum": lambda: bsr_strategy(bandwidth=6, alpha=0.99, beta=0.9),
    "band_mf": lambda: band_mf_strategy(bands=4),
    "blt": lambda: blt_strategy(max_buffers=3).optimize(40),          # fitted once: the same C for every query below
    "bisr": lambda: bisr_strategy(bandwidth=4),
    "lambda_cgd": lambda: lambda_cgd_strategy(lambda_=0.5, normalized=False),
}


def _toeplitz(c: np.ndarray, n: int) -> np.ndarray:
    c = np.concatenate([np.asarray(c, float), np.zeros(max(0, n - len(c)))])[:n]
    return np.array([[c[i - j] if i >= j else 0.0 for j in range(n)] for i in range(n)])


@pytest.mark.parametrize("name", list(_STRATEGIES))
def test_streaming_inverse_inverts_the_strategy_matrix(name):
    n = 40
    s = _STRATEGIES[name]()
    sm = s.streaming_matrix(n_steps=n)
    st = sm.init_multiply({"w": torch.zeros(5), "b": torch.zeros(2, 2)})
    g = torch.Generator().manual_seed(0)
    Z = [{"w": torch.randn(5, generator=g, dtype=torch.float64), "b": torch.randn(2, 2, generator=g, dtype=torch.float64)} for _ in range(n)]
    Y = []
    for z in Z:
        y, st = sm.multiply_next(z, st)
        Y.append(y)
    C = _toeplitz(s.strategy_coefficients(n), n)
    for leaf, shape in (("w", 5), ("b", 4)):
        Zm = np.stack([z[leaf].reshape(-1).numpy() for z in Z])
        Ym = np.stack([y[leaf].reshape(-1).double().numpy() for y in Y])
        assert Zm.shape[1] == shape and np.abs(C @ Ym - Zm).max() < 5e-5, (name, leaf, np.abs(C @ Ym - Zm).max())


@pytest.mark.parametrize("name", list(_STRATEGIES))
@pytest.mark.parametrize("min_sep,k", [(1, None), (4, None), (8, 3)])
def test_sensitivity_matches_the_dense_column_norm(name, min_sep, k):
    n = 32
    s = _STRATEGIES[name]()
    C = _toeplitz(s.strategy_coefficients(n), n)
    G = C.T @ C
    # worst participation pattern: positions separated by at least min_sep, at most k of them (brute force over starts;
    # for non-negative Gram entries the densest pattern from some start is the worst one)
    best = 0.0
    for start in range(min_sep):
        idx = list(range(start, n, min_sep))
        if k is not None:
            for off in range(0, max(1, len(idx) - k + 1)):
                sub = idx[off:off + k]
                best = max(best, float(np.abs(G[np.ix_(sub, sub)]).sum()))
        else:
            best = max(best, float(np.abs(G[np.ix_(idx, idx)]).sum()))
    got = s.sensitivity_squared(n_steps=n, min_sep=min_sep, max_participations=k)
    assert got >= best * (1 - 1e-9) - 1e-12, (name, got, best)                      # never under-reports
    assert got <= best * 1.0001 + 1e-9 or name in ("blt", "bisr", "lambda_cgd", "bsr_momentum"), (name, got, best)   # exact for non-negative C
    assert s.sensitivity(n_steps=n, min_sep=min_sep, max_participations=k) == pytest.approx(math.sqrt(got))


@pytest.mark.parametrize("name", list(_STRATEGIES))
def test_strategy_codec_round_trip(name):
    s = _STRATEGIES[name]()
    d = serialize_strategy(s)
    assert isinstance(d, dict) and d["kind"] == s.name
    back = deserialize_strategy(d)
    assert type(back) is type(s) and back == s
    assert np.allclose(back.strategy_coefficients(16), s.strategy_coefficients(16))


@pytest.mark.parametrize("name", list(_STRATEGIES))
def test_noise_scale_follows_the_rows_of_the_inverse_and_state_resumes(name):
    n, sigma, C_ = 10, 1.5, 0.7
    s = _STRATEGIES[name]()
    tmpl = {"w": torch.zeros(40000)}
    fn, st = mf_gaussian_noise(tmpl, s, n_steps=n, noise_multiplier=sigma, key=key(5))
    g = clipped(tmpl, max_norm=C_)
    Cinv = np.linalg.inv(_toeplitz(s.strategy_coefficients(n), n))
    outs = []
    mid = None
    for t in range(n):
        if t == 4:
            mid = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in state_dict(st).items()}
        nz, st = fn(g, st)
        outs.append(nz.pytree["w"].clone())
        want = sigma * C_ * math.sqrt(float((Cinv[t] ** 2).sum()))      # the accountant divides sigma by sens(C)
        assert float(nz.noise_stddev) == pytest.approx(want, rel=1e-5), (name, t)
        assert abs(nz.pytree["w"].std().item() - want) < 0.03 * want + 1e-3
    # a state written after four steps continues the same correlated stream
    fn2, st2 = mf_gaussian_noise(tmpl, s, n_steps=n, noise_multiplier=sigma, key=key(77))
    st2 = from_state_dict(st2, mid)
    for t in range(4, n):
        nz, st2 = fn2(g, st2)
        assert torch.equal(nz.pytree["w"], outs[t]), (name, t)
    with pytest.raises(RuntimeError):
        fn(g, st)                                       # past the declared horizon


def test_column_normalised_lambda_cgd_inverts_c_times_inverse_column_norms():
    n, lam = 24, 0.6
    s = lambda_cgd_strategy(lambda_=lam)                       # normalised: C~ = C D^-1 with D = column norms of C
    C = _toeplitz(lam ** np.arange(n), n)
    D = np.sqrt((C ** 2).sum(0))
    sm = s.streaming_matrix(n_steps=n)
    st = sm.init_multiply({"w": torch.zeros(3)})
    g = torch.Generator().manual_seed(1)
    Z = [torch.randn(3, generator=g, dtype=torch.float64) for _ in range(n)]
    Y = []
    for z in Z:
        y, st = sm.multiply_next({"w": z}, st)
        Y.append(y["w"].double().numpy())
    assert np.abs((C / D[None, :]) @ np.stack(Y) - np.stack([z.numpy() for z in Z])).max() < 1e-6        # the streaming state is fp32
    # every column of C~ has unit norm, so one participation has sensitivity exactly 1
    assert s.sensitivity_squared(n_steps=n, min_sep=n) == pytest.approx(1.0)
