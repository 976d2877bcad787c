"""Empirical checks of the guarantees the accounting relies on (CPU, functional API).

Modelled on the reference's validation suite
(packages/opake-transformers/tests/validation/test_dp_guarantees.py:94-594): the clipped sum moves by at most the
clipping norm when one record is added, removed or replaced; the noise has the advertised standard deviation and is a
pure function of (key, step); epsilon is monotone in steps, noise and sampling rate; two data-parallel ranks produce
the gradient a single process produces.
"""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from opake_b200.dpsgd import accounting as sacc
from opake_b200.dpsgd import clipped_grad, gaussian_noise
from opake_b200.engine.random import fold_in, key


def _loss(p, x, y):
    return ((p["w"] @ x + p["b"] - y) ** 2).sum()


def _params(seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"w": torch.randn(3, 5, generator=g), "b": torch.randn(3, generator=g)}


def _flat(tree):
    return torch.cat([tree[k].reshape(-1) for k in sorted(tree)])


def _clipped_sum(params, x, y, C):
    fn, st = clipped_grad(_loss, clipping_norm=C, normalize_by=1.0, batch_argnums=(1, 2))
    g, _ = fn(params, x, y, state=st)
    return g


@pytest.mark.parametrize("C", [0.1, 1.0, 7.5])
def test_sensitivity_is_bounded_by_the_clipping_norm(C):
    """Add / remove one record: the clipped sum moves by at most C. Replace one record: by at most 2C."""
    torch.manual_seed(3)
    p = _params()
    x, y = torch.randn(12, 5) * 4, torch.randn(12, 3) * 4          # large residuals: most records are clipped
    full = _clipped_sum(p, x, y, C)
    assert full.max_norm == pytest.approx(C) and full.sensitivity == pytest.approx(C)
    worst_remove = worst_replace = 0.0
    for i in range(12):
        keep = [j for j in range(12) if j != i]
        removed = _clipped_sum(p, x[keep], y[keep], C)
        worst_remove = max(worst_remove, (_flat(full.pytree) - _flat(removed.pytree)).norm().item())
        x2, y2 = x.clone(), y.clone()
        x2[i], y2[i] = torch.randn(5) * 10, torch.randn(3) * 10
        replaced = _clipped_sum(p, x2, y2, C)
        worst_replace = max(worst_replace, (_flat(full.pytree) - _flat(replaced.pytree)).norm().item())
    assert worst_remove <= C * (1 + 1e-6)
    assert worst_replace <= 2 * C * (1 + 1e-6)
    assert worst_remove > 0.5 * C                                  # the bound is attained up to the record's own norm


def test_a_record_with_a_small_gradient_is_not_scaled_up():
    p = _params()
    x, y = torch.randn(4, 5) * 1e-3, torch.zeros(4, 3)
    y = y + (p["w"] @ x.T).T + p["b"]                               # residual 0 -> gradient 0
    g = _clipped_sum(p, x, y, 1.0)
    assert _flat(g.pytree).norm().item() < 1e-4


@pytest.mark.parametrize("sigma,C", [(0.5, 1.0), (1.3, 0.25), (4.0, 3.0)])
def test_noise_standard_deviation_matches_sigma_times_sensitivity(sigma, C):
    from opake_b200.engine.types import clipped

    fn, st = gaussian_noise(noise_multiplier=sigma, key=key(11))
    g = clipped({"a": torch.zeros(400_000)}, max_norm=C)
    out, st = fn(g, st)
    assert out.noise_stddev == pytest.approx(sigma * C)
    emp = out.pytree["a"].std().item()
    assert abs(emp - sigma * C) < 0.01 * sigma * C
    assert abs(out.pytree["a"].mean().item()) < 0.01 * sigma * C


def test_noise_is_a_pure_function_of_key_and_step():
    from opake_b200.engine.types import clipped

    g = clipped({"a": torch.zeros(1000), "b": torch.zeros(3, 3)}, max_norm=1.0)
    fn_a, st_a = gaussian_noise(noise_multiplier=1.0, key=key(5))
    fn_b, st_b = gaussian_noise(noise_multiplier=1.0, key=key(5))
    fn_c, st_c = gaussian_noise(noise_multiplier=1.0, key=key(6))
    a1, st_a = fn_a(g, st_a)
    b1, st_b = fn_b(g, st_b)
    c1, _ = fn_c(g, st_c)
    assert all(torch.equal(a1.pytree[k], b1.pytree[k]) for k in g.pytree)          # same key, same step
    assert not torch.equal(a1.pytree["a"], c1.pytree["a"])                          # different key
    a2, _ = fn_a(g, st_a)
    b2, _ = fn_b(g, st_b)
    assert torch.equal(a2.pytree["a"], b2.pytree["a"]) and not torch.equal(a1.pytree["a"], a2.pytree["a"])
    # leaves draw from disjoint streams
    assert not torch.equal(a1.pytree["a"][:9], a1.pytree["b"].reshape(-1))
    # derived keys are stable and distinct
    assert fold_in(key(5), "noise").seed == fold_in(key(5), "noise").seed != fold_in(key(5), "sampler").seed


def test_epsilon_is_monotone_in_steps_noise_and_sampling_rate():
    delta = 1e-5
    base = sacc.poisson(sacc.gaussian(1.0), 0.01)
    eps = [(base * n).epsilon_at(delta) for n in (1, 10, 100, 1000)]
    assert all(b > a for a, b in zip(eps, eps[1:]))
    by_sigma = [(sacc.poisson(sacc.gaussian(s), 0.01) * 100).epsilon_at(delta) for s in (0.6, 0.9, 1.5, 3.0)]
    assert all(b < a for a, b in zip(by_sigma, by_sigma[1:]))
    by_q = [(sacc.poisson(sacc.gaussian(1.0), q) * 100).epsilon_at(delta) for q in (0.001, 0.01, 0.1, 0.5)]
    assert all(b > a for a, b in zip(by_q, by_q[1:]))
    # subsampling never hurts, and q = 1 is the plain mechanism
    assert (sacc.poisson(sacc.gaussian(1.0), 1.0) * 10).epsilon_at(delta) == pytest.approx(
        (sacc.gaussian(1.0) * 10).epsilon_at(delta), rel=1e-3)
    # smaller delta costs more epsilon
    p = base * 100
    assert p.epsilon_at(1e-7) > p.epsilon_at(1e-5) > p.epsilon_at(1e-3)
    # composition is order-free
    a, b = sacc.poisson(sacc.gaussian(0.8), 0.02) * 30, sacc.gaussian(2.0) * 5
    assert (a | b).epsilon_at(delta) == pytest.approx((b | a).epsilon_at(delta), rel=1e-6)
    assert math.isfinite((a | b).epsilon_at(delta))


# ------------------------------------------------------------------------------------------------ two ranks = one process
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ddp_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from opake_b200.engine.distributed import sum_gradients

    torch.manual_seed(7)
    p = _params()
    x, y = torch.randn(16, 5) * 3, torch.randn(16, 3) * 3
    per = 16 // world
    sl = slice(rank * per, (rank + 1) * per)
    g = _clipped_sum(p, x[sl], y[sl], 0.7)
    g = sum_gradients(g)
    noise_fn, st = gaussian_noise(noise_multiplier=1.1, key=key(42))
    noised, _ = noise_fn(g, st)
    if rank == 0:
        torch.save({"grad": g.pytree, "max_norm": float(g.max_norm), "noised": noised.pytree}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_data_parallel_ranks_equal_a_single_process(tmp_path):
    """Clip locally, SUM across ranks (sensitivity stays C), add the same noise everywhere: the result is what one
    process computes on the whole batch."""
    out = str(tmp_path / "ddp.pt")
    mp.spawn(_ddp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    torch.manual_seed(7)
    p = _params()
    x, y = torch.randn(16, 5) * 3, torch.randn(16, 3) * 3
    ref = _clipped_sum(p, x, y, 0.7)
    assert got["max_norm"] == pytest.approx(0.7)
    for k in ref.pytree:
        assert torch.allclose(got["grad"][k], ref.pytree[k], rtol=1e-5, atol=1e-6)
    noise_fn, st = gaussian_noise(noise_multiplier=1.1, key=key(42))
    noised, _ = noise_fn(ref, st)
    for k in ref.pytree:
        assert torch.allclose(got["noised"][k], noised.pytree[k], rtol=1e-5, atol=1e-6)
