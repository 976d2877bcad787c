"""Base + engine layers on CPU: serialization format, RngKey derivation, DP types, pytree utils, clipping numerics."""
import dataclasses
import hashlib
import math
from typing import NamedTuple

import numpy as np
import pytest
import torch

from opake_b200.base import exceptions as E
from opake_b200.base.serialization import from_state_dict, register_serializer, state_dict
from opake_b200.engine import pytree as P
from opake_b200.engine.clipping import clipped_fun, clipped_grad
from opake_b200.engine.clipping import numerics as N
from opake_b200.engine.clipping.auto import auto_clipped_grad
from opake_b200.engine.clipping.per_group import per_group
from opake_b200.engine.noise_allocation import paired_noise_stddevs, per_group_noise_stddev
from opake_b200.engine.random import RngKey, fold_in, generator_from_key, key, split
from opake_b200.engine.types import ClippedPytree, NoisedPytree, PerGroup, clipped, noised


def test_exception_taxonomy():
    assert issubclass(E.ConfigurationError, ValueError) and issubclass(E.InputTypeError, TypeError)
    assert issubclass(E.CheckpointError, RuntimeError) and issubclass(E.CalibrationError, E.ConfigurationError)
    with pytest.raises(E.PrivacyBudgetError, match="boom"):
        E.PrivacyBudgetError.raise_("boom")


@dataclasses.dataclass(frozen=True)
class _Inner:
    a: int
    t: torch.Tensor


class _NT(NamedTuple):
    x: float
    y: list


def test_state_dict_flat_paths_and_template_restore():
    obj = {"p": _Inner(1, torch.arange(3.0)), "n": _NT(2.5, [1, {"k": "v"}]), "tup": (7, 8)}
    sd = state_dict(obj)
    assert set(sd) == {"p.a", "p.t", "n.x", "n.y[0]", "n.y[1].k", "tup[0]", "tup[1]"}
    tmpl = {"p": _Inner(0, torch.zeros(3)), "n": _NT(0.0, [0, {"k": ""}]), "tup": (0, 0)}
    back = from_state_dict(tmpl, sd)
    assert back["p"].a == 1 and torch.equal(back["p"].t, torch.arange(3.0)) and back["n"].y[1]["k"] == "v"
    # missing leaves keep the template's value; shape mismatch is an error with a path note
    del sd["p.a"]
    assert from_state_dict(tmpl, sd)["p"].a == 0
    sd["p.t"] = torch.zeros(4)
    with pytest.raises(E.CheckpointError):
        from_state_dict(tmpl, sd)
    with pytest.raises(TypeError, match="not a registered type"):
        state_dict({"x": object()})


def test_rngkey_matches_blake2b_formula():
    def ref(seed, d):
        h = hashlib.blake2b(digest_size=8)
        h.update(b"i" + seed.to_bytes(16, "little", signed=True) + b"|")
        h.update((b"i" + d.to_bytes(16, "little", signed=True)) if isinstance(d, int) else (b"s" + d.encode()))
        h.update(b"|")
        return int.from_bytes(h.digest(), "little")

    k = key(42)
    assert fold_in(k, "opake.dpsgd.gaussian").seed == ref(42, "opake.dpsgd.gaussian")
    assert fold_in(k, "a", 3).seed == ref(ref(42, "a"), 3)
    assert fold_in(k, 1).seed != fold_in(k, "1").seed
    assert split(k, 3) == tuple(fold_in(k, i) for i in range(3))
    assert key(-1).seed == 2**64 - 1
    g1, g2 = generator_from_key(k), generator_from_key(k)
    assert torch.equal(torch.randn(4, generator=g1), torch.randn(4, generator=g2))
    with pytest.raises(TypeError):
        key(True)
    assert state_dict(k) == {"seed": 42, "impl": "opake_threefry_like"}


def test_clipped_pytree_arithmetic_rules():
    c = clipped({"w": torch.ones(2)}, max_norm=2.0)
    assert (c * 0.5).max_norm == 1.0 and (-c).max_norm == 2.0 and (c / 4).max_norm == 0.5
    assert (3 * c).pytree["w"].tolist() == [3.0, 3.0]
    for bad in (lambda: c + c, lambda: c - 1, lambda: c ** 2, lambda: 1 / c, lambda: c * torch.tensor(2.0)):
        with pytest.raises(TypeError):
            bad()
    n = noised({"w": torch.ones(2)}, max_norm=1.0, noise_stddev=0.5) * 2
    assert isinstance(n, NoisedPytree) and n.noise_stddev == 1.0
    pg = PerGroup({("a",): "g1", ("b",): "g2"}, {"g1": 3.0, "g2": 4.0})
    assert pg.effective == 5.0 and (pg * pg).values["g2"] == 16.0 and pg.for_path("a") == 3.0
    assert clipped({}, max_norm=pg).sensitivity == 5.0
    sig = per_group_noise_stddev(pg, 2.0)
    assert sig.values["g1"] == pytest.approx(2 * math.sqrt(3 * 7))
    s1, s2 = paired_noise_stddevs(1.5, first=0.1, second=0.01)
    assert (0.1 / s1) ** 2 + (0.01 / s2) ** 2 == pytest.approx(1 / 1.5**2)


def test_pytree_utils():
    t = {"b": {"w": torch.ones(2)}, "a": [torch.ones(3), torch.zeros(1)]}
    paths, leaves, td = P.tree_flatten_with_paths(t)
    assert paths == [("a", 0), ("a", 1), ("b", "w")]
    assert P.tree_unflatten(td, leaves)["b"]["w"] is leaves[2]
    assert P.global_norm(t).item() == pytest.approx(math.sqrt(5))
    yes, no = P.partition(lambda p, v: "w" in p, t)
    assert list(yes) == ["b"] and "b" not in no
    assert P.merge(yes, no).keys() == t.keys()
    with pytest.raises(TypeError):
        P.global_norm(clipped(t, max_norm=1.0))


def _loop_oracle(loss, w, xs, ys, C):
    tot = {k: torch.zeros_like(v) for k, v in w.items()}
    for i in range(len(xs)):
        p = {k: v.clone().requires_grad_() for k, v in w.items()}
        loss(p, xs[i], ys[i]).backward()
        n = math.sqrt(sum(v.grad.double().pow(2).sum().item() for v in p.values()))
        s = min(1.0, C / n) if n > 0 else 1.0
        for k in tot:
            tot[k] += p[k].grad * s
    return tot


def test_clipped_grad_matches_loop_and_conservative_bound():
    torch.manual_seed(0)
    w = {"w": torch.randn(3, 4), "b": torch.zeros(3)}
    loss = lambda p, x, y: ((p["w"] @ x + p["b"] - y) ** 2).sum()  # noqa: E731
    x, y = torch.randn(9, 4), torch.randn(9, 3)
    fn, st = clipped_grad(loss, clipping_norm=0.5, normalize_by=9.0, batch_argnums=(1, 2), return_aux=True, microbatch_size=4)
    (g, aux), st = fn(w, x, y, state=st)
    ref = _loop_oracle(loss, w, x, y, 0.5)
    for k in ref:
        assert torch.allclose(g.pytree[k] * 9, ref[k], rtol=1e-5, atol=1e-6)
    assert g.max_norm == pytest.approx(0.5 / 9) and aux.batch_size == 9
    assert (aux.clipped_grad_norms <= 0.5).all()          # never above the bound, even after rounding
    assert aux.clipping_rate == pytest.approx((aux.grad_norms > 0.5).float().mean().item())
    # empty batch -> zeros with the same sensitivity
    g0, _ = clipped_grad(loss, clipping_norm=0.5, batch_argnums=(1, 2))[0](w, x[:0], y[:0], state=st)
    assert g0.max_norm == 0.5 and all((v == 0).all() for v in g0.pytree.values())


def test_bf16_clip_never_exceeds_bound():
    torch.manual_seed(1)
    g = [torch.randn(16, 5000).bfloat16() * 3, torch.randn(16, 7, 3).bfloat16()]
    sq = sum(N.per_example_sq(l, torch.float64) for l in g)
    f, norms, mask = N.clip_factors(sq, 1.0, g)
    out = [N.scale_leaf(l, ff) for l, ff in zip(g, f)]
    after = torch.sqrt(sum(N.per_example_sq(o, torch.float64) for o in out))
    assert (after <= 1.0).all() and (after > 0.98).all() and mask.all()
    f2, _, _ = N.clip_factors(sq, float("inf"), g)
    assert all((x == 1).all() for x in f2)
    f3, _, _ = N.clip_factors(sq, 0.0, g)
    assert all((x == 0).all() for x in f3)


def test_auto_and_per_group_clipping():
    torch.manual_seed(2)
    w = {"lin": {"w": torch.randn(3, 4), "b": torch.zeros(3)}}
    loss = lambda p, x, y: ((p["lin"]["w"] @ x + p["lin"]["b"] - y) ** 2).sum()  # noqa: E731
    x, y = torch.randn(6, 4), torch.randn(6, 3)
    fn, st = auto_clipped_grad(loss, R=1.0, gamma=0.01, batch_argnums=(1, 2), return_aux=True)
    (g, aux), _ = fn(w, x, y, state=st)
    assert torch.allclose(aux.clipped_grad_norms, aux.grad_norms / (aux.grad_norms + 0.01), rtol=1e-3)
    pg = per_group(w, {"lin.w": 0.3, "lin.b": 0.1})
    fn, st = clipped_grad(loss, clipping_norm=pg, batch_argnums=(1, 2), return_stats=True)
    (g, stats), _ = fn(w, x, y, state=st)
    assert set(stats.num_clipped) == {"lin.w", "lin.b"} and g.max_norm.values == {"lin.w": 0.3, "lin.b": 0.1}
    with pytest.raises(ValueError, match="did not match"):
        per_group(w, {"nope": 1.0})
    with pytest.raises(ValueError, match="multiple patterns"):
        per_group(w, {"lin": 1.0, "w": 1.0}, allow_unused_patterns=True)


def test_streaming_clip_and_sum_matches_materialised_scaling():
    """The two-pass streaming path (one leaf at a time) equals scaling a full copy of the per-example gradients, for
    fixed clipping, AUTO-S, a custom scale function and the second-moment stream; the backend choice follows the rules
    of the reference's resolver."""
    import torch

    from opake_b200.engine.clipping import numerics as N
    from opake_b200.engine.clipping.streaming import resolve_stream_impl, stream_clip_and_sum

    g = torch.Generator().manual_seed(0)
    leaves = [torch.randn(6, 5, 3, generator=g) * 3, torch.randn(6, 7, generator=g), torch.randn(6, generator=g)]
    sq = sum(N.per_example_sq(l, torch.float64) for l in leaves)
    for auto in (False, True):
        sums, sq_sums, norms, mask, post = stream_clip_and_sum(leaves, 1.5, auto=auto, second_moment=True, with_postsq=True)
        factors, norms_ref, mask_ref = N.clip_factors(sq, 1.5, leaves, auto=auto, gamma=0.01)
        scaled = [N.scale_leaf(l, f) for l, f in zip(leaves, factors)]
        for a, b in zip(sums, scaled):
            assert torch.equal(a, b.sum(0, dtype=N.acc_dtype_of(b.dtype)))
        for a, b in zip(sq_sums, scaled):
            assert torch.allclose(a, (b ** 2).sum(0))
        assert torch.equal(norms, norms_ref) and torch.equal(mask, mask_ref)
        assert torch.allclose(post, torch.sqrt(sum(N.per_example_sq(s, torch.float64) for s in scaled)))
        if not auto:
            assert float(post.max()) <= 1.5
    sums, _, norms, mask, _ = stream_clip_and_sum(leaves, 1.0, scale_fn=lambda n: torch.clamp(0.5 / n, max=1.0).to(torch.float32))
    assert sums[0].shape == (5, 3) and mask.dtype == torch.bool
    assert resolve_stream_impl(leaves, 1.0) == "stream"                       # CPU leaves: no fused backend applies
    assert resolve_stream_impl(leaves, 1.0, second_moment=True) == "stream"
