"""Every preference-loss head on its own (the layout of packages/opake-alignment/tests/dpo/loss): per-example
separability (a requirement of per-example clipping), direction of the preference signal, numerical safety at extreme
log-ratios, and the f-divergence / weighting helpers."""
import inspect

import pytest
import torch
import torch.nn.functional as F

from opake_b200.alignment.dpo import loss as L

# discopop blends a logistic and an exponential term with a margin-dependent gate and is non-monotone by construction
_PAIRWISE = [n for n in L.LOSS_HEADS if n not in ("sft", "chosen_nll", "orpo", "discopop")]


def _call(name, c, r, **kw):
    fn = L.LOSS_HEADS[name]
    params = inspect.signature(fn).parameters
    if "beta" in params:
        kw.setdefault("beta", 0.3)
    return fn(c, r, **kw)


@pytest.mark.parametrize("name", sorted(set(L.LOSS_HEADS)))
def test_head_is_per_example_and_finite(name):
    torch.manual_seed(0)
    c, r = torch.randn(6), torch.randn(6)
    if name == "orpo":                              # takes log-probabilities (negative), not log-ratios
        c, r = -c.abs() - 0.1, -r.abs() - 0.1
    whole = _call(name, c, r)
    assert whole.shape == (6,) and torch.isfinite(whole).all()
    single = torch.stack([_call(name, c[i : i + 1], r[i : i + 1])[0] for i in range(6)])
    assert torch.allclose(whole, single, atol=1e-6), name           # no term couples the examples of a batch


@pytest.mark.parametrize("name", _PAIRWISE)
def test_head_prefers_chosen_over_rejected(name):
    """The gradient pushes the chosen log-ratio up or the rejected one down (both for most heads)."""
    c = torch.tensor([0.1, -0.4, 0.8], requires_grad=True)
    r = torch.tensor([0.3, 0.2, -0.5], requires_grad=True)
    _call(name, c, r).sum().backward()
    assert torch.isfinite(c.grad).all() and torch.isfinite(r.grad).all()
    assert (c.grad <= 1e-7).all() or (r.grad >= -1e-7).all(), (name, c.grad, r.grad)
    assert (c.grad.abs() + r.grad.abs() > 0).all()


@pytest.mark.parametrize("name", sorted(set(L.LOSS_HEADS)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_is_safe_at_extreme_log_ratios(name, dtype):
    c = torch.tensor([-80.0, 80.0, -80.0, 80.0, 0.0], dtype=dtype, requires_grad=True)
    r = torch.tensor([-80.0, -80.0, 80.0, 80.0, 0.0], dtype=dtype, requires_grad=True)
    if name == "orpo":
        c = torch.tensor([-80.0, -1e-4, -80.0, -1e-4, -1.0], dtype=dtype, requires_grad=True)
        r = torch.tensor([-80.0, -80.0, -1e-4, -1e-4, -1.0], dtype=dtype, requires_grad=True)
    out = _call(name, c, r)
    assert torch.isfinite(out.float()).all(), (name, out)
    out.float().sum().backward()
    assert all(t.grad is None or torch.isfinite(t.grad.float()).all() for t in (c, r)), name      # some heads ignore one side


def test_closed_forms_of_the_classic_heads():
    c, r, b = torch.tensor([0.3, -0.2]), torch.tensor([-0.1, 0.4]), 0.5
    z = b * (c - r)
    assert torch.allclose(L.sigmoid_loss(c, r, beta=b), -F.logsigmoid(z))
    assert torch.allclose(L.hinge_loss(c, r, beta=b), torch.relu(1 - z))
    assert torch.allclose(L.ipo_loss(c, r, beta=b), (c - r - 1 / (2 * b)) ** 2)
    assert torch.allclose(L.bco_loss(c, r, beta=b, delta=0.1), -F.logsigmoid(b * c - 0.1) - F.logsigmoid(-(b * r - 0.1)))
    assert torch.allclose(L.apo_down_loss(c, r, beta=b), torch.sigmoid(b * c) + 1 - torch.sigmoid(b * (c - r)))
    assert torch.allclose(L.simpo_loss(c, r, beta=2.0, gamma=0.5, label_smoothing=0.1),
                          -0.9 * F.logsigmoid(2 * (c - r) - 0.5) - 0.1 * F.logsigmoid(-(2 * (c - r) - 0.5)))
    assert torch.allclose(L.chosen_nll_loss(torch.tensor([-1.5, -0.2])), torch.tensor([1.5, 0.2]))


@pytest.mark.parametrize("kind", ["reverse_kl", "forward_kl", "js_divergence", "alpha_divergence"])
def test_f_divergence_remaps_are_monotone_and_reduce_to_the_identity_for_reverse_kl(kind):
    x = torch.linspace(-3, 3, 13)
    y = L.f_divergence_remap(x, f_divergence_type=kind, alpha=0.5)
    assert torch.isfinite(y).all() and (y[1:] >= y[:-1] - 1e-6).all()
    if kind == "reverse_kl":
        assert torch.equal(y, x)
    logits = L.f_divergence_logits(x, -x, f_divergence_type=kind, alpha=0.5)
    assert (logits[1:] >= logits[:-1] - 1e-6).all()


def test_weighting_helpers():
    # mixture of heads: a weighted sum, names must match
    c, r = torch.tensor([0.2, -0.1]), torch.tensor([0.0, 0.3])
    parts = {"sigmoid": L.sigmoid_loss(c, r, beta=0.3), "ipo": L.ipo_loss(c, r, beta=0.3)}
    assert torch.allclose(L.mpo_combine(parts, {"sigmoid": 0.8, "ipo": 0.2}), 0.8 * parts["sigmoid"] + 0.2 * parts["ipo"])
    assert torch.allclose(L.mpo_combine(parts, {"sigmoid": 1.0}), parts["sigmoid"])          # a subset of the terms
    from opake_b200.base.exceptions import ConfigurationError

    with pytest.raises(ConfigurationError):
        L.mpo_combine(parts, {"hinge": 1.0})
    with pytest.raises(ConfigurationError):
        L.mpo_combine(parts, {})
    # WPO weights: in (0, 1], one per sequence, larger for sequences the policy finds likely
    lp = torch.log(torch.tensor([[0.9, 0.8, 0.7], [0.2, 0.1, 0.3]]))
    w = L.wpo_weights(lp, torch.ones(2, 3))
    assert w.shape == (2,) and (w > 0).all() and (w <= 1.0 + 1e-6).all() and w[0] > w[1]
    # LD-DPO: alpha = 1 is the plain sum; alpha = 0 keeps only the shared-length prefix
    mask = torch.tensor([[1, 1, 1, 1], [1, 1, 0, 0]])
    full = L.ld_dpo_split(lp.new_ones(2, 4) * -0.5, mask, torch.tensor([2, 2]), 1.0)
    head = L.ld_dpo_split(lp.new_ones(2, 4) * -0.5, mask, torch.tensor([2, 2]), 0.0)
    assert torch.allclose(full, torch.tensor([-2.0, -1.0])) and torch.allclose(head, torch.tensor([-1.0, -1.0]))
