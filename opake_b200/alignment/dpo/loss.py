"""Preference-optimisation loss heads (packages/opake-alignment/src/opake/api/alignment/dpo/loss/_*.py; the sigmoid
head is _sigmoid.py:22-53). Every head is an elementwise function of per-example log-ratios
``log pi(y|x) - log pi_ref(y|x)`` (or plain log-probabilities for the reference-free ones) and returns one loss per
example, so DP per-example clipping applies directly."""
from __future__ import annotations

import math
from typing import Literal

import torch
import torch.nn.functional as F

from ...base.exceptions import ConfigurationError
from ..logprob import _compute_dtype

from ..logprob import fused_sequence_logp, sequence_logp  # noqa: E402,F401  (same names as the reference's dpo.loss)

__all__ = [
    "sequence_logp", "fused_sequence_logp",
    "sigmoid_loss", "hinge_loss", "robust_loss", "ipo_loss", "discopop_loss", "chosen_nll_loss", "apo_zero_loss",
    "apo_down_loss", "exo_loss", "nca_loss", "bco_loss", "sppo_loss", "simpo_loss", "odds_ratio_loss",
    "f_divergence_remap", "f_divergence_logits", "mpo_combine", "wpo_weights", "ld_dpo_split", "LOSS_HEADS",
]

FDivergence = Literal["reverse_kl", "forward_kl", "js_divergence", "alpha_divergence"]


def _exp_cap(dtype: torch.dtype) -> float:
    return 11.0 if dtype == torch.float16 else 80.0


def sigmoid_loss(chosen_logratio, rejected_logratio, *, beta: float, label_smoothing: float = 0.0):
    z = beta * (chosen_logratio - rejected_logratio)
    return -F.logsigmoid(z) * (1 - label_smoothing) - F.logsigmoid(-z) * label_smoothing


def hinge_loss(chosen_logratio, rejected_logratio, *, beta: float):
    return torch.relu(1 - beta * (chosen_logratio - rejected_logratio))


def robust_loss(chosen_logratio, rejected_logratio, *, beta: float, label_smoothing: float = 0.0):
    z = beta * (chosen_logratio - rejected_logratio)
    return (-F.logsigmoid(z) * (1 - label_smoothing) + F.logsigmoid(-z) * label_smoothing) / (1 - 2 * label_smoothing)


def ipo_loss(chosen_logratio, rejected_logratio, *, beta: float):
    return (chosen_logratio - rejected_logratio - 1.0 / (2.0 * beta)).pow(2)


def discopop_loss(chosen_logratio, rejected_logratio, *, beta: float, discopop_tau: float = 0.05):
    z = (chosen_logratio - rejected_logratio) * beta
    gate = torch.sigmoid(z / discopop_tau)
    expo = torch.exp(-z.clamp(min=-_exp_cap(z.dtype)))     # the clamp keeps exp finite in the compute dtype
    return -F.logsigmoid(z) * (1.0 - gate) + expo * gate


def chosen_nll_loss(chosen_logp, /, *_args, **_kwargs):
    """SFT regulariser for blends: minus the chosen log-probability; other arguments are accepted and ignored."""
    return -chosen_logp


def apo_zero_loss(chosen_logratio, rejected_logratio, *, beta: float):
    return (1 - torch.sigmoid(beta * chosen_logratio)) + torch.sigmoid(beta * rejected_logratio)


def apo_down_loss(chosen_logratio, rejected_logratio, *, beta: float):
    return torch.sigmoid(beta * chosen_logratio) + (1 - torch.sigmoid(beta * (chosen_logratio - rejected_logratio)))


def exo_loss(chosen_logratio, rejected_logratio, *, beta: float, label_smoothing: float = 1e-3):
    eps = label_smoothing if label_smoothing > 0 else 1e-3
    z = beta * (chosen_logratio - rejected_logratio)
    return (torch.sigmoid(z) * (F.logsigmoid(z) - math.log(1 - eps))
            + torch.sigmoid(-z) * (F.logsigmoid(-z) - math.log(eps)))


def nca_loss(chosen_logratio, rejected_logratio, *, beta: float):
    c, r = beta * chosen_logratio, beta * rejected_logratio
    return -F.logsigmoid(c) - 0.5 * F.logsigmoid(-c) - 0.5 * F.logsigmoid(-r)


def bco_loss(chosen_logratio, rejected_logratio, *, beta: float, delta: float = 0.0):
    """``delta`` is a reward baseline that must be public or itself differentially private."""
    return -F.logsigmoid(beta * chosen_logratio - delta) - F.logsigmoid(-(beta * rejected_logratio - delta))


def sppo_loss(chosen_logratio, rejected_logratio, *, beta: float):
    t = 0.5 / beta
    return (chosen_logratio - t).pow(2) + (rejected_logratio + t).pow(2)


def simpo_loss(chosen_logratio, rejected_logratio, *, beta: float, gamma: float = 0.0, label_smoothing: float = 0.0):
    m = beta * (chosen_logratio - rejected_logratio) - gamma
    return -F.logsigmoid(m) * (1.0 - label_smoothing) - F.logsigmoid(-m) * label_smoothing


def _log1mexp(x):
    """``log(1 - exp(x))`` for ``x < 0`` (Maechler 2012). Each branch only ever sees arguments from its own side of the
    split: otherwise the unused branch can be infinite there (``exp(x)`` rounds to 1 in bf16 for small ``|x|``) and its
    zero-weighted gradient turns into NaN."""
    near = x > -math.log(2.0)
    a = torch.where(near, x, torch.full_like(x, -1.0))
    b = torch.where(near, torch.full_like(x, -1.0), x)
    return torch.where(near, torch.log(-torch.expm1(a)), torch.log1p(-torch.exp(b)))


def odds_ratio_loss(chosen_logp, rejected_logp):
    """ORPO: ``-log sigmoid(log odds(y_w) - log odds(y_l))`` of length-normalised log-probabilities (< 0)."""
    return -F.logsigmoid((chosen_logp - _log1mexp(chosen_logp)) - (rejected_logp - _log1mexp(rejected_logp)))


def f_divergence_remap(logratio, *, f_divergence_type: FDivergence = "reverse_kl", alpha: float = 1.0):
    if f_divergence_type == "reverse_kl":
        return logratio
    cap = _exp_cap(logratio.dtype)
    if f_divergence_type == "forward_kl":
        return 1 - torch.exp(torch.clamp(-logratio, max=cap))
    if f_divergence_type == "js_divergence":
        return math.log(2.0) + F.logsigmoid(logratio)
    if f_divergence_type == "alpha_divergence":
        if abs(alpha - 1.0) < 1e-6:
            return logratio
        return (torch.exp(torch.clamp((alpha - 1) * logratio, max=cap)) - 1) / (alpha - 1)
    raise ConfigurationError(f"Unknown f_divergence_type {f_divergence_type!r}; expected one of 'reverse_kl', "
                             "'forward_kl', 'js_divergence', 'alpha_divergence'.")


def f_divergence_logits(chosen_logratio, rejected_logratio, *, f_divergence_type: FDivergence = "reverse_kl",
                        alpha: float = 1.0):
    return (f_divergence_remap(chosen_logratio, f_divergence_type=f_divergence_type, alpha=alpha)
            - f_divergence_remap(rejected_logratio, f_divergence_type=f_divergence_type, alpha=alpha))


def mpo_combine(losses: dict, weights: dict):
    """Weighted blend of already-computed per-example losses (mixed preference optimisation)."""
    missing = weights.keys() - losses.keys()
    if missing:
        raise ConfigurationError(f"weights keys {sorted(missing)} are not present in losses (available: {sorted(losses)})")
    out = None
    for name, wgt in weights.items():
        term = wgt * losses[name]
        out = term if out is None else out + term
    if out is None:
        raise ConfigurationError("weights must select at least one loss term")
    return out


def wpo_weights(per_token_logps, completion_mask, logits=None):
    """WPO importance weight ``exp(mean_t log p_t)`` (detached); with ``logits`` each token is first normalised by
    ``log sum_v p_v^2``."""
    acc = _compute_dtype(per_token_logps)
    if logits is not None:
        acc = torch.promote_types(acc, _compute_dtype(logits))
    mask = completion_mask.to(torch.bool)
    n = mask.sum(dim=-1).clamp(min=1)
    with torch.no_grad():
        lp = per_token_logps.to(acc)
        if logits is not None:
            lg = logits.to(acc)
            lp = lp - (torch.logsumexp(2.0 * lg, dim=-1) - 2.0 * torch.logsumexp(lg, dim=-1))
        return (torch.where(mask, lp, 0.0).sum(dim=-1) / n.to(acc)).exp()


def ld_dpo_split(per_token_logps, completion_mask, shared_prefix_len, alpha: float):
    """LD-DPO: completion tokens beyond the length both responses share are down-weighted by ``alpha``."""
    if not math.isfinite(alpha) or not 0.0 <= alpha <= 1.0:
        raise ConfigurationError(f"alpha (LD-DPO) must be finite and in [0, 1], got {alpha}")
    from ..logprob import _ld_weight
    w = _ld_weight(completion_mask != 0, shared_prefix_len, alpha, per_token_logps.dtype, per_token_logps.device)
    return (per_token_logps * completion_mask.to(per_token_logps.dtype) * w).sum(dim=-1)


# name -> head, for trainers that select the head from a config string
LOSS_HEADS = {
    "sigmoid": sigmoid_loss, "hinge": hinge_loss, "robust": robust_loss, "ipo": ipo_loss, "discopop": discopop_loss,
    "sft": chosen_nll_loss, "chosen_nll": chosen_nll_loss, "apo_zero": apo_zero_loss, "apo_down": apo_down_loss,
    "exo_pair": exo_loss, "exo": exo_loss, "nca_pair": nca_loss, "nca": nca_loss, "bco_pair": bco_loss, "bco": bco_loss,
    "sppo_hard": sppo_loss, "sppo": sppo_loss, "simpo": simpo_loss, "orpo": odds_ratio_loss,
}
