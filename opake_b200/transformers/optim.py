"""Optimizer factory for the trainer: Hugging Face style names and aliases to the DP-aware optimizers
(packages/opake-transformers/src/opake/api/transformers/trainer/_optim.py:44-100,224-244). ``"adamw-bc"`` is AdamW
with the DP noise bias correction of the second moment."""
from __future__ import annotations

from typing import Any, Callable

from .. import optimizers as O
from ..base.exceptions import ConfigurationError

__all__ = ["build_optimizer", "OPTIMIZER_ALIASES", "canonical_optimizer_name"]

OPTIMIZER_ALIASES = {
    "adamw": "adamw", "adamw_torch": "adamw", "adamw_torch_fused": "adamw", "adamw_hf": "adamw", "adamw-bc": "adamw-bc",
    "adamw_bc": "adamw-bc", "adam-bc": "adam-bc", "adam_bc": "adam-bc", "adam": "adam", "sgd": "sgd", "adagrad": "adagrad",
    "adadelta": "adadelta", "adafactor": "adafactor", "ademamix": "ademamix", "lion": "lion", "lion_32bit": "lion",
    "radam": "radam", "rmsprop": "rmsprop", "schedule_free": "schedule_free", "schedule_free_adamw": "schedule_free",
    "schedule_free_sgd": "schedule_free_sgd",
}


def canonical_optimizer_name(name: str) -> str:
    key = str(name).lower()
    if key not in OPTIMIZER_ALIASES:
        raise ConfigurationError(f"unknown optimizer {name!r}; known: {sorted(set(OPTIMIZER_ALIASES.values()))}")
    return OPTIMIZER_ALIASES[key]


def build_optimizer(name: str, *, lr: float | Callable[[int], float], weight_decay: float = 0.0,
                    betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, optim_args: dict | None = None):
    """Returns a ``GradientTransformation`` (``init`` / ``update``); ``lr`` may be a schedule callable."""
    kind = canonical_optimizer_name(name)
    kw: dict[str, Any] = {}
    for k, v in (optim_args or {}).items():
        try:
            kw[k] = float(v) if isinstance(v, str) and v.replace(".", "", 1).replace("e-", "", 1).replace("-", "", 1).isdigit() else v
        except ValueError:
            kw[k] = v
    if kind in ("adamw", "adamw-bc"):
        return O.adamw(lr, betas=betas, eps=eps, weight_decay=weight_decay, noise_bias_correction=(kind == "adamw-bc"), **kw)
    if kind in ("adam", "adam-bc"):
        return O.adam(lr, betas=betas, eps=eps, weight_decay=weight_decay, noise_bias_correction=(kind == "adam-bc"), **kw)
    if kind == "sgd":
        return O.sgd(lr, weight_decay=weight_decay, **kw)
    if kind == "adagrad":
        return O.adagrad(lr, weight_decay=weight_decay, **kw)
    if kind == "adadelta":
        return O.adadelta(lr, weight_decay=weight_decay, **kw)
    if kind == "adafactor":
        return O.adafactor(lr, weight_decay=weight_decay, **kw)
    if kind == "ademamix":
        return O.ademamix(lr, betas=(betas[0], betas[1], float(kw.pop("beta3", 0.9999))), eps=eps, weight_decay=weight_decay, **kw)
    if kind == "lion":
        return O.lion(lr, betas=(betas[0], float(kw.pop("beta2", 0.99))), weight_decay=weight_decay, **kw)
    if kind == "radam":
        return O.radam(lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
    if kind == "rmsprop":
        return O.rmsprop(lr, eps=eps, weight_decay=weight_decay, **kw)
    if kind == "schedule_free":
        return O.schedule_free(lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
    if kind == "schedule_free_sgd":
        return O.schedule_free(lr, betas=betas, eps=eps, weight_decay=weight_decay, adam=False, **kw)
    raise ConfigurationError(f"unknown optimizer {name!r}")
