"""PEFT / LoRA support (packages/opake-patches/src/opake/api/patches/peft/_router.py:151). LoRA ``Linear`` layers
(anything exposing ``base_layer``, ``lora_A``, ``lora_B``, ``scaling``) get a forward that calls the fused LoRA
function with its explicit, vmap-aware backward; adapters with dropout keep the stock forward."""
from __future__ import annotations

import types

import torch

from .kernels.lora import lora_linear

__all__ = ["apply_peft_model_patches", "is_lora_layer", "LoRALinear", "inject_lora"]


def is_lora_layer(m) -> bool:
    return all(hasattr(m, a) for a in ("base_layer", "lora_A", "lora_B", "scaling"))


def _lora_forward(self, x, *args, **kwargs):
    names = getattr(self, "active_adapters", None) or list(self.lora_A.keys())
    names = [names] if isinstance(names, str) else list(names)
    if getattr(self, "disable_adapters", False) or getattr(self, "merged", False) or len(names) != 1:
        return self._opake_stock_forward(x, *args, **kwargs)
    name = names[0]
    drop = self.lora_dropout[name] if hasattr(self, "lora_dropout") and name in self.lora_dropout else None
    if isinstance(drop, torch.nn.Dropout) and drop.p > 0 and self.training:
        return self._opake_stock_forward(x, *args, **kwargs)
    base = self.base_layer
    return lora_linear(x, base.weight, self.lora_A[name].weight, self.lora_B[name].weight, float(self.scaling[name]),
                       getattr(base, "bias", None))


def apply_peft_model_patches(model) -> int:
    """Returns the number of LoRA layers switched to the fused forward."""
    n = 0
    for m in model.modules():
        if is_lora_layer(m) and isinstance(getattr(m, "base_layer", None), torch.nn.Linear) and not hasattr(m, "_opake_stock_forward"):
            m._opake_stock_forward = m.forward
            m.forward = types.MethodType(_lora_forward, m)
            n += 1
    return n


class LoRALinear(torch.nn.Module):
    """Minimal LoRA wrapper with the attribute layout of PEFT, for use without the ``peft`` package."""

    def __init__(self, base: torch.nn.Linear, r: int = 8, alpha: float = 16.0, name: str = "default"):
        super().__init__()
        self.base_layer = base
        for p in base.parameters():
            p.requires_grad_(False)
        self.lora_A = torch.nn.ModuleDict({name: torch.nn.Linear(base.in_features, r, bias=False, dtype=base.weight.dtype, device=base.weight.device)})
        self.lora_B = torch.nn.ModuleDict({name: torch.nn.Linear(r, base.out_features, bias=False, dtype=base.weight.dtype, device=base.weight.device)})
        torch.nn.init.zeros_(self.lora_B[name].weight)
        self.scaling = {name: alpha / r}
        self.active_adapters = [name]
        self.disable_adapters = False
        self.merged = False

    def forward(self, x):
        name = self.active_adapters[0]
        if self.disable_adapters:
            return self.base_layer(x)
        return lora_linear(x, self.base_layer.weight, self.lora_A[name].weight, self.lora_B[name].weight, self.scaling[name],
                           self.base_layer.bias)


def inject_lora(model, target_suffixes=("q_proj", "k_proj", "v_proj", "o_proj"), r: int = 8, alpha: float = 16.0) -> int:
    """Wraps every ``nn.Linear`` whose name ends with one of ``target_suffixes`` in ``LoRALinear`` and freezes the
    rest of the model. Returns the number of wrapped layers."""
    for p in model.parameters():
        p.requires_grad_(False)
    n = 0
    for parent in list(model.modules()):
        for child_name, child in list(parent.named_children()):
            if isinstance(child, torch.nn.Linear) and child_name.endswith(tuple(target_suffixes)):
                setattr(parent, child_name, LoRALinear(child, r, alpha))
                n += 1
    return n
