"""Leaf codecs for tensors and arrays (registered on import of :mod:`opake_b200.engine`).

Format of packages/opake-engine/src/opake/api/engine/serialization/_structural.py:44-111: a tensor leaf occupies its
own path (relative key ``""``), restore checks the shape against the template and casts to the template's dtype and
device; tree-structure handles are template-restored.
"""
from __future__ import annotations

from collections.abc import Mapping
from typing import Any

import numpy as np
import torch

from ..base.exceptions import CheckpointError
from ..base.serialization import register_serializer, register_template_restored
from .pytree import TreeDef
from .random import RngKey


def _same_shape(saved, expected) -> None:
    if tuple(saved) != tuple(expected):
        raise CheckpointError(f"state_dict value has shape {tuple(saved)}; template expects {tuple(expected)}. Restore is "
                              "template-driven: rebuild the template from the configuration the checkpoint was written "
                              "with.")


def _save_tensor(t: torch.Tensor) -> dict[str, Any]:
    return {"": t.detach().clone()}


def _load_tensor(template: torch.Tensor, sd: Mapping[str, Any]) -> torch.Tensor:
    v = sd.get("")
    if v is None:
        return template
    if not isinstance(v, torch.Tensor):
        raise CheckpointError(f"state_dict value expected a torch.Tensor, got {type(v).__name__}")
    _same_shape(v.shape, template.shape)
    return v.to(dtype=template.dtype, device=template.device)


def _load_parameter(template: torch.nn.Parameter, sd: Mapping[str, Any]):
    v = _load_tensor(template, sd)
    return template if v is template else torch.nn.Parameter(v.detach(), requires_grad=template.requires_grad)


def _save_array(a: np.ndarray) -> dict[str, Any]:
    return {"": a.copy()}


def _load_array(template: np.ndarray, sd: Mapping[str, Any]) -> np.ndarray:
    v = sd.get("")
    if v is None:
        return template
    arr = np.asarray(v)
    _same_shape(arr.shape, template.shape)
    return arr.astype(template.dtype, copy=True)


register_serializer(torch.Tensor, _save_tensor, _load_tensor)
register_serializer(torch.nn.Parameter, _save_tensor, _load_parameter)
register_serializer(np.ndarray, _save_array, _load_array)
register_template_restored(TreeDef)
register_template_restored(torch.dtype)
register_template_restored(torch.device)
