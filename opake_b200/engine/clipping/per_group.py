"""Build a :class:`PerGroup` of per-parameter-group values (clipping norms) from substring patterns.

Rules as in packages/opake-engine/src/opake/api/engine/clipping/_per_group.py:44-186: a pattern matches when it is a
substring of the leaf's dotted path; every leaf must match exactly one pattern (or fall into ``fallback``); unused
patterns are an error unless allowed; values must be positive.
"""
from __future__ import annotations

import torch

from ...base.exceptions import ConfigurationError, InputTypeError
from ..pytree import param_path_display, tree_flatten_with_paths
from ..types import PerGroup


def per_group(params, patterns: dict | None = None, *, fallback: float | None = None,
              allow_unused_patterns: bool = False, **kwargs) -> PerGroup:
    table: dict[str, float] = dict(patterns or {})
    table.update(kwargs)
    if not table and fallback is None:
        raise ConfigurationError("At least one pattern must be provided.")
    for pat, val in table.items():
        if val <= 0:
            raise ConfigurationError(f"Per-group value must be positive, got {val} for pattern '{pat}'.")
    if fallback is not None and fallback <= 0:
        raise ConfigurationError(f"Fallback value must be positive, got {fallback}.")
    paths, leaves, _ = tree_flatten_with_paths(params)
    for p, l in zip(paths, leaves):
        if not isinstance(l, torch.Tensor):
            raise InputTypeError(f"per_group expects tensor leaves; {param_path_display(p)!r} is {type(l).__name__}")
    groups, hit = {}, set()
    for path in paths:
        shown = param_path_display(path)
        found = [pat for pat in table if pat in shown]
        if not found:
            if fallback is None:
                raise ConfigurationError(f"Parameter path {path!r} (display {shown!r}) did not match any pattern. "
                                         f"Available patterns: {list(table)}. Use fallback=<value> to catch unmatched "
                                         "parameters.")
            groups[path] = "fallback"
        elif len(found) > 1:
            raise ConfigurationError(f"Parameter path {path!r} (display {shown!r}) matched multiple patterns: {found}. "
                                     "Each parameter must match exactly one pattern.")
        else:
            groups[path] = found[0]
            hit.add(found[0])
    unused = [p for p in table if p not in hit]
    if unused and not allow_unused_patterns:
        raise ConfigurationError(f"Patterns did not match any parameter: {unused}. Sample parameter paths: "
                                 f"{[param_path_display(p) for p in paths[:3]]}. Use allow_unused_patterns=True when "
                                 "intentionally sharing patterns across architectures.")
    used = set(groups.values())
    values = {p: float(v) for p, v in table.items() if p in used}
    if fallback is not None and "fallback" in used:
        values["fallback"] = float(fallback)
    return PerGroup(groups=groups, values=values)


__all__ = ["per_group"]
