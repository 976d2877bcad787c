"""JSON-able nested ``{"type": ClassName, field: ...}`` codec of processes and the ``Accountant`` state
(format of packages/opake-accounting/src/opake/api/accounting/core/_process_codec.py:28-170 and
_accountant.py:230-263; this is what ``accountant.json`` in a checkpoint contains). Composition spines are walked
iteratively so thousands of composed steps do not hit the recursion limit.
"""
from __future__ import annotations

import dataclasses
from typing import Any

from ..base.exceptions import CheckpointError
from ..base.serialization import lookup_serializer, register_serializer
from ..base.serialization import state_dict as _state_dict
from .core import _PROCESS_REGISTRY, CachedProcess, Composed, DpProcess, Repeated

_PRIMS = (int, float, bool, str, type(None))
_WRAPPERS = {"Composed": ("left", "right"), "Repeated": ("inner",), "CachedProcess": ("inner",)}


def process_to_dict(p: DpProcess) -> dict[str, Any]:
    root: dict[str, Any] = {}
    stack = [(p, root)]
    while stack:
        node, out = stack.pop()
        custom = lookup_serializer(type(node))
        if custom is not None and custom[0] is not _generic_save:
            out.update(custom[0](node))      # classes with their own codec (e.g. strategy-carrying mechanisms)
            out.setdefault("type", type(node).__name__)
            continue
        out["type"] = type(node).__name__
        for f in dataclasses.fields(node):
            v = getattr(node, f.name)
            if type(v) in (Composed, Repeated, CachedProcess):
                slot: dict[str, Any] = {}
                out[f.name] = slot
                stack.append((v, slot))
            elif isinstance(v, DpProcess):
                out[f.name] = dict(_state_dict(v))
            elif isinstance(v, (*_PRIMS, tuple, list)):
                out[f.name] = list(v) if isinstance(v, tuple) else v
    return root


def _leaf(node: dict[str, Any]) -> DpProcess:
    name = node.get("type")
    cls = _PROCESS_REGISTRY.get(name)
    if cls is None:
        # mechanism classes register themselves when their module is imported: a process file may be read before
        # the DP-SGD / DP-FTRL accounting modules were touched
        import importlib

        for mod in ("opake_b200.dpsgd.accounting", "opake_b200.dpftrl.accounting"):
            importlib.import_module(mod)
        cls = _PROCESS_REGISTRY.get(name)
    if cls is None:
        raise CheckpointError(f"unknown DpProcess type {name!r}")
    pair = lookup_serializer(cls)
    if pair is not None and pair[1] is not _generic_load:
        return pair[1](cls.__new__(cls), dict(node))
    kwargs = {}
    for f in dataclasses.fields(cls):
        if f.name in node:
            raw = node[f.name]
            if isinstance(raw, dict) and "type" in raw:
                raw = process_from_dict(raw)
            elif isinstance(raw, list):
                raw = tuple(raw)
            kwargs[f.name] = raw
        elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING:
            raise CheckpointError(f"missing required field {f.name!r} for {cls.__name__}")
    extra = set(node) - {"type"} - {f.name for f in dataclasses.fields(cls)}
    if extra:
        raise CheckpointError(f"unexpected keys for {cls.__name__}: {sorted(extra)!r}")
    return cls(**kwargs)


def process_from_dict(sd: dict[str, Any]) -> DpProcess:
    built: dict[int, DpProcess] = {}
    stack: list[tuple[dict, bool]] = [(sd, False)]
    while stack:
        node, expanded = stack.pop()
        t = node.get("type")
        if t is None:
            raise CheckpointError("missing required field 'type' for serialized DpProcess")
        kids = _WRAPPERS.get(t)
        if kids is None:
            built[id(node)] = _leaf(node)
            continue
        if not expanded:
            stack.append((node, True))
            for k in kids:
                child = node.get(k)
                if not isinstance(child, dict):
                    raise CheckpointError(f"field {k!r} of {t} must be a serialized DpProcess dict, got {type(child).__name__}")
                stack.append((child, False))
            continue
        cls = _PROCESS_REGISTRY[t]
        kwargs = {}
        for f in dataclasses.fields(cls):
            if f.name in kids:
                kwargs[f.name] = built[id(node[f.name])]
            elif f.name in node:
                kwargs[f.name] = node[f.name]
        built[id(node)] = cls(**kwargs)
    return built[id(sd)]


def _generic_save(p):
    return process_to_dict(p)


def _generic_load(_template, sd):
    return process_from_dict(dict(sd))


register_serializer(DpProcess, _generic_save, _generic_load)

__all__ = ["process_to_dict", "process_from_dict"]
