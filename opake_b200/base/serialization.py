"""Flat, path-keyed state dictionaries with template-driven restore.

The on-disk format is the reference's (packages/opake-base/src/opake/api/base/serialization/_dispatch.py:23-106,
_structural.py:37-114, _registry.py:27-81): ``state_dict(obj)`` is a flat ``dict[str, leaf]``; dataclass / NamedTuple
fields and mapping keys join with ``.``, sequence positions attach as ``[i]``; a type with a registered codec owns
everything below its path; restore walks a *template* object and keeps the template's value for anything the
dictionary does not mention. Leaves that no codec claims are an error, never a silent drop.

Implementation: one small :class:`_Codecs` table (exact type -> (save, load), resolved along the MRO) and a pair of
recursive visitors over "container kinds", each kind described by how to enumerate ``(child, relative-key)`` pairs
and how to rebuild from restored children.
"""
from __future__ import annotations

import dataclasses
from collections.abc import Callable, Iterable, Mapping
from typing import Any, Protocol, runtime_checkable

__all__ = ["FromStateDictFn", "SerializedState", "Serializer", "StateDictFn", "from_state_dict", "lookup_serializer",
           "register_serializer", "register_template_restored", "resolve_serializer", "state_dict"]

SerializedState = dict[str, Any]
StateDictFn = Callable[[Any], dict[str, Any]]
FromStateDictFn = Callable[[Any, Mapping[str, Any]], Any]


@runtime_checkable
class Serializer(Protocol):
    def state_dict(self, obj: Any) -> dict[str, Any]: ...

    def from_state_dict(self, template: Any, sd: Mapping[str, Any]) -> Any: ...


class _Codecs:
    def __init__(self) -> None:
        self._by_type: dict[type, tuple[StateDictFn, FromStateDictFn]] = {}

    def add(self, typ: type, save: StateDictFn, load: FromStateDictFn) -> None:
        self._by_type[typ] = (save, load)

    def exact(self, typ: type):
        return self._by_type.get(typ)

    def nearest(self, typ: type):
        for klass in typ.__mro__:
            hit = self._by_type.get(klass)
            if hit is not None:
                return hit
        return None


_CODECS = _Codecs()
_SCALARS = (int, float, bool, str, type(None))


def register_serializer(typ: type, state_dict_fn: StateDictFn, from_state_dict_fn: FromStateDictFn) -> None:
    """Install (or replace) the codec of ``typ``; subclasses without their own codec inherit it."""
    _CODECS.add(typ, state_dict_fn, from_state_dict_fn)


def register_template_restored(typ: type) -> None:
    """Mark ``typ`` as carrying no run state: nothing is written, restore returns the template's object."""
    _CODECS.add(typ, lambda _obj: {}, lambda template, _sd: template)


def lookup_serializer(typ: type):
    return _CODECS.exact(typ)


def resolve_serializer(typ: type):
    return _CODECS.nearest(typ)


# ----------------------------------------------------------------------------------------------- paths
def _child_path(parent: str, rel: str) -> str:
    if not parent:
        return rel
    if not rel:
        return parent
    return parent + rel if rel.startswith("[") else f"{parent}.{rel}"


def _slice_below(sd: Mapping[str, Any], prefix: str) -> dict[str, Any]:
    """Entries of ``sd`` located at or below ``prefix``, re-keyed relative to it."""
    if not prefix:
        return dict(sd)
    n = len(prefix)
    out: dict[str, Any] = {}
    for k, v in sd.items():
        if not k.startswith(prefix):
            continue
        if len(k) == n:
            out[""] = v
        elif k[n] == ".":
            out[k[n + 1:]] = v
        elif k[n] == "[":
            out[k[n:]] = v
    return out


# ----------------------------------------------------------------------------------------------- container kinds
def _is_namedtuple(o: Any) -> bool:
    return isinstance(o, tuple) and hasattr(o, "_fields")


def _children(o: Any) -> Iterable[tuple[str, Any]] | None:
    """``(relative key, child)`` pairs of a generic container, or ``None`` when ``o`` is not one."""
    if dataclasses.is_dataclass(o) and not isinstance(o, type):
        return [(f.name, getattr(o, f.name)) for f in dataclasses.fields(o)]
    if _is_namedtuple(o):
        return [(f, getattr(o, f)) for f in o._fields]
    if isinstance(o, (tuple, list)):
        return [(f"[{i}]", v) for i, v in enumerate(o)]
    if isinstance(o, Mapping):
        return [(str(k), v) for k, v in o.items()]
    return None


def _rebuild(template: Any, restored: list[Any]) -> Any:
    if dataclasses.is_dataclass(template) and not isinstance(template, type):
        names = [f.name for f in dataclasses.fields(template)]
        return dataclasses.replace(template, **dict(zip(names, restored)))
    if _is_namedtuple(template):
        return type(template)(*restored)
    if isinstance(template, tuple):
        return type(template)(restored) if type(template) is not tuple else tuple(restored)
    if isinstance(template, list):
        return list(restored)
    return dict(zip(template.keys(), restored))


def _no_codec(o: Any, path: str, verb: str) -> TypeError:
    where = f"at {path!r}" if path else "at the root"
    return TypeError(
        f"Cannot {verb} {type(o).__module__}.{type(o).__qualname__} {where}: it is not a registered type, not a generic "
        "container (dataclass / NamedTuple / tuple / list / mapping) and not a primitive. Register a handler with "
        "`register_serializer`, or declare the type inert with `register_template_restored`.")


def _save(o: Any, path: str, out: dict[str, Any]) -> None:
    codec = _CODECS.nearest(type(o))
    if codec is not None:
        for rel, leaf in codec[0](o).items():
            out[_child_path(path, rel)] = leaf
        return
    kids = _children(o)
    if kids is not None:
        for rel, child in kids:
            _save(child, _child_path(path, rel), out)
        return
    if isinstance(o, _SCALARS):
        out[path] = o
        return
    raise _no_codec(o, path, "serialize")


def _load(template: Any, sd: Mapping[str, Any], path: str) -> Any:
    codec = _CODECS.nearest(type(template))
    if codec is not None:
        try:
            return codec[1](template, _slice_below(sd, path))
        except Exception as exc:
            exc.add_note(f"while restoring {path!r}" if path else "while restoring the root")
            raise
    kids = _children(template)
    if kids is not None:
        return _rebuild(template, [_load(child, sd, _child_path(path, rel)) for rel, child in kids])
    if isinstance(template, _SCALARS):
        return sd.get(path, template)
    raise _no_codec(template, path, "restore")


def state_dict(obj: Any) -> dict[str, Any]:
    """Flatten ``obj`` into ``{path: leaf}``."""
    out: dict[str, Any] = {}
    _save(obj, "", out)
    return out


def from_state_dict(template: Any, sd: Mapping[str, Any]) -> Any:
    """Rebuild an object shaped like ``template`` from ``sd``; leaves missing from ``sd`` keep the template's value."""
    return _load(template, sd, "")
