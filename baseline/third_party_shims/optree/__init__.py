"""Minimal stand-in for the ``optree`` package (flatten / unflatten of nested Python containers).

Semantics follow optree's documented defaults: ``dict`` children are visited in sorted key order (insertion order when
the keys cannot be sorted), ``OrderedDict`` in insertion order, ``None`` is an internal node without children
(``none_is_leaf=False``), tuples / lists / deques / named tuples are sequences, everything else is a leaf.
"""
from __future__ import annotations

from collections import OrderedDict, defaultdict, deque
from typing import Any, Callable, Iterable

__version__ = "0.17.0+standin"


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields")


def _sorted_keys(d: dict) -> list:
    try:
        return sorted(d)
    except TypeError:
        return list(d)


class PyTreeSpec:
    """Structure of a pytree without its leaves."""

    __slots__ = ("kind", "meta", "children", "num_leaves", "none_is_leaf")

    def __init__(self, kind: str, meta: Any, children: tuple, none_is_leaf: bool = False):
        self.kind, self.meta, self.children, self.none_is_leaf = kind, meta, tuple(children), none_is_leaf
        self.num_leaves = 1 if kind == "leaf" else sum(c.num_leaves for c in self.children)

    @property
    def num_children(self) -> int:
        return len(self.children)

    @property
    def num_nodes(self) -> int:
        return 1 + sum(c.num_nodes for c in self.children)

    def is_leaf(self) -> bool:
        return self.kind == "leaf"

    def _key(self):
        meta = self.meta
        if self.kind in ("dict", "ordereddict", "defaultdict"):
            meta = tuple(meta) if self.kind != "defaultdict" else (meta[0], tuple(meta[1]))
        return (self.kind, meta, self.children)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, PyTreeSpec) and self._key() == other._key()

    def __ne__(self, other: object) -> bool:
        return not self == other

    def __hash__(self) -> int:
        try:
            return hash(self._key())
        except TypeError:
            return hash((self.kind, self.num_leaves))

    def unflatten(self, leaves: Iterable[Any]) -> Any:
        it = iter(leaves)
        out = self._build(it)
        for _ in it:
            raise ValueError("too many leaves for this PyTreeSpec")
        return out

    def _build(self, it) -> Any:
        k = self.kind
        if k == "leaf":
            try:
                return next(it)
            except StopIteration:
                raise ValueError("too few leaves for this PyTreeSpec") from None
        kids = [c._build(it) for c in self.children]
        if k == "none":
            return None
        if k == "tuple":
            return tuple(kids)
        if k == "list":
            return kids
        if k == "deque":
            return deque(kids, maxlen=self.meta)
        if k == "namedtuple":
            return self.meta(*kids)
        if k == "dict":
            return dict(zip(self.meta, kids))
        if k == "ordereddict":
            return OrderedDict(zip(self.meta, kids))
        if k == "defaultdict":
            return defaultdict(self.meta[0], zip(self.meta[1], kids))
        raise ValueError(f"unknown node kind {k!r}")

    def entries(self) -> list:
        if self.kind in ("dict", "ordereddict"):
            return list(self.meta)
        if self.kind == "defaultdict":
            return list(self.meta[1])
        return list(range(len(self.children)))

    def paths(self) -> list[tuple]:
        out: list[tuple] = []
        self._paths((), out)
        return out

    def _paths(self, prefix: tuple, out: list) -> None:
        if self.kind == "leaf":
            out.append(prefix)
            return
        for e, c in zip(self.entries(), self.children):
            c._paths(prefix + (e,), out)

    def __repr__(self) -> str:
        return f"PyTreeSpec({self._repr()})"

    def _repr(self) -> str:
        k = self.kind
        if k == "leaf":
            return "*"
        if k == "none":
            return "None"
        kids = [c._repr() for c in self.children]
        if k in ("dict", "ordereddict", "defaultdict"):
            keys = self.entries()
            return "{" + ", ".join(f"{a!r}: {b}" for a, b in zip(keys, kids)) + "}"
        if k == "list":
            return "[" + ", ".join(kids) + "]"
        return "(" + ", ".join(kids) + ("," if len(kids) == 1 else "") + ")"


def _flatten(tree: Any, leaves: list, is_leaf: Callable | None, none_is_leaf: bool) -> PyTreeSpec:
    if is_leaf is not None and is_leaf(tree):
        leaves.append(tree)
        return PyTreeSpec("leaf", None, ())
    if tree is None:
        if none_is_leaf:
            leaves.append(tree)
            return PyTreeSpec("leaf", None, ())
        return PyTreeSpec("none", None, ())
    rec = lambda x: _flatten(x, leaves, is_leaf, none_is_leaf)  # noqa: E731
    if _is_namedtuple(tree):
        return PyTreeSpec("namedtuple", type(tree), [rec(c) for c in tree])
    t = type(tree)
    if t is tuple:
        return PyTreeSpec("tuple", None, [rec(c) for c in tree])
    if t is list:
        return PyTreeSpec("list", None, [rec(c) for c in tree])
    if t is deque:
        return PyTreeSpec("deque", tree.maxlen, [rec(c) for c in tree])
    if t is OrderedDict:
        keys = list(tree)
        return PyTreeSpec("ordereddict", tuple(keys), [rec(tree[k]) for k in keys])
    if t is defaultdict:
        keys = _sorted_keys(tree)
        return PyTreeSpec("defaultdict", (tree.default_factory, tuple(keys)), [rec(tree[k]) for k in keys])
    if t is dict:
        keys = _sorted_keys(tree)
        return PyTreeSpec("dict", tuple(keys), [rec(tree[k]) for k in keys])
    leaves.append(tree)
    return PyTreeSpec("leaf", None, ())


def tree_flatten(tree: Any, is_leaf: Callable | None = None, *, none_is_leaf: bool = False, namespace: str = ""):
    leaves: list = []
    spec = _flatten(tree, leaves, is_leaf, none_is_leaf)
    spec.none_is_leaf = none_is_leaf
    return leaves, spec


def tree_flatten_with_path(tree: Any, is_leaf: Callable | None = None, *, none_is_leaf: bool = False, namespace: str = ""):
    leaves, spec = tree_flatten(tree, is_leaf, none_is_leaf=none_is_leaf)
    return spec.paths(), leaves, spec


def tree_leaves(tree: Any, is_leaf: Callable | None = None, *, none_is_leaf: bool = False, namespace: str = "") -> list:
    return tree_flatten(tree, is_leaf, none_is_leaf=none_is_leaf)[0]


def tree_structure(tree: Any, is_leaf: Callable | None = None, *, none_is_leaf: bool = False, namespace: str = "") -> PyTreeSpec:
    return tree_flatten(tree, is_leaf, none_is_leaf=none_is_leaf)[1]


def tree_unflatten(treespec: PyTreeSpec, leaves: Iterable[Any]) -> Any:
    return treespec.unflatten(leaves)


def _flatten_up_to(spec: PyTreeSpec, tree: Any, out: list) -> None:
    if spec.kind == "leaf":
        out.append(tree)
        return
    if spec.kind == "none":
        if tree is not None:
            raise ValueError("pytree structure mismatch: expected None")
        return
    if spec.kind in ("dict", "ordereddict", "defaultdict"):
        keys = spec.entries()
        if not isinstance(tree, dict) or set(tree) != set(keys):
            raise ValueError("pytree structure mismatch: dictionary keys differ")
        kids = [tree[k] for k in keys]
    else:
        if not isinstance(tree, (tuple, list, deque)) or len(tree) != len(spec.children):
            raise ValueError("pytree structure mismatch: sequence arity differs")
        kids = list(tree)
    for c, k in zip(spec.children, kids):
        _flatten_up_to(c, k, out)


def tree_map(func: Callable, tree: Any, *rests: Any, is_leaf: Callable | None = None, none_is_leaf: bool = False,
             namespace: str = "") -> Any:
    leaves, spec = tree_flatten(tree, is_leaf, none_is_leaf=none_is_leaf)
    cols = [leaves]
    for r in rests:
        flat: list = []
        _flatten_up_to(spec, r, flat)
        cols.append(flat)
    return spec.unflatten(func(*xs) for xs in zip(*cols))


def tree_map_(func: Callable, tree: Any, *rests: Any, **kw: Any) -> Any:
    tree_map(func, tree, *rests, **kw)
    return tree


def treespec_is_leaf(spec: PyTreeSpec) -> bool:
    return spec.is_leaf()


__all__ = ["PyTreeSpec", "tree_flatten", "tree_flatten_with_path", "tree_leaves", "tree_structure", "tree_unflatten",
           "tree_map", "tree_map_", "treespec_is_leaf"]
