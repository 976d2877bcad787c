"""Data-parallel plumbing on ``torch.distributed`` (NCCL between GPUs, gloo between CPU ranks).

Public surface of packages/opake-engine/src/opake/api/engine/distributed/ (collectives.py:17-130, gradients.py:47-257,
_state.py:40-613, _shard.py:20-59). Differences that matter on NVSwitch machines: gradient pytrees are reduced as ONE
flat bucket per dtype instead of one collective per leaf (launch latency, not link count, bounds small collectives),
and metadata equality checks ride on a single fingerprint reduction. The sharded engine
(:mod:`opake_b200.parallel.engine`) does not use these collectives at all for gradients — it reduces inside its fused
step kernel — so this module serves the functional API and the control plane.
"""
from __future__ import annotations

import math
from collections.abc import Callable, Mapping, Sized
from dataclasses import fields, is_dataclass, replace
from typing import Any

import torch
import torch.distributed as dist
from torch.utils.data import Subset

from ..base.exceptions import ConfigurationError, InputTypeError, OperationError
from .pytree import tree_flatten, tree_leaves, tree_map, tree_unflatten
from .types import ClippedPytree, NoisedPytree, PerGroup

_OPS = {"sum": "SUM", "mean": "AVG", "avg": "AVG", "max": "MAX", "min": "MIN", "product": "PRODUCT"}


# ------------------------------------------------------------------------------------------- collectives
def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def get_rank() -> int:
    return dist.get_rank() if is_distributed() else 0


def get_world_size() -> int:
    return dist.get_world_size() if is_distributed() else 1


def _op(op: str):
    if op not in _OPS:
        raise ConfigurationError(f"Unsupported reduction op {op!r}; expected one of {sorted(_OPS)}")
    return getattr(dist.ReduceOp, _OPS[op])


def all_reduce_(tensor: torch.Tensor, op: str = "sum") -> None:
    red = _op(op)
    if not is_distributed():
        return
    if op in ("mean", "avg") and dist.get_backend() == "gloo":
        dist.all_reduce(tensor, dist.ReduceOp.SUM)
        tensor.div_(get_world_size())
        return
    dist.all_reduce(tensor, red)


def all_reduce(tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
    out = tensor.clone()
    all_reduce_(out, op)
    return out


def barrier() -> None:
    if is_distributed():
        dist.barrier()


def is_main_process() -> bool:
    return get_rank() == 0


num_processes = get_world_size
process_index = get_rank
wait_for_everyone = barrier


def gather_for_metrics(tensor: torch.Tensor) -> torch.Tensor:
    if not is_distributed():
        return tensor
    t = tensor.contiguous()
    if t.dim() == 0:
        t = t.unsqueeze(0)
    sizes = [torch.zeros(1, dtype=torch.int64, device=t.device) for _ in range(get_world_size())]
    dist.all_gather(sizes, torch.tensor([t.shape[0]], dtype=torch.int64, device=t.device))
    mx = int(max(s.item() for s in sizes))
    pad = torch.zeros((mx, *t.shape[1:]), dtype=t.dtype, device=t.device)
    pad[: t.shape[0]] = t
    outs = [torch.empty_like(pad) for _ in range(get_world_size())]
    dist.all_gather(outs, pad)
    return torch.cat([o[: int(s.item())] for o, s in zip(outs, sizes)], 0)


# ------------------------------------------------------------------------------------------- equality asserts
def assert_scalar_equal(value: float | int, *, name: str, device: torch.device | None = None, atol: float = 0.0) -> None:
    if not is_distributed():
        return
    t = torch.tensor([float(value), -float(value)], dtype=torch.float64, device=device)
    if t.device.type == "cuda" or dist.get_backend() != "nccl":
        dist.all_reduce(t, dist.ReduceOp.MAX)
    hi, lo = t[0].item(), -t[1].item()
    if abs(hi - lo) > atol:
        raise OperationError(f"{name} differs across ranks: min={lo}, max={hi}")


def assert_string_equal(value: str | None, *, name: str) -> None:
    if not is_distributed():
        return
    got: list = [None] * get_world_size()
    dist.all_gather_object(got, value)
    if any(g != got[0] for g in got):
        raise OperationError(f"{name} differs across ranks: {got}")


def _assert_object_equal(value: Any, *, name: str) -> None:
    if not is_distributed():
        return
    got: list = [None] * get_world_size()
    dist.all_gather_object(got, value)
    if any(g != got[0] for g in got):
        raise OperationError(f"{name} differs across ranks")


def assert_pytree_equal(pytree: Any, *, name: str, atol: float = 0.0) -> None:
    """Compare a (sum, sum of squares, min, max) fingerprint of every tensor leaf across ranks."""
    if not is_distributed():
        return
    leaves = tree_leaves(pytree)
    if not leaves:
        return
    fp = torch.stack([torch.stack([l.double().sum(), (l.double() ** 2).sum(), l.double().min(), l.double().max()])
                      for l in leaves]).flatten()
    hi, lo = fp.clone(), -fp.clone()
    dist.all_reduce(hi, dist.ReduceOp.MAX)
    dist.all_reduce(lo, dist.ReduceOp.MAX)
    if ((hi + lo).abs() > atol).any():
        raise OperationError(f"{name} differs across ranks")


def reduce_scalar(value: float | int, op: str = "sum", device: torch.device | None = None) -> float | int:
    """Reduce a Python scalar; integers stay exact (int64)."""
    _op(op)
    if not is_distributed():
        return value
    is_int = isinstance(value, int) and not isinstance(value, bool) and op not in ("mean", "avg")
    t = torch.tensor([value], dtype=torch.int64 if is_int else torch.float64, device=device)
    all_reduce_(t, op)
    return int(t.item()) if is_int else float(t.item())


def gather_pytree(pytree: Any, dim: int = 0) -> Any:
    if not is_distributed():
        return pytree
    payload = tree_map(lambda x: x.detach().cpu() if isinstance(x, torch.Tensor) else x, pytree)
    got: list = [None] * get_world_size()
    dist.all_gather_object(got, payload)
    return tree_map(lambda *xs: torch.cat([x if x.dim() else x.unsqueeze(0) for x in xs], dim)
                    if isinstance(xs[0], torch.Tensor) else xs[0], *got)


def gather_tensors(tensor: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return gather_pytree(tensor, dim)


# ------------------------------------------------------------------------------------------- gradient reduction
def _meta_after(p: ClippedPytree, op: str, world: int) -> ClippedPytree:
    noised = isinstance(p, NoisedPytree)
    if op == "sum":
        if noised and p.noise_stddev is not None:
            return replace(p, noise_stddev=math.sqrt(world) * p.noise_stddev)
        return p
    if op == "mean":
        out = replace(p, max_norm=(1.0 / world) * p.max_norm)
        if noised and p.noise_stddev is not None:
            out = replace(out, noise_stddev=(1.0 / math.sqrt(world)) * p.noise_stddev)
        return out
    raise ConfigurationError(f"Unsupported wrapper reduction op: {op}")


def _check_wrapper(p: ClippedPytree, op: str) -> None:
    if op not in ("sum", "mean"):
        raise InputTypeError(f"{type(p).__name__} distributed reduction only supports op='sum' or op='mean'. Use "
                             "`.pytree` and reconstruct with an explicit max_norm for other reductions.")
    mn = p.max_norm
    meta = (dict(mn.values), {tuple(k): v for k, v in mn.groups.items()}) if isinstance(mn, PerGroup) else mn
    _assert_object_equal((type(p).__name__, meta), name="ClippedPytree metadata")


def _bucketed_all_reduce_(leaves: list[torch.Tensor], op: str) -> None:
    by = {}
    for l in leaves:
        by.setdefault((l.dtype, l.device), []).append(l)
    for group in by.values():
        if len(group) == 1 and group[0].is_contiguous():
            all_reduce_(group[0], op)
            continue
        flat = torch.cat([g.reshape(-1) for g in group])
        all_reduce_(flat, op)
        off = 0
        for g in group:
            g.copy_(flat[off : off + g.numel()].view_as(g))
            off += g.numel()


def reduce_pytree_(pytree: Any, op: str = "sum") -> None:
    """In-place reduction of tensor leaves. Wrappers whose metadata would change must use :func:`reduce_pytree`."""
    _op(op)
    if isinstance(pytree, ClippedPytree):
        _check_wrapper(pytree, op)
        world = get_world_size()
        if world > 1 and (op == "mean" or (isinstance(pytree, NoisedPytree) and pytree.noise_stddev is not None)):
            raise InputTypeError("in-place reduction would change the wrapper's public metadata; use reduce_pytree()")
        target = pytree.pytree
    else:
        target = pytree
    if is_distributed():
        _bucketed_all_reduce_(tree_leaves(target), op)


def reduce_pytree(pytree: Any, op: str = "sum") -> Any:
    _op(op)
    clone = (lambda x: x.clone() if isinstance(x, torch.Tensor) else x)
    if isinstance(pytree, ClippedPytree):
        _check_wrapper(pytree, op)
        out = replace(pytree, pytree=tree_map(clone, pytree.pytree))
        if is_distributed():
            _bucketed_all_reduce_(tree_leaves(out.pytree), op)
        return _meta_after(out, op, get_world_size())
    out = tree_map(clone, pytree)
    if is_distributed():
        _bucketed_all_reduce_(tree_leaves(out), op)
    return out


def sum_gradients_(gradients: Any) -> None:
    reduce_pytree_(gradients, "sum")


def sum_gradients(gradients: Any) -> Any:
    return reduce_pytree(gradients, "sum")


# ------------------------------------------------------------------------------------------- state sync
_FIELD_OPS = {"sum", "mean", "max", "min", "product", "assert_equal", "assert_optional_equal", "local"}
_SYNC_TYPES: dict[type, Callable[[Any], Any]] = {}


def sync_object(state: Any, field_ops: Mapping[str, Any], device: torch.device | None = None) -> Any:
    """Reduce scalar fields of a dataclass across ranks (schema validated before any collective is issued)."""
    if not is_dataclass(state):
        raise InputTypeError(f"state must be a dataclass, got {type(state)}")
    names = [f.name for f in fields(state)]
    unknown, missing = set(field_ops) - set(names), set(names) - set(field_ops)
    if unknown or missing:
        parts = ([f"unknown fields: {sorted(unknown)}"] if unknown else []) + \
                ([f"missing fields: {sorted(missing)}"] if missing else [])
        raise ConfigurationError("field_ops must define every dataclass field; " + "; ".join(parts) + ".")
    for n in names:
        op = field_ops[n]
        if not (callable(op) or op in _FIELD_OPS):
            raise ConfigurationError(f"field {n!r}: unknown op {op!r}")
    if not is_distributed():
        return state
    updates = {}
    for n in names:
        op, v = field_ops[n], getattr(state, n)
        if callable(op):
            r = op(v, device)
            if r is not None:
                updates[n] = r
        elif op == "local":
            continue
        elif op == "assert_equal":
            assert_string_equal(repr(v), name=n) if not isinstance(v, (int, float)) else assert_scalar_equal(v, name=n, device=device)
        elif op == "assert_optional_equal":
            assert_string_equal(repr(v), name=n)
        else:
            updates[n] = reduce_scalar(v, op, device)
    return replace(state, **updates)


def register_sync_type(state_type: type, sync_fn: Callable[[Any], Any]) -> None:
    _SYNC_TYPES[state_type] = sync_fn


def sync(*states: Any) -> Any:
    """Synchronise state objects with the function registered for their type (identity when none / single rank)."""

    def one(s):
        for klass in type(s).__mro__:
            fn = _SYNC_TYPES.get(klass)
            if fn is not None:
                return fn(s)
        return s

    out = tuple(one(s) for s in states)
    return out[0] if len(out) == 1 else out


# ------------------------------------------------------------------------------------------- dataset shard
def local_shard_bounds(n: int, *, rank: int = 0, world_size: int = 1) -> tuple[int, int]:
    if n < 0:
        raise ConfigurationError(f"dataset_size must be >= 0, got {n}")
    if world_size < 1:
        raise ConfigurationError(f"world_size must be >= 1, got {world_size}")
    if not 0 <= rank < world_size:
        raise ConfigurationError(f"rank must be in [0, world_size), got rank={rank}, world_size={world_size}")
    if world_size == 1:
        return 0, n
    per = n // world_size
    return rank * per, (n if rank == world_size - 1 else (rank + 1) * per)


def local_shard(dataset: Sized, *, rank: int = 0, world_size: int = 1) -> Subset:
    """Contiguous shard of ``dataset`` for ``rank``; the remainder goes to the last rank."""
    lo, hi = local_shard_bounds(len(dataset), rank=rank, world_size=world_size)
    return Subset(dataset, range(lo, hi))


__all__ = ["all_reduce", "all_reduce_", "barrier", "gather_for_metrics", "get_rank", "get_world_size", "is_distributed",
           "is_main_process", "local_shard", "num_processes", "process_index", "reduce_pytree", "reduce_pytree_",
           "sum_gradients", "sum_gradients_", "sync", "sync_object", "register_sync_type", "wait_for_everyone",
           "assert_scalar_equal", "assert_string_equal", "assert_pytree_equal", "reduce_scalar", "gather_pytree",
           "gather_tensors", "local_shard_bounds"]
